// Tensor-core GEMV over tile-major repacked GGUF weights (decode rows).
//
// Why tensor cores for a GEMV: at B200's HBM rate one SM receives ~41 Q4_K
// weights per clock, which leaves ~3 issue slots per weight across its 128
// lanes -- and integer/logic instructions issue at half rate.  A SIMT decode
// (extract, int->float, FMA) needs far more than that, so the dot products run
// on the integer tensor-core path, `mma.sync.m16n8k32.s32.u8.s8`, where a
// quantised weight needs no conversion at all: four packed nibbles become four
// u8 operands with one AND (a Q8_0 byte is an operand as stored), products and
// sums are exact in int32, and one F32 scale per 32 (Q4_K, Q8_0) or 16 (Q6_K)
// inputs folds the block's scale and the activation span's scale into the
// accumulator.  The formats' offsets (Q4_K minimum, Q6_K -32, Q8_0 -128) are
// removed through per-16-input sums of the activations.  Activations arrive as
// three signed 8-bit digits per input (see ActOperand), produced by the
// previous kernel's epilogue.
//
// Execution: one persistent CTA per SM.  A producer warp streams the CTA's
// contiguous byte range of weight tiles into a shared-memory ring with bulk
// (TMA) copies completing on mbarriers; it starts before the programmatic
// dependency on the previous kernel resolves, so weights are already in
// flight while that kernel drains.  Twenty-four consumer warps in three teams
// take the ring stages in turn (or, for launches with many units per CTA such
// as the output head, each team owns whole units); each warp owns one
// 16 x 256 tile of a stage.  Per unit of 32 output rows the warps leave their
// partial sums in shared memory and move on; a dedicated epilogue warp adds
// them in a fixed order (deterministic results) and applies the epilogue:
// store, residual add, SwiGLU, and the operand form of the result for the
// next projection.  Scale folds and header decodes use the packed FP32 pair
// instructions of sm_100 (two IEEE operations per issue slot).
// Every wait is bounded: on expiry the kernel raises an error flag and runs
// to completion without waiting again.
#include <cuda_fp16.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "blocks.cuh"
#include "gemv.cuh"
#include "operand.cuh"

namespace ribn {

// ---------------------------------------------------------------------------
// host repack
// ---------------------------------------------------------------------------
namespace {

// four consecutive inputs of one row: one 32-bit A-fragment register of the integer MMA
inline void put4(unsigned char* dst, const unsigned char* src, unsigned char flip) {
    dst[0] = src[0] ^ flip; dst[1] = src[1] ^ flip; dst[2] = src[2] ^ flip; dst[3] = src[3] ^ flip;
}

void repack_tile(int type, const unsigned char* raw, long long n, long long k_blocks_per_row, int rt, int kb,
                 unsigned char* tile) {
    static const unsigned char zeros[256] = {0};
    for (int lane = 0; lane < 32; ++lane) {
        const int g = lane >> 2, t = lane & 3;
        for (int rs = 0; rs < 2; ++rs) {
            const long long row = (long long)rt * kTileRows + g + rs * 8;
            const bool live = row < n;
            if (type == kQ4_K) {
                const unsigned char* blk = live ? raw + (row * k_blocks_per_row + kb) * 144 : zeros;
                for (int j = 0; j < 4; ++j) {
                    for (int h = 0; h < 2; ++h) {
                        const unsigned char* src = blk + 16 + j * 32 + 16 * h + 4 * t;
                        put4(tile + j * 512 + lane * 16 + (rs * 2 + h) * 4, live ? src : zeros, 0);
                    }
                }
            } else if (type == kQ6_K) {
                const unsigned char* blk = live ? raw + (row * k_blocks_per_row + kb) * 210 : zeros;
                for (int c = 0; c < 2; ++c) {
                    for (int h = 0; h < 2; ++h) {
                        const int l0 = 16 * h + 4 * t;
                        unsigned char* ql = tile + (c * 2 + h) * 512 + lane * 16 + rs * 8;
                        put4(ql, blk + c * 64 + l0, 0);
                        put4(ql + 4, blk + c * 64 + 32 + l0, 0);
                        put4(tile + 2048 + c * 512 + lane * 16 + (h * 2 + rs) * 4, blk + 128 + c * 32 + l0, 0);
                    }
                }
            } else {  // Q8_0: eight 34-byte blocks per 256 inputs, stored as q + 128
                for (int b = 0; b < 8; ++b) {
                    const unsigned char* blk = live ? raw + (row * k_blocks_per_row + kb * 8 + b) * 34 : nullptr;
                    for (int h = 0; h < 2; ++h) {
                        unsigned char* dst = tile + b * 512 + lane * 16 + (rs * 2 + h) * 4;
                        if (live) put4(dst, blk + 2 + 16 * h + 4 * t, 0x80);
                        else memset(dst, 0x80, 4);
                    }
                }
            }
        }
    }
    for (int r = 0; r < kTileRows; ++r) {
        const long long row = (long long)rt * kTileRows + r;
        const bool live = row < n;
        if (type == kQ4_K) {
            const unsigned char* blk = raw + (row * k_blocks_per_row + kb) * 144;
            if (live) memcpy(tile + 2048 + r * 16, blk, 16); else memset(tile + 2048 + r * 16, 0, 16);
        } else if (type == kQ6_K) {
            const unsigned char* blk = raw + (row * k_blocks_per_row + kb) * 210;
            if (live) {
                memcpy(tile + 3072 + r * 16, blk + 192, 16);
                memcpy(tile + 3328 + r * 2, blk + 208, 2);
            } else {
                memset(tile + 3072 + r * 16, 0, 16);
                memset(tile + 3328 + r * 2, 0, 2);
            }
        } else {
            for (int b = 0; b < 8; ++b) {
                const unsigned char* blk = raw + (row * k_blocks_per_row + kb * 8 + b) * 34;
                if (live) memcpy(tile + 4096 + r * 16 + b * 2, blk, 2); else memset(tile + 4096 + r * 16 + b * 2, 0, 2);
            }
        }
    }
}

}  // namespace

void repack_host(int type, const unsigned char* raw, long long n, long long k, unsigned char* out, int threads) {
    const int row_tiles = (int)((n + kTileRows - 1) / kTileRows);
    const int k_tiles = (int)(k / kTileCols);
    const long long blocks_per_row = k / block_elems(type);
    const size_t tile_bytes = (size_t)packed_tile_bytes(type);
    auto work = [&](int begin, int end) {
        for (int rt = begin; rt < end; ++rt) {
            for (int kb = 0; kb < k_tiles; ++kb) {
                repack_tile(type, raw, n, blocks_per_row, rt, kb, out + ((size_t)rt * k_tiles + kb) * tile_bytes);
            }
        }
    };
    threads = std::max(1, std::min(threads, row_tiles));
    if (threads == 1) { work(0, row_tiles); return; }
    std::vector<std::thread> pool;
    const int per = (row_tiles + threads - 1) / threads;
    for (int i = 0; i < threads; ++i) {
        const int b = i * per, e = std::min(row_tiles, b + per);
        if (b < e) pool.emplace_back(work, b, e);
    }
    for (auto& th : pool) th.join();
}

// ---------------------------------------------------------------------------
// device
// ---------------------------------------------------------------------------
namespace {

constexpr int kConsumerWarps = 24;  // three teams of eight; team i consumes stages i, i + 3, ...
constexpr int kTeamWarps = 8;
constexpr int kTeams = kConsumerWarps / kTeamWarps;
constexpr int kStageTiles = 8;      // tiles per bulk copy / ring slot (one per warp of a team)
constexpr int kProducerWarp = kConsumerWarps;
constexpr int kEpilogueWarp = kConsumerWarps + 1;  // first of kEpilogueWarps: one per team
constexpr int kEpilogueWarps = kTeams;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = (kConsumerWarps + 1 + kEpilogueWarps) * 32;
constexpr int kMaxRuns = 4;         // row-tile runs per unit: 2 tiles of one matrix, or 2 x (gate, up)
constexpr int kHdrStride = 20;      // floats per header row: 16 scales + offset sum + pad (conflict-free rows)
constexpr int kPlanePad = 32;       // bytes between activation digit planes (distinct banks per plane)
constexpr uint32_t kSpinLimit = 1u << 22;  // bounded waits: default number of polls before giving up
constexpr uint32_t kNibbles = 0x0F0F0F0Fu;
constexpr uint32_t kHighNibbles = 0xF0F0F0F0u;
constexpr uint32_t kTopBits = 0x30303030u;
constexpr int kMagicInt = 0x4B400000;      // bits of 12582912.0f: int accumulate on top of it, read as float
constexpr float kMagic = 12582912.0f;
constexpr int kBarFull = 1, kBarFree = 3;  // named barriers of team t, buffer b: full = 1 + 4 t + b, free = 3 + 4 t + b

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the error flag) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (error_flag != nullptr) atomicExch(error_flag, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Named barriers shared by the warps that cooperate on a unit and their epilogue warp.
__device__ __forceinline__ void bar_arrive(int id, int threads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D = A(u8, 16 x 32) * B(s8, 32 x 8) + magic; the result registers are read as floats.
__device__ __forceinline__ void imma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(kMagicInt));
}
__device__ __forceinline__ void imma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(kMagicInt));
}
// (a & mask) | other in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t other) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(other));
    return r;
}
// bytes i and i + 1 of w as floats minus `bias` (both exact), as one packed subtraction
__device__ __forceinline__ float2 bytes_f32x2(uint32_t w, int i, float bias) {
    const float2 raw = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (uint32_t)i)),
                                   __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (uint32_t)(i + 1))));
    return __fadd2_rn(raw, make_float2(-bias, -bias));
}

// Shared-memory accesses by 32-bit shared-space address: the hot loop then needs one add per access
// instead of generic 64-bit pointer arithmetic.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds32f(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint32_t v;
    asm volatile("{\n\t.reg .u16 t;\n\tld.shared.u16 t, [%1];\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128f(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t addr, float a) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}

// Shared-memory map of the CTA (generic pointers for set-up and the epilogue warps).
struct Shared {
    unsigned char* ring;
    signed char* xq;   // [3 * members][K + kPlanePad] digit planes
    float* sx;         // [members][K / 32]
    float* sxs;        // [members][K / 16]
    float* hdr;        // [kConsumerWarps][members][16][kHdrStride]
    float* red;        // [kTeams][2][kTeamWarps][kMaxRuns][members][16]
    float* scale;      // [kGemvMaxMembers]
    uint32_t full, empty, xbar;  // shared-space addresses of the mbarrier arrays
    int K, members;
};

// Per-lane shared-space addresses of a consumer warp, fixed for the whole kernel.
struct Lane {
    uint32_t b;        // this lane's MMA column in the digit planes (+ 8 t), or a zeroed word
    uint32_t b_mask;   // all ones for a live column, zero for the empty columns (they read the zeroed word)
    uint32_t sx, sxs;  // scale arrays
    uint32_t hdr_wr;   // decode role: header row (lane >> 1) of member 0
    uint32_t hdr_rd;   // fold role: header row g of this lane's member (row g + 8 is 8 rows further)
    int members, K;
    int half;          // decode role: which half of the row's scales
};

constexpr uint32_t kHdrRow = kHdrStride * 4;        // bytes per header row
constexpr uint32_t kHdrMember = 16 * kHdrRow;       // bytes per member's header block
constexpr uint32_t kHdrOff = 64;                    // byte offset of the row's offset sum

struct Accum {
    float c[4];  // (row g, col 2t), (row g, col 2t+1), (row g+8, col 2t), (row g+8, col 2t+1)
    float s[2];  // offset terms of rows g, g+8
};

// Packed FP32 pairs (sm_100): each component is the same IEEE operation as the scalar form, so the
// results do not change; the pair form halves the instructions issued for the fold.
__device__ __forceinline__ void fold(Accum& a, const int (&c)[4], float s0, float s1) {
    const float2 minus = make_float2(-kMagic, -kMagic);
    const float2 lo = __fadd2_rn(make_float2(__int_as_float(c[0]), __int_as_float(c[1])), minus);
    const float2 hi = __fadd2_rn(make_float2(__int_as_float(c[2]), __int_as_float(c[3])), minus);
    const float2 r0 = __ffma2_rn(make_float2(s0, s0), lo, make_float2(a.c[0], a.c[1]));
    const float2 r1 = __ffma2_rn(make_float2(s1, s1), hi, make_float2(a.c[2], a.c[3]));
    a.c[0] = r0.x; a.c[1] = r0.y; a.c[2] = r1.x; a.c[3] = r1.y;
}

__device__ __forceinline__ uint2 load_b(const Lane& ln, uint32_t offset) {
    return lds64(ln.b + (offset & ln.b_mask));
}

// ---- Q4_K: w = gs * q - gm  =>  (gs * sx) * C  -  gm * (sx * sum digits) ------------------------
template <int MEMBERS>
__device__ __forceinline__ void tile_q4k(uint32_t tile, const Lane& ln, int kb, int lane, Accum& acc) {
    {
        // lane -> (row, half): scales and offsets of groups 4 half .. 4 half + 3, for every member
        const uint4 h = lds128(tile + 2048 + (lane >> 1) * 16);
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        const uint32_t sc = ln.half ? ((h.w & kNibbles) | ((h.y >> 2) & kTopBits)) : (h.y & 0x3F3F3F3Fu);
        const uint32_t mn = ln.half ? (((h.w >> 4) & kNibbles) | ((h.z >> 2) & kTopBits)) : (h.z & 0x3F3F3F3Fu);
        // Odd groups reach the MMA as 16 q (their nibbles stay in the high half of each byte), so their
        // scale carries the exact factor 1/16.
        // pair form of the same operations (packed FP32, sm_100): components 0 / 1 and 2 / 3
        const float2 dd = make_float2(d, d * 0.0625f), mm2 = make_float2(dmin, dmin);
        const float2 gs01 = __fmul2_rn(dd, bytes_f32x2(sc, 0, 8388608.0f)), gs23 = __fmul2_rn(dd, bytes_f32x2(sc, 2, 8388608.0f));
        const float2 gm01 = __fmul2_rn(mm2, bytes_f32x2(mn, 0, 8388608.0f)), gm23 = __fmul2_rn(mm2, bytes_f32x2(mn, 2, 8388608.0f));
#pragma unroll
        for (int mm = 0; mm < MEMBERS; ++mm) {
            const float4 sx = lds128f(ln.sx + (uint32_t)(mm * (ln.K / 32) + kb * 8 + ln.half * 4) * 4);
            const uint32_t sxs = ln.sxs + (uint32_t)(mm * (ln.K / 16) + kb * 16 + ln.half * 8) * 4;
            const float4 sa = lds128f(sxs), sb = lds128f(sxs + 16);
            const uint32_t out = ln.hdr_wr + mm * kHdrMember;
            const float2 h01 = __fmul2_rn(gs01, make_float2(sx.x, sx.y)), h23 = __fmul2_rn(gs23, make_float2(sx.z, sx.w));
            sts128f(out + ln.half * 16, h01.x, h01.y, h23.x, h23.y);
            const float2 ta = __fadd2_rn(make_float2(sa.x, sa.z), make_float2(sa.y, sa.w));
            const float2 tb = __fadd2_rn(make_float2(sb.x, sb.z), make_float2(sb.y, sb.w));
            float off = gm01.x * ta.x;
            off = fmaf(gm01.y, ta.y, off);
            off = fmaf(gm23.x, tb.x, off);
            off = fmaf(gm23.y, tb.y, off);
            off += __shfl_xor_sync(0xffffffffu, off, 1);
            if (ln.half == 0) sts32f(out + kHdrOff, -off);
        }
    }
    __syncwarp();
    const uint32_t wbase = tile + lane * 16, bbase = kb * 256;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 w = lds128(wbase + j * 512);
        const uint2 be = load_b(ln, bbase + j * 64), bo = load_b(ln, bbase + j * 64 + 32);
        const float2 f0 = lds64f(ln.hdr_rd + j * 8), f1 = lds64f(ln.hdr_rd + 8 * kHdrRow + j * 8);
        int ce[4], co[4];
        imma_k32(ce, w.x & kNibbles, w.z & kNibbles, w.y & kNibbles, w.w & kNibbles, be.x, be.y);
        imma_k32(co, w.x & kHighNibbles, w.z & kHighNibbles, w.y & kHighNibbles, w.w & kHighNibbles, bo.x, bo.y);
        fold(acc, ce, f0.x, f1.x);
        fold(acc, co, f0.y, f1.y);
    }
    acc.s[0] += lds32f(ln.hdr_rd + kHdrOff);
    acc.s[1] += lds32f(ln.hdr_rd + 8 * kHdrRow + kHdrOff);
    __syncwarp();
}

// ---- Q6_K: w = gs * (q - 32), one scale per 16 inputs (k16 MMA) ---------------------------------
template <int MEMBERS>
__device__ __forceinline__ void tile_q6k(uint32_t tile, const Lane& ln, int kb, int lane, Accum& acc) {
    {
        // lane -> (row, half): the eight 16-input scales half * 8 .. half * 8 + 7 (groups half * 4 ..)
        const int row = lane >> 1;
        const uint2 s8 = lds64(tile + 3072 + row * 16 + ln.half * 8);
        const float d = __half2float(__ushort_as_half((unsigned short)lds16(tile + 3328 + row * 2)));
        float gs[8];
        {
            // signed byte: flip the sign bit, read as unsigned on top of 2^23, subtract 2^23 + 128 (exact); pair form
            const float2 dd = make_float2(d, d);
            const uint32_t lo = s8.x ^ 0x80808080u, hi = s8.y ^ 0x80808080u;
            const float2 g01 = __fmul2_rn(dd, bytes_f32x2(lo, 0, 8388736.0f)), g23 = __fmul2_rn(dd, bytes_f32x2(lo, 2, 8388736.0f));
            const float2 g45 = __fmul2_rn(dd, bytes_f32x2(hi, 0, 8388736.0f)), g67 = __fmul2_rn(dd, bytes_f32x2(hi, 2, 8388736.0f));
            gs[0] = g01.x; gs[1] = g01.y; gs[2] = g23.x; gs[3] = g23.y;
            gs[4] = g45.x; gs[5] = g45.y; gs[6] = g67.x; gs[7] = g67.y;
        }
#pragma unroll
        for (int mm = 0; mm < MEMBERS; ++mm) {
            const float4 sx = lds128f(ln.sx + (uint32_t)(mm * (ln.K / 32) + kb * 8 + ln.half * 4) * 4);
            const uint32_t sxs = ln.sxs + (uint32_t)(mm * (ln.K / 16) + kb * 16 + ln.half * 8) * 4;
            const float4 sa = lds128f(sxs), sb = lds128f(sxs + 16);
            const uint32_t out = ln.hdr_wr + mm * kHdrMember;
            const float2 h01 = __fmul2_rn(make_float2(gs[0], gs[1]), make_float2(sx.x, sx.x));
            const float2 h23 = __fmul2_rn(make_float2(gs[2], gs[3]), make_float2(sx.y, sx.y));
            const float2 h45 = __fmul2_rn(make_float2(gs[4], gs[5]), make_float2(sx.z, sx.z));
            const float2 h67 = __fmul2_rn(make_float2(gs[6], gs[7]), make_float2(sx.w, sx.w));
            sts128f(out + ln.half * 32, h01.x, h01.y, h23.x, h23.y);
            sts128f(out + ln.half * 32 + 16, h45.x, h45.y, h67.x, h67.y);
            float off = gs[0] * sa.x;
            off = fmaf(gs[1], sa.y, off); off = fmaf(gs[2], sa.z, off); off = fmaf(gs[3], sa.w, off);
            off = fmaf(gs[4], sb.x, off); off = fmaf(gs[5], sb.y, off); off = fmaf(gs[6], sb.z, off); off = fmaf(gs[7], sb.w, off);
            off += __shfl_xor_sync(0xffffffffu, off, 1);
            if (ln.half == 0) sts32f(out + kHdrOff, -32.0f * off);
        }
    }
    __syncwarp();
    const uint32_t wbase = tile + lane * 16, bbase = kb * 256;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const uint4 qh = lds128(wbase + 2048 + c * 512);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 w = lds128(wbase + (c * 2 + h) * 512);
            const uint32_t wh0 = h == 0 ? qh.x : qh.z, wh1 = h == 0 ? qh.y : qh.w;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint32_t l0 = (v & 1) ? w.y : w.x, l1 = (v & 1) ? w.w : w.z;
                // the variant's two high bits sit at bits 2v..2v+1 of each high-bit byte: move them to bits 4..5
                uint32_t t0, t1;
                if (v == 0) { t0 = wh0 << 4; t1 = wh1 << 4; }
                else if (v == 1) { t0 = wh0 << 2; t1 = wh1 << 2; }
                else if (v == 2) { t0 = wh0; t1 = wh1; }
                else { t0 = wh0 >> 2; t1 = wh1 >> 2; }
                const uint32_t a0 = and_or(v < 2 ? l0 : l0 >> 4, kNibbles, t0 & kTopBits);
                const uint32_t a1 = and_or(v < 2 ? l1 : l1 >> 4, kNibbles, t1 & kTopBits);
                const int sub = (c * 4 + v) * 2 + h;
                const uint2 b = load_b(ln, bbase + (c * 4 + v) * 32);
                int cc[4];
                imma_k16(cc, a0, a1, h == 0 ? b.x : b.y);
                fold(acc, cc, lds32f(ln.hdr_rd + sub * 4), lds32f(ln.hdr_rd + 8 * kHdrRow + sub * 4));
            }
        }
    }
    acc.s[0] += lds32f(ln.hdr_rd + kHdrOff);
    acc.s[1] += lds32f(ln.hdr_rd + 8 * kHdrRow + kHdrOff);
    __syncwarp();
}

// ---- Q8_0: stored byte u = q + 128 is the u8 operand as is; w = d * (u - 128) -----------------------
template <int MEMBERS>
__device__ __forceinline__ void tile_q8_0(uint32_t tile, const Lane& ln, int kb, int lane, Accum& acc) {
    {
        const uint2 d4 = lds64(tile + 4096 + (lane >> 1) * 16 + ln.half * 8);
        float d[4];
        d[0] = __half2float(__ushort_as_half((unsigned short)(d4.x & 0xffffu)));
        d[1] = __half2float(__ushort_as_half((unsigned short)(d4.x >> 16)));
        d[2] = __half2float(__ushort_as_half((unsigned short)(d4.y & 0xffffu)));
        d[3] = __half2float(__ushort_as_half((unsigned short)(d4.y >> 16)));
#pragma unroll
        for (int mm = 0; mm < MEMBERS; ++mm) {
            const float4 sx = lds128f(ln.sx + (uint32_t)(mm * (ln.K / 32) + kb * 8 + ln.half * 4) * 4);
            const uint32_t sxs = ln.sxs + (uint32_t)(mm * (ln.K / 16) + kb * 16 + ln.half * 8) * 4;
            const float4 sa = lds128f(sxs), sb = lds128f(sxs + 16);
            const uint32_t out = ln.hdr_wr + mm * kHdrMember;
            sts128f(out + ln.half * 16, d[0] * sx.x, d[1] * sx.y, d[2] * sx.z, d[3] * sx.w);
            float off = d[0] * (sa.x + sa.y);
            off = fmaf(d[1], sa.z + sa.w, off);
            off = fmaf(d[2], sb.x + sb.y, off);
            off = fmaf(d[3], sb.z + sb.w, off);
            off += __shfl_xor_sync(0xffffffffu, off, 1);
            if (ln.half == 0) sts32f(out + kHdrOff, -128.0f * off);
        }
    }
    __syncwarp();
    const uint32_t wbase = tile + lane * 16, bbase = kb * 256;
#pragma unroll
    for (int b8 = 0; b8 < 8; ++b8) {
        const uint4 w = lds128(wbase + b8 * 512);
        const uint2 b = load_b(ln, bbase + b8 * 32);
        int cc[4];
        imma_k32(cc, w.x, w.z, w.y, w.w, b.x, b.y);
        fold(acc, cc, lds32f(ln.hdr_rd + b8 * 4), lds32f(ln.hdr_rd + 8 * kHdrRow + b8 * 4));
    }
    acc.s[0] += lds32f(ln.hdr_rd + kHdrOff);
    acc.s[1] += lds32f(ln.hdr_rd + 8 * kHdrRow + kHdrOff);
    __syncwarp();
}

// Where a unit's rows live: segment index and first row tile.
struct UnitPlace { int seg, rt0; };

__device__ __forceinline__ UnitPlace place_unit(const GemvArgs& a, bool swiglu, int u) {
    UnitPlace p{0, 2 * u};
    if (!swiglu) {
        while (p.seg + 1 < a.n_segments && p.rt0 >= ((a.seg[p.seg].row_tiles + 1) & ~1)) {
            p.rt0 -= (a.seg[p.seg].row_tiles + 1) & ~1;
            ++p.seg;
        }
    }
    return p;
}

// A team's position in its own sequence of ring stages: unit, run within the unit, stage within the run.
struct Cursor {
    int u, r, st;
};

// SHARED = false: each team of eight warps owns whole units (many units per CTA: the output head).
// SHARED = true: all 24 warps cooperate on every unit, the teams taking alternate stages (the layer
// projections, which give a CTA only one to three units).
template <int MEMBERS, bool SHARED>
__global__ void __launch_bounds__(kThreads, 1) gemv_mma_kernel(const GemvArgs a, const int slots_per_team,
                                                               const int slot_bytes) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int K = a.k, planes = 3 * MEMBERS, slots = slots_per_team * kTeams;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t spin_limit = a.spin_limit ? a.spin_limit : kSpinLimit;
    const bool swiglu = a.epilogue == kSwiGLU;
    const int runs = swiglu ? 4 : 2;  // row-tile runs per unit
    Shared sh;
    {
        unsigned char* p = smem_raw;
        sh.ring = p; p += (size_t)slots * slot_bytes;
        sh.xq = reinterpret_cast<signed char*>(p); p += (size_t)planes * (K + kPlanePad);
        sh.sx = reinterpret_cast<float*>(p); p += (size_t)MEMBERS * (K / 32) * sizeof(float);
        sh.sxs = reinterpret_cast<float*>(p); p += (size_t)MEMBERS * (K / 16) * sizeof(float);
        sh.hdr = reinterpret_cast<float*>(p); p += (size_t)kConsumerWarps * MEMBERS * 16 * kHdrStride * sizeof(float);
        sh.red = reinterpret_cast<float*>(p); p += (size_t)2 * kConsumerWarps * kMaxRuns * MEMBERS * 16 * sizeof(float);
        sh.scale = reinterpret_cast<float*>(p); p += 16;  // the zeroed word read by the empty MMA columns
        sh.full = smem_u32(p); p += (size_t)slots * 8;
        sh.empty = smem_u32(p); p += (size_t)slots * 8;
        sh.xbar = smem_u32(p);
        sh.K = K; sh.members = MEMBERS;
    }
    const int k_tiles = K / kTileCols;
    const int stages_per_run = (k_tiles + kStageTiles - 1) / kStageTiles;
    int total_units = 0;
    if (swiglu) total_units = (a.seg[0].row_tiles + 1) / 2;
    else for (int i = 0; i < a.n_segments; ++i) total_units += (a.seg[i].row_tiles + 1) / 2;
    const int u0 = (int)((long long)blockIdx.x * total_units / gridDim.x);
    const int u1 = (int)((long long)(blockIdx.x + 1) * total_units / gridDim.x);

    if (threadIdx.x == 0) {
        for (int i = 0; i < slots; ++i) { mbar_init(sh.full + i * 8, 1); mbar_init(sh.empty + i * 8, kTeamWarps); }
        mbar_init(sh.xbar, 1);
        sh.scale[0] = sh.scale[1] = sh.scale[2] = sh.scale[3] = 0.0f;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream begin (its weight prefetch does not depend on this one).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Where run r of unit u lives; false when the unit has no such run (odd tail of a segment).
    auto locate = [&](int u, int r, const GemvSegment*& seg, int& rt) -> bool {
        const UnitPlace pl = place_unit(a, swiglu, u);
        seg = &a.seg[swiglu ? (r & 1) : pl.seg];
        rt = pl.rt0 + (swiglu ? (r >> 1) : r);
        return rt < seg->row_tiles;
    };

    if (warp == kProducerWarp) {
        // ---------------- producer: team t's k-th stage goes to slot (k % S) * 3 + t ----------------
        if (lane == 0) {
            constexpr int kCursors = SHARED ? 1 : kTeams;
            const int unit_step = SHARED ? 1 : kTeams;
            const uint32_t ring_len = SHARED ? (uint32_t)slots : (uint32_t)slots_per_team;  // slots a cursor cycles through
            Cursor cur[kCursors];
            uint32_t k[kCursors];
            for (int t = 0; t < kCursors; ++t) { cur[t] = Cursor{u0 + t, 0, 0}; k[t] = 0; }
            bool alive = true, any = true;
            while (any && alive) {
                any = false;
                for (int t = 0; t < kCursors && alive; ++t) {
                    Cursor& c = cur[t];
                    const GemvSegment* seg = nullptr;
                    int rt = 0;
                    while (c.u < u1 && !locate(c.u, c.r, seg, rt)) {  // skip runs the unit does not have
                        if (++c.r == runs) { c.r = 0; c.u += unit_step; }
                    }
                    if (c.u >= u1) continue;
                    any = true;
                    const uint32_t tile_bytes = (uint32_t)packed_tile_bytes(seg->type);
                    const uint32_t slot = SHARED ? k[t] % ring_len : (k[t] % ring_len) * kTeams + t;
                    if (k[t] >= ring_len) {
                        alive = mbar_wait(sh.empty + slot * 8, ((k[t] / ring_len) - 1u) & 1u, a.error_flag, 1, spin_limit);
                        if (!alive) break;
                    }
                    const int tiles = min(kStageTiles, k_tiles - c.st * kStageTiles);
                    const uint32_t bytes = (uint32_t)tiles * tile_bytes;
                    mbar_expect_tx(sh.full + slot * 8, bytes);
                    bulk_g2s(smem_u32(sh.ring + (size_t)slot * slot_bytes),
                             seg->data + ((size_t)rt * k_tiles + (size_t)c.st * kStageTiles) * tile_bytes, bytes,
                             sh.full + slot * 8);
                    ++k[t];
                    if (++c.st == stages_per_run) {
                        c.st = 0;
                        if (++c.r == runs) { c.r = 0; c.u += unit_step; }
                    }
                }
            }
        }
        return;
    }

    asm volatile("griddepcontrol.wait;" ::: "memory");  // activations and the residual come from the previous kernel

    if (warp > kEpilogueWarp && SHARED) return;  // one epilogue warp serves the single cooperating set
    // cooperating set: its warps, barrier participants, and where its partial sums live
    constexpr int kSetWarps = SHARED ? kConsumerWarps : kTeamWarps;
    const int bar_threads = kSetWarps * 32 + 32;
    const int unit_step = SHARED ? 1 : kTeams;
    if (warp >= kEpilogueWarp) {
        // ---------------- epilogue warp: lane = one of the unit's 32 output rows ----------------
        const int team = SHARED ? 0 : warp - kEpilogueWarp;
        float inv_norm[MEMBERS];
#pragma unroll
        for (int m = 0; m < MEMBERS; ++m) {
            // RMSNorm factor: fixed-order sum of the producer's per-32 sums of squares.
            inv_norm[m] = 1.0f;
            if (a.in_has_norm) {
                const float* ss = a.in.ss32 + (size_t)m * (K / 32);
                float sum = 0.0f;
                // four loads in flight per trip (the additions keep their order)
                for (int i0 = lane; i0 < K / 32; i0 += 128) {
                    float part[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) part[u] = i0 + 32 * u < K / 32 ? ss[i0 + 32 * u] : 0.0f;
#pragma unroll
                    for (int u = 0; u < 4; ++u) sum += part[u];
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                inv_norm[m] = 1.0f / sqrtf(sum / (float)K + a.eps);
            }
        }
        int buf = 0;
        for (int u = u0 + team; u < u1; u += unit_step, buf ^= 1) {
            const UnitPlace pl = place_unit(a, swiglu, u);
            const GemvSegment& s = a.seg[swiglu ? 0 : pl.seg];
            const int half = lane >> 4, row = lane & 15;
            const int rt = pl.rt0 + half;
            const int n_index = rt * kTileRows + row;
            const bool valid = rt < s.row_tiles && n_index < s.n;
            // Fetch what does not depend on the consumers before waiting for them.
            float prior[MEMBERS];
#pragma unroll
            for (int m = 0; m < MEMBERS; ++m) {
                prior[m] = (valid && a.epilogue == kResidual) ? s.y[(size_t)m * s.n + n_index] : 0.0f;
            }
            const float norm_w = (valid && a.out.dig != nullptr && a.out_norm_weight != nullptr) ? a.out_norm_weight[n_index] : 1.0f;
            bar_sync(kBarFull + team * 4 + buf, bar_threads);  // the set's warps have left their partial sums of this unit
            float v0[MEMBERS], v1[MEMBERS];
            const float* base = sh.red + (size_t)(team * 2 + buf) * kSetWarps * kMaxRuns * MEMBERS * 16;
            const int run0 = swiglu ? 2 * half : half;
#pragma unroll
            for (int m = 0; m < MEMBERS; ++m) {
                float x0 = 0.0f, x1 = 0.0f;
#pragma unroll 8
                for (int w = 0; w < kSetWarps; ++w) {
                    x0 += base[(((size_t)w * kMaxRuns + run0) * MEMBERS + m) * 16 + row];
                    if (swiglu) x1 += base[(((size_t)w * kMaxRuns + run0 + 1) * MEMBERS + m) * 16 + row];
                }
                v0[m] = x0 * inv_norm[m];
                v1[m] = x1 * inv_norm[m];
            }
            __syncwarp();
            bar_arrive(kBarFree + team * 4 + buf, bar_threads);  // the buffer may be overwritten
#pragma unroll
            for (int m = 0; m < MEMBERS; ++m) {
                float result = 0.0f, square = 0.0f;
                if (valid) {
                    if (a.epilogue == kResidual) {
                        result = prior[m] + v0[m];
                        s.y[(size_t)m * s.n + n_index] = result;
                        square = result * result;
                    } else if (swiglu) {
                        result = v0[m] / (1.0f + expf(-v0[m])) * v1[m];
                        if (a.swiglu_f32 != nullptr) a.swiglu_f32[(size_t)m * s.n + n_index] = result;
                    } else {
                        result = v0[m];
                        s.y[(size_t)m * s.n + n_index] = result;
                    }
                }
                if (a.out.dig != nullptr && pl.rt0 * kTileRows < s.n) {
                    ActOperand out = a.out;
                    if (a.epilogue != kResidual) out.ss32 = nullptr;
                    operand_store_span(out, m, s.n, pl.rt0 / 2, lane, result * norm_w, square);
                }
            }
        }
        return;
    }

    // ---------------- consumers: a team of eight warps owns whole units; each warp takes one tile per stage ----------------
    if (warp == 0) {
        // One copy per lane: digit planes, then the two scale arrays.
        const uint32_t plane_bytes = (uint32_t)K, sx_bytes = (uint32_t)MEMBERS * (K / 32) * 4u,
                       sxs_bytes = (uint32_t)MEMBERS * (K / 16) * 4u;
        if (lane == 0) mbar_expect_tx(sh.xbar, plane_bytes * (uint32_t)planes + sx_bytes + sxs_bytes);
        __syncwarp();
        if (lane < planes) {
            bulk_g2s(smem_u32(sh.xq + (size_t)lane * (K + kPlanePad)), a.in.dig + (size_t)lane * K, plane_bytes, sh.xbar);
        } else if (lane == planes) {
            bulk_g2s(smem_u32(sh.sx), a.in.sx, sx_bytes, sh.xbar);
        } else if (lane == planes + 1) {
            bulk_g2s(smem_u32(sh.sxs), a.in.sxs16, sxs_bytes, sh.xbar);
        }
    }
    bool alive = mbar_wait(sh.xbar, 0, a.error_flag, 2, spin_limit);

    const int g = lane >> 2, t = lane & 3;
    const int team = warp / kTeamWarps, member_warp = warp % kTeamWarps;
    Lane ln;
    {
        const uint32_t hdr = smem_u32(sh.hdr) + (uint32_t)warp * MEMBERS * kHdrMember;
        const bool live = (g & 3) < 3 && (g >> 2) < MEMBERS;
        ln.b_mask = live ? 0xffffffffu : 0u;
        ln.b = live ? smem_u32(sh.xq) + (uint32_t)((g >> 2) * 3 + (g & 3)) * (uint32_t)(K + kPlanePad) + 8 * t
                    : smem_u32(sh.scale);
        ln.sx = smem_u32(sh.sx);
        ln.sxs = smem_u32(sh.sxs);
        ln.hdr_wr = hdr + (lane >> 1) * kHdrRow;
        // lanes whose columns belong to no member (t >= 2 with one member) read member 0's rows: the same
        // addresses as their neighbours (a broadcast) instead of another block in the same banks
        ln.hdr_rd = hdr + (uint32_t)min(t >> 1, MEMBERS - 1) * kHdrMember + g * kHdrRow;
        ln.members = MEMBERS;
        ln.K = K;
        ln.half = lane & 1;
    }
    const uint32_t ring = smem_u32(sh.ring);
    const int set = SHARED ? 0 : team, set_warp = SHARED ? warp : member_warp;
    const uint32_t ring_len = SHARED ? (uint32_t)slots : (uint32_t)slots_per_team;
    // The set's stage counter k, in step with the producer's, kept as (k % ring_len, (k / ring_len) & 1, k % kTeams)
    // and advanced incrementally: no divisions in the stage loop.
    uint32_t ring_pos = 0, ring_parity = 0;
    int turn = 0;
    int buf = 0, done = 0;
    for (int u = u0 + set; u < u1; u += unit_step, buf ^= 1, ++done) {
        Accum acc[kMaxRuns];
#pragma unroll
        for (int r = 0; r < kMaxRuns; ++r) {
            acc[r].c[0] = acc[r].c[1] = acc[r].c[2] = acc[r].c[3] = 0.0f;
            acc[r].s[0] = acc[r].s[1] = 0.0f;
        }
#pragma unroll
        for (int r = 0; r < kMaxRuns; ++r) {
            if (r >= runs) break;
            const GemvSegment* seg = nullptr;
            int rt = 0;
            if (!locate(u, r, seg, rt)) continue;
            const int type = seg->type;
            const int tile_bytes = packed_tile_bytes(type);
            for (int st = 0; st < stages_per_run; ++st) {
                if (!SHARED || turn == team) {  // SHARED: the teams take the stages in turn
                    const uint32_t slot = SHARED ? ring_pos : ring_pos * kTeams + team;
                    if (alive) alive = mbar_wait(sh.full + slot * 8, ring_parity, a.error_flag, 3, spin_limit);
                    const int kb = st * kStageTiles + member_warp;
                    if (kb < k_tiles) {
                        const uint32_t tile = ring + slot * (uint32_t)slot_bytes + (uint32_t)(member_warp * tile_bytes);
                        if (type == kQ4_K) tile_q4k<MEMBERS>(tile, ln, kb, lane, acc[r]);
                        else if (type == kQ6_K) tile_q6k<MEMBERS>(tile, ln, kb, lane, acc[r]);
                        else tile_q8_0<MEMBERS>(tile, ln, kb, lane, acc[r]);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sh.empty + slot * 8);  // this warp has left the stage
                }
                if (++ring_pos == ring_len) { ring_pos = 0; ring_parity ^= 1u; }
                if (++turn == kTeams) turn = 0;
            }
        }
        // Per-warp partial of (row, member): digits 1 and 2 are this lane's two columns, digit 3 is the
        // first column of the next lane; lanes with even t own member t / 2.
        if (done >= 2) bar_sync(kBarFree + set * 4 + buf, bar_threads);  // the epilogue warp has read this buffer
        float* red = sh.red + ((size_t)(set * 2 + buf) * kSetWarps + set_warp) * kMaxRuns * MEMBERS * 16;
#pragma unroll
        for (int r = 0; r < kMaxRuns; ++r) {
            if (r >= runs) break;
            const float d3a = __shfl_down_sync(0xffffffffu, acc[r].c[0], 1);
            const float d3b = __shfl_down_sync(0xffffffffu, acc[r].c[2], 1);
            if ((t & 1) == 0 && (t >> 1) < MEMBERS) {
                const float va = acc[r].c[0] + acc[r].c[1] * (1.0f / 128.0f) + d3a * (1.0f / 16384.0f) + acc[r].s[0];
                const float vb = acc[r].c[2] + acc[r].c[3] * (1.0f / 128.0f) + d3b * (1.0f / 16384.0f) + acc[r].s[1];
                float* dst = red + ((size_t)r * MEMBERS + (t >> 1)) * 16;
                dst[g] = va;
                dst[g + 8] = vb;
            }
        }
        __syncwarp();
        bar_arrive(kBarFull + set * 4 + buf, bar_threads);
    }
}

// f32 rows -> operand form: one warp per 32-span of one member.
__global__ void to_operand_kernel(const float* x, const int32_t* index, const float* norm_weight, int members, int k,
                                  ActOperand out) {
    const int lane = threadIdx.x & 31;
    const long long span_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long spans = (long long)members * (k / 32);
    if (span_id >= spans) return;
    const int m = (int)(span_id / (k / 32)), span = (int)(span_id - (long long)m * (k / 32));
    const int kk = span * 32 + lane;
    float v = x[(size_t)(index ? index[m] : m) * k + kk];
    const float sq = v * v;
    if (norm_weight != nullptr) v *= norm_weight[kk];
    ActOperand o = out;
    if (norm_weight == nullptr) o.ss32 = nullptr;
    operand_store_span(o, m, k, span, lane, v, sq);
}

// A wait nobody ends: one thread polls an mbarrier that no copy and no thread completes, through the same
// bounded wait as the kernels above, and leaves `code` in the error word when the limit runs out.
__global__ void wait_probe_kernel(int* error_flag, uint32_t spin_limit, int code) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_wait(smem_u32(&bar), 0, error_flag, code, spin_limit);
    }
}

int sm_count() {
    static int counts[kMaxDevices] = {0};  // per device ordinal
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (counts[dev] == 0) {
        if (cudaDeviceGetAttribute(&counts[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || counts[dev] <= 0) counts[dev] = 148;
    }
    return counts[dev];
}

}  // namespace

// Leaves a few KB of the SM's shared memory to small kernels that overlap this one's tail or head.
constexpr size_t kSmemBudget = 208 * 1024;

cudaError_t gemv_prepare() {
    static bool configured_on[kMaxDevices] = {false};  // function attributes are per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    bool& configured = configured_on[dev];
    if (!configured) {
        const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
        cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<1, false>, at, (int)kSmemBudget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<1, true>, at, (int)kSmemBudget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<2, false>, at, (int)kSmemBudget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<2, true>, at, (int)kSmemBudget);
        if (e != cudaSuccess) return e;
        sm_count();
        configured = true;
    }
    return cudaSuccess;
}

cudaError_t launch_wait_probe(cudaStream_t stream, int* error_flag, uint32_t spin_limit, int code) {
    if (error_flag == nullptr || spin_limit == 0 || spin_limit > (1u << 20)) return cudaErrorInvalidValue;
    wait_probe_kernel<<<1, 32, 0, stream>>>(error_flag, spin_limit, code);
    return cudaGetLastError();
}

cudaError_t launch_to_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                              int members, int k, ActOperand out) {
    if (members <= 0 || k % 32 != 0) return cudaErrorInvalidValue;
    const long long warps = (long long)members * (k / 32);
    to_operand_kernel<<<(unsigned int)((warps + 3) / 4), 128, 0, stream>>>(x, index, norm_weight, members, k, out);
    return cudaGetLastError();
}

cudaError_t launch_gemv_mma(cudaStream_t stream, const GemvArgs& args, bool programmatic) {
    if (args.members < 1 || args.members > kGemvMaxMembers || args.k % kTileCols != 0 || args.in.dig == nullptr ||
        args.in.sx == nullptr || args.in.sxs16 == nullptr || (args.in_has_norm && args.in.ss32 == nullptr)) {
        return cudaErrorInvalidValue;
    }
    int units = 0, slot_bytes = 0;
    if (args.epilogue == kSwiGLU) {
        if (args.n_segments != 2 || args.seg[0].row_tiles != args.seg[1].row_tiles || args.seg[0].n != args.seg[1].n) {
            return cudaErrorInvalidValue;
        }
        units = (args.seg[0].row_tiles + 1) / 2;
    } else {
        for (int i = 0; i < args.n_segments; ++i) units += (args.seg[i].row_tiles + 1) / 2;
    }
    for (int i = 0; i < args.n_segments; ++i) {
        const int b = packed_tile_bytes(args.seg[i].type);
        if (b == 0) return cudaErrorInvalidValue;
        slot_bytes = std::max(slot_bytes, b);
        if (args.out.dig != nullptr && args.seg[i].n % 32 != 0) return cudaErrorInvalidValue;
    }
    if (units <= 0) return cudaSuccess;
    const int K = args.k, planes = 3 * args.members;
    slot_bytes *= kStageTiles;
    const size_t fixed = (size_t)planes * (K + kPlanePad) + (size_t)args.members * (K / 32) * 4 +
                         (size_t)args.members * (K / 16) * 4 +
                         (size_t)kConsumerWarps * args.members * 16 * kHdrStride * 4 +
                         (size_t)2 * kConsumerWarps * kMaxRuns * args.members * 16 * 4 + 16 + 8;
    const size_t budget = kSmemBudget;
    if (fixed + (size_t)kTeams * (slot_bytes + 16) > budget) {
        if (args.members == 1) return cudaErrorInvalidValue;
        // Too many activation columns for this K: one launch per input vector.
        for (int m = 0; m < args.members; ++m) {
            GemvArgs one = args;
            one.members = 1;
            for (int i = 0; i < args.n_segments; ++i) one.seg[i].y = args.seg[i].y + (size_t)m * args.seg[i].n;
            one.in.dig = args.in.dig + (size_t)m * 3 * K;
            one.in.sx = args.in.sx + (size_t)m * (K / 32);
            one.in.sxs16 = args.in.sxs16 + (size_t)m * (K / 16);
            if (args.in.ss32) one.in.ss32 = args.in.ss32 + (size_t)m * (K / 32);
            const int n_out = args.seg[0].n;
            if (args.out.dig) one.out.dig = args.out.dig + (size_t)m * 3 * n_out;
            if (args.out.sx) one.out.sx = args.out.sx + (size_t)m * (n_out / 32);
            if (args.out.sxs16) one.out.sxs16 = args.out.sxs16 + (size_t)m * (n_out / 16);
            if (args.out.ss32) one.out.ss32 = args.out.ss32 + (size_t)m * (n_out / 32);
            if (args.swiglu_f32) one.swiglu_f32 = args.swiglu_f32 + (size_t)m * n_out;
            cudaError_t e = launch_gemv_mma(stream, one, programmatic);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    // Every team has its own ring slots, so a warp observes each phase of the barriers it waits on
    // (the one-bit parity wait requires that).
    const int slots_per_team = (int)std::min<size_t>(3, (budget - fixed) / ((size_t)kTeams * (slot_bytes + 16)));
    if (slots_per_team < 1) return cudaErrorInvalidValue;
    const size_t smem = fixed + (size_t)slots_per_team * kTeams * (slot_bytes + 16);
    {
        cudaError_t e = gemv_prepare();
        if (e != cudaSuccess) return e;
    }
    const int grid = std::min(units, sm_count());
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned int)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    // Few units per CTA: let all the warps cooperate on each unit.
    const bool shared = units < 2 * kTeams * grid;
    if (args.members == 1) {
        return shared ? cudaLaunchKernelEx(&cfg, gemv_mma_kernel<1, true>, args, slots_per_team, slot_bytes)
                      : cudaLaunchKernelEx(&cfg, gemv_mma_kernel<1, false>, args, slots_per_team, slot_bytes);
    }
    return shared ? cudaLaunchKernelEx(&cfg, gemv_mma_kernel<2, true>, args, slots_per_team, slot_bytes)
                  : cudaLaunchKernelEx(&cfg, gemv_mma_kernel<2, false>, args, slots_per_team, slot_bytes);
}

}  // namespace ribn
