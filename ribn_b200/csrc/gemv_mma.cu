// Tensor-core GEMV over tile-major repacked GGUF weights (decode rows).
//
// Why tensor cores for a GEMV: at B200's HBM rate one SM receives ~41 Q4_K
// weights per clock, which leaves ~3 issue slots per weight across its 128
// lanes -- and integer/logic instructions issue at half rate.  A SIMT decode
// (extract, int->float, FMA) needs far more than that, so the dot products run
// on the integer tensor-core path, `mma.sync.m16n8k32.s32.u8.s8`, where a
// quantised weight needs no conversion at all: four packed nibbles become four
// u8 operands with one AND (a Q8_0 byte is an operand as stored) and products
// and sums are exact in int32.  The K-quants' integer group scales (6-bit for
// Q4_K, signed 8-bit per 16 inputs for Q6_K) multiply those integer sums as
// integers; one F32 step per 256 inputs applies the super-block scale and the
// activations' scale.  The formats' offsets (Q4_K minimum, Q6_K -32, Q8_0 -128)
// are removed through per-group sums of the activations.
//
// Activations arrive as plain F32 vectors (optionally with an RMSNorm weight to
// fold in) and every CTA converts them itself, once, into three signed 8-bit
// digit planes with one scale per 256 inputs: no operand-form hand-over between
// kernels, and a producer's epilogue is a plain F32 store.
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
// RMSNorm factor, then store, residual add or SwiGLU.
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
constexpr int kPlanePad = 32;       // bytes between activation digit planes (distinct banks per plane)
constexpr uint32_t kSpinLimit = 1u << 22;  // bounded waits: default number of polls before giving up
constexpr uint32_t kNibbles = 0x0F0F0F0Fu;
constexpr uint32_t kHighNibbles = 0xF0F0F0F0u;
constexpr uint32_t kTopBits = 0x30303030u;
constexpr uint32_t kSixBits = 0x3F3F3F3Fu;
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
// All consumer warps (a barrier id of its own: 1..12 belong to the teams' full / free barriers).
__device__ __forceinline__ void consumer_barrier() {
    asm volatile("bar.sync 13, %0;" ::"n"(kConsumerThreads) : "memory");
}

// D = A(u8, 16 x 32) * B(s8, 32 x 8), int32 results.
__device__ __forceinline__ void imma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, int init) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(init));
}
__device__ __forceinline__ void imma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// (a & mask) | other in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t other) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(other));
    return r;
}
// byte i (compile-time) of w, zero- or sign-extended
template <int I>
__device__ __forceinline__ int ubyte(uint32_t w) { return (int)__byte_perm(w, 0u, 0x4440u | (uint32_t)I); }
template <int I>
__device__ __forceinline__ int sbyte(uint32_t w) { return (int)(signed char)(w >> (8 * I)); }
__device__ __forceinline__ float half_lo(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu))); }
__device__ __forceinline__ float half_hi(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }

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
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint32_t v;
    asm volatile("{\n\t.reg .u16 t;\n\tld.shared.u16 t, [%1];\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(v) : "r"(addr));
    return v;
}

// Shared-memory map of the CTA (generic pointers for set-up and the epilogue warps).
//
// The input vectors arrive as F32 and every CTA turns them into the integer-MMA operand form itself, once,
// before its first tile: per 256 inputs (one k tile) of a member one scale sxt = max|x| / 127 and three signed
// 8-bit digit planes with  x ~= sxt * (d1 + d2 / 128 + d3 / 16384)  (|error| <= max|x| * 2.4e-7), stored in the
// MMA's B-fragment byte order (`operand_position`).  Alongside, per k tile: `cs` = the eight MMA columns'
// scales (sxt times the plane's weight; 0 for the unused columns), so that a row's result is the plain sum
// over columns of  scale * integer sum;  `t32` / `t16` = the sums of the dequantised inputs over each
// 32-input group / 16-input sub-group, which remove the formats' offsets (Q4_K minimum, Q6_K -32, Q8_0 -128).
struct Shared {
    unsigned char* ring;
    signed char* xq;   // [3 * members][K + kPlanePad] digit planes
    float* cs;         // [k_tiles][8]
    float* t32;        // [members][k_tiles][8]
    float* t16;        // [members][k_tiles][16]
    float* ssw;        // [members][32]: per-warp sums of squares of the raw inputs (RMSNorm)
    float* red;        // [kTeams][2][kTeamWarps][kMaxRuns][members][16]
    float* zero;       // a zeroed 16-byte word read by the empty MMA columns
    uint32_t full, empty;  // shared-space addresses of the mbarrier arrays
};

// Per-lane shared-space addresses of a consumer warp, fixed for the whole kernel.
struct Lane {
    uint32_t b;        // this lane's MMA column in the digit planes (+ 8 t), or the zeroed word
    uint32_t b_mask;   // all ones for a live column, zero for the empty columns (they read the zeroed word)
    uint32_t cs;       // column scales of this lane's two columns: cs + kb * 32
    uint32_t t32, t16; // this lane's member's offset sums: + kb * 32 / + kb * 64
    int g, t;
    bool has_member;   // this lane's columns belong to a member (t / 2 < members)
};

__device__ __forceinline__ uint2 load_b(const Lane& ln, uint32_t offset) {
    return lds64(ln.b + (offset & ln.b_mask));
}

// A lane's share of the result: rows g and g + 8, the sum over its two MMA columns (both belong to member
// t / 2).  Lanes whose columns belong to no member (t >= 2 with one member) carry exact zeros, so a row's
// sums are added in the same order whatever the number of members: batching changes no bit.
struct Accum {
    float r[2];
};

// A tile is processed as two halves of 128 inputs (`hf`), one after the other.

// ---- Q4_K: w = d * (sc * q) - dmin * m ------------------------------------------------------------
// The 6-bit group scales multiply the integer MMA results as integers (exact); one F32 step per half tile
// applies d and the column scales; the minima meet the group sums of the inputs.
template <int MEMBERS>
__device__ __forceinline__ void tile_q4k(uint32_t tile, const Lane& ln, int kb, int hf, int lane, Accum& acc) {
    const uint4 h0 = lds128(tile + 2048 + ln.g * 16), h1 = lds128(tile + 2048 + (ln.g + 8) * 16);
    // scales of this half's four groups as bytes (groups 0..3 sit in word y, 4..7 in w plus two bits of y)
    const uint32_t s0 = hf ? and_or(h0.w, kNibbles, (h0.y >> 2) & kTopBits) : (h0.y & kSixBits);
    const uint32_t s1 = hf ? and_or(h1.w, kNibbles, (h1.y >> 2) & kTopBits) : (h1.y & kSixBits);
    int ae[4] = {0, 0, 0, 0}, ao[4] = {0, 0, 0, 0};  // even groups; odd groups (carrying a factor 16)
    const uint32_t wbase = tile + hf * 1024 + lane * 16, bbase = kb * 256 + hf * 128;
#define RIBN_Q4K_STEP(J, BE, BO)                                                                             \
    {                                                                                                        \
        const uint4 w = lds128(wbase + J * 512);                                                             \
        const uint2 be = load_b(ln, bbase + J * 64), bo = load_b(ln, bbase + J * 64 + 32);                   \
        int ce[4], co[4];                                                                                    \
        imma_k32(ce, w.x & kNibbles, w.z & kNibbles, w.y & kNibbles, w.w & kNibbles, be.x, be.y, 0);        \
        imma_k32(co, w.x & kHighNibbles, w.z & kHighNibbles, w.y & kHighNibbles, w.w & kHighNibbles, bo.x, bo.y, 0); \
        const int e0 = ubyte<BE>(s0), e1 = ubyte<BE>(s1), o0 = ubyte<BO>(s0), o1 = ubyte<BO>(s1);            \
        ae[0] += e0 * ce[0]; ae[1] += e0 * ce[1]; ae[2] += e1 * ce[2]; ae[3] += e1 * ce[3];                  \
        ao[0] += o0 * co[0]; ao[1] += o0 * co[1]; ao[2] += o1 * co[2]; ao[3] += o1 * co[3];                  \
    }
    RIBN_Q4K_STEP(0, 0, 1)
    RIBN_Q4K_STEP(1, 2, 3)
#undef RIBN_Q4K_STEP
    const float2 cs = lds64f(ln.cs + kb * 32);
    const float u0 = fmaf((float)ao[0], 0.0625f, (float)ae[0]), u1 = fmaf((float)ao[1], 0.0625f, (float)ae[1]);
    const float u2 = fmaf((float)ao[2], 0.0625f, (float)ae[2]), u3 = fmaf((float)ao[3], 0.0625f, (float)ae[3]);
    const float r0 = fmaf(cs.y, u1, cs.x * u0) * half_lo(h0.x), r1 = fmaf(cs.y, u3, cs.x * u2) * half_lo(h1.x);
    // minima: lane (member t / 2, t % 2) takes two of this half's four groups for both of its rows
    float off0 = 0.0f, off1 = 0.0f;
    if (ln.has_member) {
        const uint32_t m0 = hf ? and_or(h0.w >> 4, kNibbles, (h0.z >> 2) & kTopBits) : (h0.z & kSixBits);
        const uint32_t m1 = hf ? and_or(h1.w >> 4, kNibbles, (h1.z >> 2) & kTopBits) : (h1.z & kSixBits);
        const uint32_t p0 = (ln.t & 1) ? m0 >> 16 : m0, p1 = (ln.t & 1) ? m1 >> 16 : m1;
        const float2 ts = lds64f(ln.t32 + kb * 32 + hf * 16 + (ln.t & 1) * 8);
        off0 = fmaf((float)ubyte<1>(p0), ts.y, (float)ubyte<0>(p0) * ts.x);
        off1 = fmaf((float)ubyte<1>(p1), ts.y, (float)ubyte<0>(p1) * ts.x);
    }
    acc.r[0] += fmaf(-half_hi(h0.x), off0, r0);
    acc.r[1] += fmaf(-half_hi(h1.x), off1, r1);
}

// ---- Q6_K: w = d * sc * (q - 32), one signed 8-bit scale per 16 inputs (k16 MMA) ------------------------
template <int MEMBERS>
__device__ __forceinline__ void tile_q6k(uint32_t tile, const Lane& ln, int kb, int hf, int lane, Accum& acc) {
    // the eight sub-group scales of this half, rows g and g + 8
    const uint2 s0 = lds64(tile + 3072 + ln.g * 16 + hf * 8), s1 = lds64(tile + 3072 + (ln.g + 8) * 16 + hf * 8);
    const float d0 = __half2float(__ushort_as_half((unsigned short)lds16(tile + 3328 + ln.g * 2)));
    const float d1 = __half2float(__ushort_as_half((unsigned short)lds16(tile + 3328 + (ln.g + 8) * 2)));
    int ai[4] = {0, 0, 0, 0};
    const uint32_t wbase = tile + lane * 16, bbase = kb * 256 + hf * 128;
    const uint4 qh = lds128(wbase + 2048 + hf * 512);
    // sub-group V * 2 + H of the half: word V / 2 of its scales, byte (V % 2) * 2 + H
#define RIBN_Q6K_STEP(H, V, W0, W1)                                                                           \
    {                                                                                                         \
        const uint32_t l0 = (V & 1) ? w.y : w.x, l1 = (V & 1) ? w.w : w.z;                                    \
        uint32_t t0, t1;                                                                                      \
        if (V == 0) { t0 = wh0 << 4; t1 = wh1 << 4; }                                                         \
        else if (V == 1) { t0 = wh0 << 2; t1 = wh1 << 2; }                                                    \
        else if (V == 2) { t0 = wh0; t1 = wh1; }                                                              \
        else { t0 = wh0 >> 2; t1 = wh1 >> 2; }                                                                \
        const uint32_t a0 = and_or(V < 2 ? l0 : l0 >> 4, kNibbles, t0 & kTopBits);                            \
        const uint32_t a1 = and_or(V < 2 ? l1 : l1 >> 4, kNibbles, t1 & kTopBits);                            \
        const uint2 b = load_b(ln, bbase + V * 32);                                                           \
        int cc[4];                                                                                            \
        imma_k16(cc, a0, a1, H == 0 ? b.x : b.y);                                                             \
        const int sa = sbyte<(V & 1) * 2 + H>(W0), sb = sbyte<(V & 1) * 2 + H>(W1);                           \
        ai[0] += sa * cc[0]; ai[1] += sa * cc[1]; ai[2] += sb * cc[2]; ai[3] += sb * cc[3];                   \
    }
#define RIBN_Q6K_HALF(H)                                                                                      \
    {                                                                                                         \
        const uint4 w = lds128(wbase + (hf * 2 + H) * 512);                                                   \
        const uint32_t wh0 = H == 0 ? qh.x : qh.z, wh1 = H == 0 ? qh.y : qh.w;                                \
        RIBN_Q6K_STEP(H, 0, s0.x, s1.x)                                                                       \
        RIBN_Q6K_STEP(H, 1, s0.x, s1.x)                                                                       \
        RIBN_Q6K_STEP(H, 2, s0.y, s1.y)                                                                       \
        RIBN_Q6K_STEP(H, 3, s0.y, s1.y)                                                                       \
    }
    RIBN_Q6K_HALF(0)
    RIBN_Q6K_HALF(1)
#undef RIBN_Q6K_HALF
#undef RIBN_Q6K_STEP
    const float2 cs = lds64f(ln.cs + kb * 32);
    const float r0 = fmaf(cs.y, (float)ai[1], cs.x * (float)ai[0]);
    const float r1 = fmaf(cs.y, (float)ai[3], cs.x * (float)ai[2]);
    // the -32 offset: sum over sub-groups of scale x (sum of the inputs); lane (member t / 2, t % 2) takes four of
    // this half's eight sub-groups
    float off0 = 0.0f, off1 = 0.0f;
    if (ln.has_member) {
        const uint32_t w0 = (ln.t & 1) ? s0.y : s0.x, w1 = (ln.t & 1) ? s1.y : s1.x;
        const float4 ts = lds128f(ln.t16 + kb * 64 + hf * 32 + (ln.t & 1) * 16);
        off0 = (float)sbyte<0>(w0) * ts.x; off0 = fmaf((float)sbyte<1>(w0), ts.y, off0);
        off0 = fmaf((float)sbyte<2>(w0), ts.z, off0); off0 = fmaf((float)sbyte<3>(w0), ts.w, off0);
        off1 = (float)sbyte<0>(w1) * ts.x; off1 = fmaf((float)sbyte<1>(w1), ts.y, off1);
        off1 = fmaf((float)sbyte<2>(w1), ts.z, off1); off1 = fmaf((float)sbyte<3>(w1), ts.w, off1);
    }
    acc.r[0] = fmaf(d0, fmaf(-32.0f, off0, r0), acc.r[0]);
    acc.r[1] = fmaf(d1, fmaf(-32.0f, off1, r1), acc.r[1]);
}

// ---- Q8_0: stored byte u = q + 128 is the u8 operand as is; w = d_b * (u - 128), one binary16 d per 32 -----
template <int MEMBERS>
__device__ __forceinline__ void tile_q8_0(uint32_t tile, const Lane& ln, int kb, int hf, int lane, Accum& acc) {
    // the four block scales of this half, rows g and g + 8
    const uint2 e0 = lds64(tile + 4096 + ln.g * 16 + hf * 8), e1 = lds64(tile + 4096 + (ln.g + 8) * 16 + hf * 8);
    const float2 cs = lds64f(ln.cs + kb * 32);
    const uint32_t wbase = tile + hf * 2048 + lane * 16, bbase = kb * 256 + hf * 128;
    const float dd0[4] = {half_lo(e0.x), half_hi(e0.x), half_lo(e0.y), half_hi(e0.y)};
    const float dd1[4] = {half_lo(e1.x), half_hi(e1.x), half_lo(e1.y), half_hi(e1.y)};
    float r0 = 0.0f, r1 = 0.0f;
#pragma unroll
    for (int b4 = 0; b4 < 4; ++b4) {
        const uint4 w = lds128(wbase + b4 * 512);
        const uint2 b = load_b(ln, bbase + b4 * 32);
        int cc[4];
        imma_k32(cc, w.x, w.z, w.y, w.w, b.x, b.y, kMagicInt);
        const float c0 = __int_as_float(cc[0]) - kMagic, c1 = __int_as_float(cc[1]) - kMagic;
        const float c2 = __int_as_float(cc[2]) - kMagic, c3 = __int_as_float(cc[3]) - kMagic;
        r0 = fmaf(dd0[b4], fmaf(cs.y, c1, cs.x * c0), r0);
        r1 = fmaf(dd1[b4], fmaf(cs.y, c3, cs.x * c2), r1);
    }
    // the -128 offset: lane (member t / 2, t % 2) takes two of this half's four blocks
    float off0 = 0.0f, off1 = 0.0f;
    if (ln.has_member) {
        const float2 ts = lds64f(ln.t32 + kb * 32 + hf * 16 + (ln.t & 1) * 8);
        const bool upper = (ln.t & 1) != 0;
        off0 = fmaf(upper ? dd0[3] : dd0[1], ts.y, (upper ? dd0[2] : dd0[0]) * ts.x);
        off1 = fmaf(upper ? dd1[3] : dd1[1], ts.y, (upper ? dd1[2] : dd1[0]) * ts.x);
    }
    acc.r[0] += fmaf(-128.0f, off0, r0);
    acc.r[1] += fmaf(-128.0f, off1, r1);
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

__device__ __forceinline__ float warp_sum_fixed(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

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
    const int k_tiles = K / kTileCols;
    Shared sh;
    {
        unsigned char* p = smem_raw;
        sh.ring = p; p += (size_t)slots * slot_bytes;
        sh.xq = reinterpret_cast<signed char*>(p); p += (size_t)planes * (K + kPlanePad);
        sh.cs = reinterpret_cast<float*>(p); p += (size_t)k_tiles * 8 * sizeof(float);
        sh.t32 = reinterpret_cast<float*>(p); p += (size_t)MEMBERS * k_tiles * 8 * sizeof(float);
        sh.t16 = reinterpret_cast<float*>(p); p += (size_t)MEMBERS * k_tiles * 16 * sizeof(float);
        sh.ssw = reinterpret_cast<float*>(p); p += (size_t)MEMBERS * 32 * sizeof(float);
        sh.red = reinterpret_cast<float*>(p); p += (size_t)2 * kConsumerWarps * kMaxRuns * MEMBERS * 16 * sizeof(float);
        sh.zero = reinterpret_cast<float*>(p); p += 16;
        sh.full = smem_u32(p); p += (size_t)slots * 8;
        sh.empty = smem_u32(p);
    }
    const int stages_per_run = (k_tiles + kStageTiles - 1) / kStageTiles;
    int total_units = 0;
    if (swiglu) total_units = (a.seg[0].row_tiles + 1) / 2;
    else for (int i = 0; i < a.n_segments; ++i) total_units += (a.seg[i].row_tiles + 1) / 2;
    const int u0 = (int)((long long)blockIdx.x * total_units / gridDim.x);
    const int u1 = (int)((long long)(blockIdx.x + 1) * total_units / gridDim.x);

    if (threadIdx.x == 0) {
        for (int i = 0; i < slots; ++i) { mbar_init(sh.full + i * 8, 1); mbar_init(sh.empty + i * 8, kTeamWarps); }
        sh.zero[0] = sh.zero[1] = sh.zero[2] = sh.zero[3] = 0.0f;
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
        // The weights do not depend on the previous kernel: the ring fills before that kernel has finished.
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
        bool have_norm = false;
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
            bar_sync(kBarFull + team * 4 + buf, bar_threads);  // the set's warps have left their partial sums of this unit
            if (!have_norm) {
                // RMSNorm factor: the consumer warps' sums of squares, added in warp order (they were written
                // before the consumers' first arrival at this barrier).
#pragma unroll
                for (int m = 0; m < MEMBERS; ++m) {
                    inv_norm[m] = 1.0f;
                    if (a.norm_weight != nullptr) {
                        float sum = 0.0f;
                        for (int w = 0; w < kConsumerWarps; ++w) sum += sh.ssw[m * 32 + w];
                        inv_norm[m] = 1.0f / sqrtf(sum / (float)K + a.eps);
                    }
                }
                have_norm = true;
            }
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
                if (valid) {
                    float* y = s.y + (size_t)m * s.n + n_index;
                    if (a.epilogue == kResidual) *y = prior[m] + v0[m];
                    else if (swiglu) *y = v0[m] / (1.0f + expf(-v0[m])) * v1[m];
                    else *y = v0[m];
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // First every consumer warp turns its share of the input vectors into the operand form (see Shared).
    {
        float ss_local[MEMBERS];
#pragma unroll
        for (int m = 0; m < MEMBERS; ++m) ss_local[m] = 0.0f;
        for (int item = warp; item < MEMBERS * k_tiles; item += kConsumerWarps) {
            const int m = item / k_tiles, kt = item - m * k_tiles;
            const float* src = a.x + (size_t)(a.x_index != nullptr ? a.x_index[m] : m) * K + (size_t)kt * kTileCols + lane * 8;
            const float4 xa = *reinterpret_cast<const float4*>(src), xb = *reinterpret_cast<const float4*>(src + 4);
            float v[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            float ssq = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ssq = fmaf(v[i], v[i], ssq);
            if (a.norm_weight != nullptr) {
                const float* wsrc = a.norm_weight + (size_t)kt * kTileCols + lane * 8;
                const float4 wa = *reinterpret_cast<const float4*>(wsrc), wb = *reinterpret_cast<const float4*>(wsrc + 4);
                v[0] *= wa.x; v[1] *= wa.y; v[2] *= wa.z; v[3] *= wa.w; v[4] *= wb.x; v[5] *= wb.y; v[6] *= wb.z; v[7] *= wb.w;
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            amax = operand_warp_max(amax);
            const float sxt = amax / 127.0f;
            const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
            uint32_t p1[2] = {0u, 0u}, p2[2] = {0u, 0u}, p3[2] = {0u, 0u};
            float total = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                int d1, d2, d3;
                total += operand_digits(v[i], inv, d1, d2, d3);
                p1[i >> 2] |= ((uint32_t)d1 & 0xffu) << (8 * (i & 3));
                p2[i >> 2] |= ((uint32_t)d2 & 0xffu) << (8 * (i & 3));
                p3[i >> 2] |= ((uint32_t)d3 & 0xffu) << (8 * (i & 3));
            }
            // inputs 8 lane .. 8 lane + 7 of the tile: span lane / 4, then `operand_position` inside the span
            signed char* plane = sh.xq + (size_t)(m * 3) * (K + kPlanePad) + kt * kTileCols + (lane >> 2) * 32 +
                                 16 * (lane & 1) + 4 * ((lane >> 1) & 1);
            *reinterpret_cast<uint32_t*>(plane) = p1[0];
            *reinterpret_cast<uint32_t*>(plane + 8) = p1[1];
            *reinterpret_cast<uint32_t*>(plane + (K + kPlanePad)) = p2[0];
            *reinterpret_cast<uint32_t*>(plane + (K + kPlanePad) + 8) = p2[1];
            *reinterpret_cast<uint32_t*>(plane + 2 * (K + kPlanePad)) = p3[0];
            *reinterpret_cast<uint32_t*>(plane + 2 * (K + kPlanePad) + 8) = p3[1];
            const float s16 = total + __shfl_xor_sync(0xffffffffu, total, 1);
            const float s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
            if ((lane & 1) == 0) sh.t16[((size_t)m * k_tiles + kt) * 16 + (lane >> 1)] = sxt * s16;
            if ((lane & 3) == 0) sh.t32[((size_t)m * k_tiles + kt) * 8 + (lane >> 2)] = sxt * s32;
            // column scales: columns 4 m .. 4 m + 2 are this member's digit planes, column 4 m + 3 stays empty
            if (lane < 4) {
                const float weight = lane == 0 ? 1.0f : lane == 1 ? (1.0f / 128.0f) : lane == 2 ? (1.0f / 16384.0f) : 0.0f;
                sh.cs[kt * 8 + m * 4 + lane] = sxt * weight;
                if (MEMBERS == 1) sh.cs[kt * 8 + 4 + lane] = 0.0f;
            }
            ss_local[m] += warp_sum_fixed(ssq);
        }
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MEMBERS; ++m) sh.ssw[m * 32 + warp] = ss_local[m];
        }
    }
    consumer_barrier();
    bool alive = true;

    const int g = lane >> 2, t = lane & 3;
    const int team = warp / kTeamWarps, member_warp = warp % kTeamWarps;
    Lane ln;
    {
        const bool live = (g & 3) < 3 && (g >> 2) < MEMBERS;
        const int member = (t >> 1) < MEMBERS ? (t >> 1) : 0;
        ln.has_member = (t >> 1) < MEMBERS;
        ln.b_mask = live ? 0xffffffffu : 0u;
        ln.b = live ? smem_u32(sh.xq) + (uint32_t)((g >> 2) * 3 + (g & 3)) * (uint32_t)(K + kPlanePad) + 8 * t
                    : smem_u32(sh.zero);
        ln.cs = smem_u32(sh.cs) + 8 * t;
        ln.t32 = smem_u32(sh.t32) + (uint32_t)member * k_tiles * 32;
        ln.t16 = smem_u32(sh.t16) + (uint32_t)member * k_tiles * 64;
        ln.g = g;
        ln.t = t;
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
        for (int r = 0; r < kMaxRuns; ++r) acc[r].r[0] = acc[r].r[1] = 0.0f;
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
                        if (type == kQ4_K) {
                            tile_q4k<MEMBERS>(tile, ln, kb, 0, lane, acc[r]);
                            tile_q4k<MEMBERS>(tile, ln, kb, 1, lane, acc[r]);
                        } else if (type == kQ6_K) {
                            tile_q6k<MEMBERS>(tile, ln, kb, 0, lane, acc[r]);
                            tile_q6k<MEMBERS>(tile, ln, kb, 1, lane, acc[r]);
                        } else {
                            tile_q8_0<MEMBERS>(tile, ln, kb, 0, lane, acc[r]);
                            tile_q8_0<MEMBERS>(tile, ln, kb, 1, lane, acc[r]);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sh.empty + slot * 8);  // this warp has left the stage
                }
                if (++ring_pos == ring_len) { ring_pos = 0; ring_parity ^= 1u; }
                if (++turn == kTeams) turn = 0;
            }
        }
        // Per-warp partial of (row, member): the lanes of one member's columns are folded in a fixed order.
        if (done >= 2) bar_sync(kBarFree + set * 4 + buf, bar_threads);  // the epilogue warp has read this buffer
        float* red = sh.red + ((size_t)(set * 2 + buf) * kSetWarps + set_warp) * kMaxRuns * MEMBERS * 16;
#pragma unroll
        for (int r = 0; r < kMaxRuns; ++r) {
            if (r >= runs) break;
            float va = acc[r].r[0], vb = acc[r].r[1];
            va += __shfl_xor_sync(0xffffffffu, va, 1);
            vb += __shfl_xor_sync(0xffffffffu, vb, 1);
            if ((t & 1) == 0 && (t >> 1) < MEMBERS) {
                float* dst = red + ((size_t)r * MEMBERS + (t >> 1)) * 16;
                dst[g] = va;
                dst[g + 8] = vb;
            }
        }
        __syncwarp();
        bar_arrive(kBarFull + set * 4 + buf, bar_threads);
    }
}

// A wait nobody ends: one thread polls an mbarrier that no copy and no thread completes, through the same
// bounded wait as the kernel above, and leaves `code` in the error word when the limit runs out.
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

cudaError_t launch_gemv_mma(cudaStream_t stream, const GemvArgs& args, bool programmatic) {
    if (args.members < 1 || args.members > kGemvMaxMembers || args.k % kTileCols != 0 || args.x == nullptr) {
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
    }
    if (units <= 0) return cudaSuccess;
    const int K = args.k, planes = 3 * args.members, k_tiles = K / kTileCols;
    slot_bytes *= kStageTiles;
    const size_t fixed = (size_t)planes * (K + kPlanePad) + (size_t)k_tiles * 8 * 4 +
                         (size_t)args.members * k_tiles * (8 + 16) * 4 + (size_t)args.members * 32 * 4 +
                         (size_t)2 * kConsumerWarps * kMaxRuns * args.members * 16 * 4 + 16 + 8;
    const size_t budget = kSmemBudget;
    if (fixed + (size_t)kTeams * (slot_bytes + 16) > budget) {
        if (args.members == 1) return cudaErrorInvalidValue;
        // Too many activation columns for this K: one launch per input vector.
        for (int m = 0; m < args.members; ++m) {
            GemvArgs one = args;
            one.members = 1;
            for (int i = 0; i < args.n_segments; ++i) one.seg[i].y = args.seg[i].y + (size_t)m * args.seg[i].n;
            if (args.x_index != nullptr) one.x_index = args.x_index + m;
            else one.x = args.x + (size_t)m * K;
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
