// Tensor-core GEMV over tile-major repacked GGUF weights (decode rows).
//
// Why tensor cores for a GEMV: at B200's HBM rate one SM receives ~41 Q4_K
// weights per clock, which leaves ~3 issue slots per weight across its 128
// lanes.  A SIMT decode (extract, int->float, FMA) needs more than that, so
// the dot products run on `mma.sync.m16n8k16` and the lanes only unpack.
// A weight enters the A operand as the bfloat16 `0x4300 | q` = 128 + q (one
// LOP3 per two weights, exact); the 128 and the formats' own offsets (Q4_K
// minimum, Q6_K -32, Q8_0 -128) are removed through per-16-input sums of the
// activations.  Block scales multiply the F32 accumulator once per 32 (Q4_K,
// Q8_0 nibble planes) or 16 (Q6_K) inputs.  Activations enter the B operand
// as three bfloat16 columns per input vector (hi + mid + lo, see ActOperand),
// produced by the previous kernel's epilogue.
//
// Execution: one persistent CTA per SM.  A producer warp streams the CTA's
// contiguous byte range of weight tiles into a shared-memory ring with bulk
// (TMA) copies completing on mbarriers; it starts before the programmatic
// dependency on the previous kernel resolves, so weights are already in
// flight while that kernel drains.  Eight consumer warps split each row
// tile's k tiles, reduce through shared memory in a fixed order
// (deterministic results), and warp 0 runs the epilogue (store, residual add,
// SwiGLU, and the operand form of the result for the next projection).
// Every wait is bounded: on expiry the kernel raises an error flag and runs
// to completion without waiting again.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "blocks.cuh"
#include "gemv.cuh"

namespace ribn {

// ---------------------------------------------------------------------------
// host repack
// ---------------------------------------------------------------------------
namespace {

// stored [k0, k2, k1, k3]: (w & 0x000F000F) -> (k0, k1), ((w >> 8) & ...) -> (k2, k3)
inline void put4(unsigned char* dst, const unsigned char* src, unsigned char flip) {
    dst[0] = src[0] ^ flip; dst[1] = src[2] ^ flip; dst[2] = src[1] ^ flip; dst[3] = src[3] ^ flip;
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

constexpr int kConsumerWarps = 16;  // two teams of eight; a team consumes every other stage
constexpr int kTeamWarps = 8;
constexpr int kStageTiles = 8;      // tiles per bulk copy / ring slot (one per warp of a team)
constexpr int kHdrStride = 20;      // floats per header row (80 bytes: conflict-free across the 8 row groups)
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one producer warp
constexpr int kXPad = 32;                        // elements of padding per activation column (64 bytes)
constexpr uint32_t kSpinLimit = 1u << 22;        // bounded waits: iterations before giving up
constexpr uint32_t kLowMask = 0x000F000Fu;
constexpr uint32_t kTopMask = 0x00300030u;
constexpr uint32_t kBias = 0x43004300u;          // bfloat16 128.0 in both halves: 0x4300 | q == 128 + q for q < 128

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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
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
__device__ __forceinline__ void consumer_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (w & mask) | other in one LOP3
__device__ __forceinline__ uint32_t pick(uint32_t w, uint32_t mask, uint32_t other = kBias) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "r"(mask), "r"(other));  // (a & b) | c
    return r;
}

struct Shared {
    unsigned char* ring;
    __nv_bfloat16* xs;  // [cols][K + kXPad]
    float* s16;         // [members][K / 16]
    float* s32;         // [members][K / 32]
    float* hdr;         // [kConsumerWarps][16][kHdrStride]
    float* red;         // [2][kConsumerWarps][runs][16][8]
    float* scale;       // [kGemvMaxMembers]
    uint32_t full, empty, xbar;  // shared-space addresses of the mbarrier arrays
};

struct Accum {
    float c[4];  // (row g, col 2t), (row g, col 2t+1), (row g+8, col 2t), (row g+8, col 2t+1)
    float s[2];  // offset terms of rows g, g+8 for the member whose sums this lane carries
};

__device__ __forceinline__ uint2 load_b(const Shared& sh, int stride, int g, int t, int cols, int k0) {
    if (g < cols) return *reinterpret_cast<const uint2*>(sh.xs + (size_t)g * stride + k0 + 4 * t);
    return make_uint2(0u, 0u);
}

__device__ __forceinline__ float byte_of(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xffu); }

// One group of 32 (or 16) inputs: scale the MMA result into the accumulators
// and add the offset term `coef * sum(x)` for the member this lane carries.
__device__ __forceinline__ void fold(Accum& a, const float (&c)[4], float s0, float s1, float k0, float k1, float sv) {
    a.c[0] = fmaf(s0, c[0], a.c[0]);
    a.c[1] = fmaf(s0, c[1], a.c[1]);
    a.c[2] = fmaf(s1, c[2], a.c[2]);
    a.c[3] = fmaf(s1, c[3], a.c[3]);
    a.s[0] = fmaf(k0, sv, a.s[0]);
    a.s[1] = fmaf(k1, sv, a.s[1]);
}

// ---- Q4_K: value = gs * q - gm, A = 128 + q  =>  gs * C - (128 gs + gm) * S --------
__device__ __forceinline__ void tile_q4k(const unsigned char* tile, const Shared& sh, int stride, int cols, int members,
                                         int kb, int warp, int lane, Accum& acc) {
    const int g = lane >> 2, t = lane & 3;
    uint4 qv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) qv[j] = *reinterpret_cast<const uint4*>(tile + j * 512 + lane * 16);
    float* hdr = sh.hdr + warp * (16 * kHdrStride);
    {
        const int row = lane >> 1, sel = lane & 1;
        const uint4 h = *reinterpret_cast<const uint4*>(tile + 2048 + row * 16);
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
        const uint32_t mn_lo = h.z & 0x3F3F3F3Fu, mn_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float gs_lo = d * byte_of(sc_lo, i), gs_hi = d * byte_of(sc_hi, i);
            if (sel == 0) {
                f[i] = gs_lo; f[4 + i] = gs_hi;
            } else {
                f[i] = -fmaf(128.0f, gs_lo, dmin * byte_of(mn_lo, i));
                f[4 + i] = -fmaf(128.0f, gs_hi, dmin * byte_of(mn_hi, i));
            }
        }
        float4* dst = reinterpret_cast<float4*>(hdr + row * kHdrStride + sel * 8);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncwarp();
    const float* h0 = hdr + g * kHdrStride;
    const float* h1 = hdr + (g + 8) * kHdrStride;
    const float* s32 = sh.s32 + (size_t)(t < members ? t : 0) * (stride - kXPad) / 32;
    const float live = t < members ? 1.0f : 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t r0a = qv[j].x, r0b = qv[j].y, r1a = qv[j].z, r1b = qv[j].w;
        const int ke = kb * 256 + (2 * j) * 32, ko = ke + 32;
        float ce[4] = {0.f, 0.f, 0.f, 0.f}, co[4] = {0.f, 0.f, 0.f, 0.f};
        uint2 b = load_b(sh, stride, g, t, cols, ke);
        mma_bf16(ce, pick(r0a, kLowMask), pick(r1a, kLowMask), pick(r0a >> 8, kLowMask), pick(r1a >> 8, kLowMask), b.x, b.y);
        b = load_b(sh, stride, g, t, cols, ke + 16);
        mma_bf16(ce, pick(r0b, kLowMask), pick(r1b, kLowMask), pick(r0b >> 8, kLowMask), pick(r1b >> 8, kLowMask), b.x, b.y);
        b = load_b(sh, stride, g, t, cols, ko);
        mma_bf16(co, pick(r0a >> 4, kLowMask), pick(r1a >> 4, kLowMask), pick(r0a >> 12, kLowMask),
                 pick(r1a >> 12, kLowMask), b.x, b.y);
        b = load_b(sh, stride, g, t, cols, ko + 16);
        mma_bf16(co, pick(r0b >> 4, kLowMask), pick(r1b >> 4, kLowMask), pick(r0b >> 12, kLowMask),
                 pick(r1b >> 12, kLowMask), b.x, b.y);
        const float2 sv = *reinterpret_cast<const float2*>(s32 + kb * 8 + 2 * j);
        const float2 sc0 = *reinterpret_cast<const float2*>(h0 + 2 * j), sc1 = *reinterpret_cast<const float2*>(h1 + 2 * j);
        const float2 of0 = *reinterpret_cast<const float2*>(h0 + 8 + 2 * j), of1 = *reinterpret_cast<const float2*>(h1 + 8 + 2 * j);
        fold(acc, ce, sc0.x, sc1.x, of0.x, of1.x, sv.x * live);
        fold(acc, co, sc0.y, sc1.y, of0.y, of1.y, sv.y * live);
    }
    __syncwarp();
}

// ---- Q6_K: value = gs * (q - 32), A = 128 + q  =>  gs * C - 160 gs * S (per 16 inputs) ---
__device__ __forceinline__ void tile_q6k(const unsigned char* tile, const Shared& sh, int stride, int cols, int members,
                                         int kb, int warp, int lane, Accum& acc) {
    const int g = lane >> 2, t = lane & 3;
    uint4 ql[4], qh[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) ql[i] = *reinterpret_cast<const uint4*>(tile + i * 512 + lane * 16);
#pragma unroll
    for (int c = 0; c < 2; ++c) qh[c] = *reinterpret_cast<const uint4*>(tile + 2048 + c * 512 + lane * 16);
    float* hdr = sh.hdr + warp * (16 * kHdrStride);
    {
        const int row = lane >> 1, half = lane & 1;
        const uint2 s8 = *reinterpret_cast<const uint2*>(tile + 3072 + row * 16 + half * 8);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(tile + 3328 + row * 2)));
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[i] = d * (float)(signed char)((s8.x >> (8 * i)) & 0xffu);
            f[4 + i] = d * (float)(signed char)((s8.y >> (8 * i)) & 0xffu);
        }
        float4* dst = reinterpret_cast<float4*>(hdr + row * kHdrStride + half * 8);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncwarp();
    const float* h0 = hdr + g * kHdrStride;
    const float* h1 = hdr + (g + 8) * kHdrStride;
    const float* s16 = sh.s16 + (size_t)(t < members ? t : 0) * (stride - kXPad) / 16;
    const float live = t < members ? -160.0f : 0.0f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 w = ql[c * 2 + h];
            const uint32_t wh0 = h == 0 ? qh[c].x : qh[c].z;
            const uint32_t wh1 = h == 0 ? qh[c].y : qh[c].w;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint32_t l0 = (v & 1) ? w.y : w.x, l1 = (v & 1) ? w.w : w.z;
                const int ls = (v < 2) ? 0 : 4;
                // high bits of variant v sit at bits 2v..2v+1 of each byte; move them to bits 4..5
                uint32_t t0, t1, t2, t3;
                if (v == 0) { t0 = wh0 << 4; t1 = wh1 << 4; t2 = wh0 >> 4; t3 = wh1 >> 4; }
                else if (v == 1) { t0 = wh0 << 2; t1 = wh1 << 2; t2 = wh0 >> 6; t3 = wh1 >> 6; }
                else if (v == 2) { t0 = wh0; t1 = wh1; t2 = wh0 >> 8; t3 = wh1 >> 8; }
                else { t0 = wh0 >> 2; t1 = wh1 >> 2; t2 = wh0 >> 10; t3 = wh1 >> 10; }
                const uint32_t a0 = pick(l0 >> ls, kLowMask, pick(t0, kTopMask));
                const uint32_t a1 = pick(l1 >> ls, kLowMask, pick(t1, kTopMask));
                const uint32_t a2 = pick(l0 >> (ls + 8), kLowMask, pick(t2, kTopMask));
                const uint32_t a3 = pick(l1 >> (ls + 8), kLowMask, pick(t3, kTopMask));
                const int group = c * 4 + v, sub = group * 2 + h;
                const int k0 = kb * 256 + group * 32 + 16 * h;
                float cc[4] = {0.f, 0.f, 0.f, 0.f};
                const uint2 b = load_b(sh, stride, g, t, cols, k0);
                mma_bf16(cc, a0, a1, a2, a3, b.x, b.y);
                const float sv = s16[kb * 16 + sub] * live;
                fold(acc, cc, h0[sub], h1[sub], h0[sub], h1[sub], sv);
            }
        }
    }
    __syncwarp();
}

// ---- Q8_0: stored u = q + 128 = 16 * hn + ln; value = d * (16 (hn - 8) + ln) ------------
//      two nibble planes, A = 128 + nibble  =>  d * (16 C_h + C_l) - d * (16 * 136 + 128) * S
__device__ __forceinline__ void tile_q8_0(const unsigned char* tile, const Shared& sh, int stride, int cols, int members,
                                          int kb, int warp, int lane, Accum& acc) {
    const int g = lane >> 2, t = lane & 3;
    float* hdr = sh.hdr + warp * (16 * kHdrStride);
    {
        const int row = lane >> 1, half = lane & 1;
        const uint2 d4 = *reinterpret_cast<const uint2*>(tile + 4096 + row * 16 + half * 8);
        float4 f;
        f.x = __half2float(__ushort_as_half((unsigned short)(d4.x & 0xffffu)));
        f.y = __half2float(__ushort_as_half((unsigned short)(d4.x >> 16)));
        f.z = __half2float(__ushort_as_half((unsigned short)(d4.y & 0xffffu)));
        f.w = __half2float(__ushort_as_half((unsigned short)(d4.y >> 16)));
        *reinterpret_cast<float4*>(hdr + row * kHdrStride + half * 4) = f;
    }
    __syncwarp();
    const float* h0 = hdr + g * kHdrStride;
    const float* h1 = hdr + (g + 8) * kHdrStride;
    const float* s32 = sh.s32 + (size_t)(t < members ? t : 0) * (stride - kXPad) / 32;
    const float live = t < members ? -(16.0f * 136.0f + 128.0f) : 0.0f;
#pragma unroll
    for (int b8 = 0; b8 < 8; ++b8) {
        const uint4 w = *reinterpret_cast<const uint4*>(tile + b8 * 512 + lane * 16);
        const int k0 = kb * 256 + b8 * 32;
        float cl[4] = {0.f, 0.f, 0.f, 0.f}, ch[4] = {0.f, 0.f, 0.f, 0.f};
        uint2 b = load_b(sh, stride, g, t, cols, k0);
        mma_bf16(cl, pick(w.x, kLowMask), pick(w.z, kLowMask), pick(w.x >> 8, kLowMask), pick(w.z >> 8, kLowMask), b.x, b.y);
        mma_bf16(ch, pick(w.x >> 4, kLowMask), pick(w.z >> 4, kLowMask), pick(w.x >> 12, kLowMask),
                 pick(w.z >> 12, kLowMask), b.x, b.y);
        b = load_b(sh, stride, g, t, cols, k0 + 16);
        mma_bf16(cl, pick(w.y, kLowMask), pick(w.w, kLowMask), pick(w.y >> 8, kLowMask), pick(w.w >> 8, kLowMask), b.x, b.y);
        mma_bf16(ch, pick(w.y >> 4, kLowMask), pick(w.w >> 4, kLowMask), pick(w.y >> 12, kLowMask),
                 pick(w.w >> 12, kLowMask), b.x, b.y);
        float cc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cc[i] = fmaf(16.0f, ch[i], cl[i]);
        const float sv = s32[kb * 8 + b8] * live;
        fold(acc, cc, h0[b8], h1[b8], h0[b8], h1[b8], sv);
    }
    __syncwarp();
}

// hi + mid + lo bfloat16 split of one value; returns the reconstructed sum.
__device__ __forceinline__ float split3(float v, __nv_bfloat16& hi, __nv_bfloat16& mid, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    mid = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(mid);
    lo = __float2bfloat16_rn(r2);
    return __bfloat162float(hi) + __bfloat162float(mid) + __bfloat162float(lo);
}

__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(kThreads, 1) gemv_mma_kernel(const GemvArgs a, const int slots, const int slot_bytes) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int K = a.k, stride = K + kXPad, cols = 3 * a.members;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool swiglu = a.epilogue == kSwiGLU;
    const int runs = swiglu ? 2 : 1;  // matrices per unit
    Shared sh;
    {
        unsigned char* p = smem_raw;
        sh.ring = p; p += (size_t)slots * slot_bytes;
        sh.xs = reinterpret_cast<__nv_bfloat16*>(p); p += (size_t)cols * stride * sizeof(__nv_bfloat16);
        sh.s16 = reinterpret_cast<float*>(p); p += (size_t)a.members * (K / 16) * sizeof(float);
        sh.s32 = reinterpret_cast<float*>(p); p += (size_t)a.members * (K / 32) * sizeof(float);
        sh.hdr = reinterpret_cast<float*>(p); p += (size_t)kConsumerWarps * 16 * kHdrStride * sizeof(float);
        sh.red = reinterpret_cast<float*>(p); p += (size_t)2 * kConsumerWarps * runs * 128 * sizeof(float);
        sh.scale = reinterpret_cast<float*>(p); p += 16;
        sh.full = smem_u32(p); p += (size_t)slots * 8;
        sh.empty = smem_u32(p); p += (size_t)slots * 8;
        sh.xbar = smem_u32(p);
    }
    const int k_tiles = K / kTileCols;
    const int stages_per_run = (k_tiles + kStageTiles - 1) / kStageTiles;
    const int stages_per_unit = runs * stages_per_run;
    int total_units = 0;
    if (swiglu) total_units = a.seg[0].row_tiles;
    else for (int i = 0; i < a.n_segments; ++i) total_units += a.seg[i].row_tiles;
    const int u0 = (int)((long long)blockIdx.x * total_units / gridDim.x);
    const int u1 = (int)((long long)(blockIdx.x + 1) * total_units / gridDim.x);

    if (threadIdx.x == 0) {
        for (int i = 0; i < slots; ++i) { mbar_init(sh.full + i * 8, 1); mbar_init(sh.empty + i * 8, kTeamWarps); }
        mbar_init(sh.xbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream begin (its weight prefetch does not depend on this one).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == kConsumerWarps) {
        // ---------------- producer: one bulk copy per stage of up to 8 contiguous tiles ----------------
        if (lane == 0) {
            bool alive = true;
            uint32_t n = 0;
            for (int u = u0; u < u1 && alive; ++u) {
                int seg = 0, rt = u;
                if (!swiglu) {
                    while (seg + 1 < a.n_segments && rt >= a.seg[seg].row_tiles) { rt -= a.seg[seg].row_tiles; ++seg; }
                }
                for (int r = 0; r < runs && alive; ++r) {
                    const GemvSegment& s = a.seg[swiglu ? r : seg];
                    const uint32_t tile_bytes = (uint32_t)packed_tile_bytes(s.type);
                    const unsigned char* run = s.data + (size_t)rt * k_tiles * tile_bytes;
                    for (int st = 0; st < stages_per_run; ++st, ++n) {
                        const uint32_t slot = n % (uint32_t)slots;
                        if (n >= (uint32_t)slots) {
                            alive = mbar_wait(sh.empty + slot * 8, ((n / (uint32_t)slots) - 1u) & 1u, a.error_flag, 1);
                            if (!alive) break;
                        }
                        const int tiles = min(kStageTiles, k_tiles - st * kStageTiles);
                        const uint32_t bytes = (uint32_t)tiles * tile_bytes;
                        mbar_expect_tx(sh.full + slot * 8, bytes);
                        bulk_g2s(smem_u32(sh.ring + (size_t)slot * slot_bytes),
                                 run + (size_t)st * kStageTiles * tile_bytes, bytes, sh.full + slot * 8);
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations come from the previous kernel
    if (threadIdx.x == 0) {
        const uint32_t col_bytes = (uint32_t)K * 2u, sum_bytes = (uint32_t)a.members * (K / 16) * 4u;
        mbar_expect_tx(sh.xbar, col_bytes * (uint32_t)cols + sum_bytes);
        for (int c = 0; c < cols; ++c) {
            bulk_g2s(smem_u32(sh.xs + (size_t)c * stride), a.in.x + (size_t)c * K, col_bytes, sh.xbar);
        }
        bulk_g2s(smem_u32(sh.s16), a.in.s16, sum_bytes, sh.xbar);
    }
    if (warp < a.members) {
        // RMSNorm factor of member `warp`: fixed-order sum of the producer's per-16 sums of squares.
        float inv = 1.0f;
        if (a.in_has_norm) {
            const float* ss = a.in.ss16 + (size_t)warp * (K / 16);
            float sum = 0.0f;
            for (int i = lane; i < K / 16; i += 32) sum += ss[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            inv = 1.0f / sqrtf(sum / (float)K + a.eps);
        }
        if (lane == 0) sh.scale[warp] = inv;
    }
    bool alive = mbar_wait(sh.xbar, 0, a.error_flag, 2);
    for (int i = threadIdx.x; i < a.members * (K / 32); i += kConsumerThreads) {
        const int m = i / (K / 32), grp = i - m * (K / 32);
        sh.s32[i] = sh.s16[(size_t)m * (K / 16) + 2 * grp] + sh.s16[(size_t)m * (K / 16) + 2 * grp + 1];
    }
    consumer_barrier();

    const int g = lane >> 2, t = lane & 3;
    const int team = warp / kTeamWarps, member_warp = warp % kTeamWarps;
    int buf = 0;
    for (int u = u0; u < u1; ++u) {
        int seg = 0, rt = u;
        if (!swiglu) {
            while (seg + 1 < a.n_segments && rt >= a.seg[seg].row_tiles) { rt -= a.seg[seg].row_tiles; ++seg; }
        }
        Accum acc[2];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            acc[w].c[0] = acc[w].c[1] = acc[w].c[2] = acc[w].c[3] = 0.0f;
            acc[w].s[0] = acc[w].s[1] = 0.0f;
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (r >= runs) break;
            const int type = a.seg[swiglu ? r : seg].type;
            const int tile_bytes = packed_tile_bytes(type);
            for (int st = 0; st < stages_per_run; ++st) {
                const uint32_t n = (uint32_t)(u - u0) * (uint32_t)stages_per_unit + (uint32_t)(r * stages_per_run + st);
                if ((int)(n & 1u) != team) continue;  // the other team's stage
                const uint32_t slot = n % (uint32_t)slots;
                if (alive) alive = mbar_wait(sh.full + slot * 8, (n / (uint32_t)slots) & 1u, a.error_flag, 3);
                const int kb = st * kStageTiles + member_warp;
                if (kb < k_tiles) {
                    const unsigned char* tile = sh.ring + (size_t)slot * slot_bytes + (size_t)member_warp * tile_bytes;
                    if (type == kQ4_K) tile_q4k(tile, sh, stride, cols, a.members, kb, warp, lane, acc[r]);
                    else if (type == kQ6_K) tile_q6k(tile, sh, stride, cols, a.members, kb, warp, lane, acc[r]);
                    else tile_q8_0(tile, sh, stride, cols, a.members, kb, warp, lane, acc[r]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sh.empty + slot * 8);  // this warp has left the stage
            }
        }
        // Offset terms join the carrier column of this lane's member: member m's hi column is 3m,
        // which is (t = 0, c[0]/c[2]) for m = 0 and (t = 1, c[1]/c[3]) for m = 1.
        float* red = sh.red + ((size_t)buf * kConsumerWarps + warp) * runs * 128;
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            if (w >= runs) break;
            if (t == 0) { acc[w].c[0] += acc[w].s[0]; acc[w].c[2] += acc[w].s[1]; }
            if (t == 1) { acc[w].c[1] += acc[w].s[0]; acc[w].c[3] += acc[w].s[1]; }
            float* r = red + w * 128;
            *reinterpret_cast<float2*>(r + g * 8 + 2 * t) = make_float2(acc[w].c[0], acc[w].c[1]);
            *reinterpret_cast<float2*>(r + (g + 8) * 8 + 2 * t) = make_float2(acc[w].c[2], acc[w].c[3]);
        }
        consumer_barrier();
        if (warp == 0) {
            // ---------------- epilogue: lane -> (member, row) ----------------
            const int m = lane >> 4, row = lane & 15;
            const GemvSegment& s = a.seg[swiglu ? 0 : seg];
            const int n_index = rt * kTileRows + row;
            const bool valid = m < a.members && n_index < s.n;
            const float* base = sh.red + (size_t)buf * kConsumerWarps * runs * 128;
            float v0 = 0.0f, v1 = 0.0f;
            if (m < a.members) {
#pragma unroll 4
                for (int w = 0; w < kConsumerWarps; ++w) {
#pragma unroll
                    for (int term = 0; term < 3; ++term) {
                        v0 += base[(size_t)w * runs * 128 + row * 8 + m * 3 + term];
                        if (swiglu) v1 += base[(size_t)w * runs * 128 + 128 + row * 8 + m * 3 + term];
                    }
                }
                const float scale = sh.scale[m];
                v0 *= scale;
                v1 *= scale;
            }
            float result = 0.0f, square = 0.0f;
            if (valid) {
                float* y = s.y + (size_t)m * s.n + n_index;
                if (a.epilogue == kResidual) {
                    result = *y + v0;
                    *y = result;
                    square = result * result;
                } else if (swiglu) {
                    result = v0 / (1.0f + expf(-v0)) * v1;
                    if (a.swiglu_f32 != nullptr) a.swiglu_f32[(size_t)m * s.n + n_index] = result;
                } else {
                    result = v0;
                    *y = v0;
                }
            }
            if (a.out.x != nullptr) {
                float v = result;
                if (valid && a.out_norm_weight != nullptr) v *= a.out_norm_weight[n_index];
                __nv_bfloat16 hi, mid, lo;
                const float recon = split3(v, hi, mid, lo);
                if (valid) {
                    __nv_bfloat16* ox = a.out.x + (size_t)m * 3 * s.n + n_index;
                    ox[0] = hi; ox[s.n] = mid; ox[2 * (size_t)s.n] = lo;
                }
                const float sum = half_warp_sum(recon), sq = half_warp_sum(square);
                if (row == 0 && m < a.members && rt * kTileRows < s.n) {
                    a.out.s16[(size_t)m * (s.n / 16) + rt] = sum;
                    if (a.out.ss16 != nullptr && a.epilogue == kResidual) a.out.ss16[(size_t)m * (s.n / 16) + rt] = sq;
                }
            }
        }
        buf ^= 1;
    }
}

// f32 rows -> operand form: one warp per 16 inputs of one member.
__global__ void to_operand_kernel(const float* x, const int32_t* index, const float* norm_weight, int members, int k,
                                  ActOperand out) {
    const int lane = threadIdx.x & 31;
    const long long pair = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // two 16-spans per warp
    const long long span = pair * 2 + (lane >> 4);
    const long long spans = (long long)members * (k / 16);
    const bool live = span < spans;
    const int m = live ? (int)(span / (k / 16)) : 0, sub = live ? (int)(span - (long long)m * (k / 16)) : 0;
    const int kk = sub * 16 + (lane & 15);
    float v = 0.0f, sq = 0.0f;
    if (live) {
        v = x[(size_t)(index ? index[m] : m) * k + kk];
        sq = v * v;
        if (norm_weight != nullptr) v *= norm_weight[kk];
    }
    __nv_bfloat16 hi, mid, lo;
    const float recon = split3(v, hi, mid, lo);
    if (live) {
        __nv_bfloat16* ox = out.x + (size_t)m * 3 * k + kk;
        ox[0] = hi; ox[k] = mid; ox[2 * (size_t)k] = lo;
    }
    const float sum = half_warp_sum(recon), ss = half_warp_sum(sq);
    if (live && (lane & 15) == 0) {
        out.s16[(size_t)m * (k / 16) + sub] = sum;
        if (norm_weight != nullptr && out.ss16 != nullptr) out.ss16[(size_t)m * (k / 16) + sub] = ss;
    }
}

int sm_count() {
    static int count = 0;
    if (count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0) count = 148;
    }
    return count;
}

}  // namespace

cudaError_t launch_to_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                              int members, int k, ActOperand out) {
    if (members <= 0 || k % 16 != 0) return cudaErrorInvalidValue;
    const long long warps = ((long long)members * (k / 16) + 1) / 2;
    to_operand_kernel<<<(unsigned int)((warps + 3) / 4), 128, 0, stream>>>(x, index, norm_weight, members, k, out);
    return cudaGetLastError();
}

cudaError_t launch_gemv_mma(cudaStream_t stream, const GemvArgs& args, bool programmatic) {
    if (args.members < 1 || args.members > kGemvMaxMembers || args.k % kTileCols != 0 || args.in.x == nullptr ||
        args.in.s16 == nullptr || (args.in_has_norm && args.in.ss16 == nullptr)) {
        return cudaErrorInvalidValue;
    }
    int units = 0, slot_bytes = 0;
    if (args.epilogue == kSwiGLU) {
        if (args.n_segments != 2 || args.seg[0].row_tiles != args.seg[1].row_tiles || args.seg[0].n != args.seg[1].n) {
            return cudaErrorInvalidValue;
        }
        units = args.seg[0].row_tiles;
    } else {
        for (int i = 0; i < args.n_segments; ++i) units += args.seg[i].row_tiles;
    }
    for (int i = 0; i < args.n_segments; ++i) {
        const int b = packed_tile_bytes(args.seg[i].type);
        if (b == 0) return cudaErrorInvalidValue;
        slot_bytes = std::max(slot_bytes, b);
        if (args.out.x != nullptr && args.seg[i].n % 16 != 0) return cudaErrorInvalidValue;
    }
    if (units <= 0) return cudaSuccess;
    const int K = args.k, cols = 3 * args.members, runs = args.epilogue == kSwiGLU ? 2 : 1;
    slot_bytes *= kStageTiles;
    const size_t fixed = (size_t)cols * (K + kXPad) * 2 + (size_t)args.members * (K / 16) * 4 +
                         (size_t)args.members * (K / 32) * 4 + (size_t)kConsumerWarps * 16 * kHdrStride * 4 +
                         (size_t)2 * kConsumerWarps * runs * 128 * 4 + 16 + 8;
    const size_t budget = 226 * 1024;
    if (fixed + (size_t)2 * (slot_bytes + 16) > budget) {
        if (args.members == 1) return cudaErrorInvalidValue;
        // Too many activation columns for this K: one launch per input vector.
        for (int m = 0; m < args.members; ++m) {
            GemvArgs one = args;
            one.members = 1;
            for (int i = 0; i < args.n_segments; ++i) one.seg[i].y = args.seg[i].y + (size_t)m * args.seg[i].n;
            one.in.x = args.in.x + (size_t)m * 3 * K;
            one.in.s16 = args.in.s16 + (size_t)m * (K / 16);
            if (args.in.ss16) one.in.ss16 = args.in.ss16 + (size_t)m * (K / 16);
            const int n_out = args.seg[0].n;
            if (args.out.x) one.out.x = args.out.x + (size_t)m * 3 * n_out;
            if (args.out.s16) one.out.s16 = args.out.s16 + (size_t)m * (n_out / 16);
            if (args.out.ss16) one.out.ss16 = args.out.ss16 + (size_t)m * (n_out / 16);
            if (args.swiglu_f32) one.swiglu_f32 = args.swiglu_f32 + (size_t)m * n_out;
            cudaError_t e = launch_gemv_mma(stream, one, programmatic);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    int slots = (int)std::min<size_t>(6, (budget - fixed) / ((size_t)slot_bytes + 16));
    const size_t smem = fixed + (size_t)slots * (slot_bytes + 16);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        if (e != cudaSuccess) return e;
        configured = budget;
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
    return cudaLaunchKernelEx(&cfg, gemv_mma_kernel, args, slots, slot_bytes);
}

}  // namespace ribn
