// Tensor-core GEMV over tile-major repacked GGUF weights (decode, 1..4 rows).
//
// Why tensor cores for a GEMV: at B200's HBM rate one SM receives ~41 Q4_K
// weights per clock, which leaves ~3 issue slots per weight across its 128
// lanes.  A SIMT decode (extract, int->float, FMA) needs more than that, so
// the dot products run on `mma.sync.m16n8k16` instead and the lanes only
// unpack.  Weights enter the A operand as *subnormal binary16 integers*: a
// nibble masked into mantissa bits 0..3 (or 4..7) of a half is the exact
// value q * 2^-24 (q * 2^-20), so "dequantisation" is one AND per two
// weights and every product is exact.  Block scales multiply the fp32
// accumulator once per 32 (Q4_K, Q8_0) or 16 (Q6_K) inputs; the Q4_K minimum,
// the Q6_K -32 and the Q8_0 -128 offsets are applied through per-group sums
// of the activations.  Activations enter the B operand as two binary16
// columns per input vector, hi = f16(x) and lo = f16(x - hi), after a
// per-vector power-of-two scale, so the 8 MMA columns carry 4 vectors at
// ~22-bit precision.
//
// One CTA (8 warps) owns one 16-row tile; its warps split K and reduce
// through shared memory in a fixed order, so results are deterministic.
#include <cuda_fp16.h>
#include <string.h>

#include <thread>
#include <vector>

#include "blocks.cuh"
#include "gemv.cuh"

namespace ribn {

// ---------------------------------------------------------------------------
// host repack
// ---------------------------------------------------------------------------
namespace {

inline void put4(unsigned char* dst, const unsigned char* src, bool interleave, unsigned char flip) {
    if (interleave) {  // stored [k0, k2, k1, k3]: (w & 0x000F000F) -> (k0, k1), ((w >> 8) & ...) -> (k2, k3)
        dst[0] = src[0] ^ flip; dst[1] = src[2] ^ flip; dst[2] = src[1] ^ flip; dst[3] = src[3] ^ flip;
    } else {
        dst[0] = src[0] ^ flip; dst[1] = src[1] ^ flip; dst[2] = src[2] ^ flip; dst[3] = src[3] ^ flip;
    }
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
                        put4(tile + j * 512 + lane * 16 + (rs * 2 + h) * 4, live ? src : zeros, true, 0);
                    }
                }
            } else if (type == kQ6_K) {
                const unsigned char* blk = live ? raw + (row * k_blocks_per_row + kb) * 210 : zeros;
                for (int c = 0; c < 2; ++c) {
                    for (int h = 0; h < 2; ++h) {
                        const int l0 = 16 * h + 4 * t;
                        unsigned char* ql = tile + (c * 2 + h) * 512 + lane * 16 + rs * 8;
                        put4(ql, blk + c * 64 + l0, true, 0);
                        put4(ql + 4, blk + c * 64 + 32 + l0, true, 0);
                        put4(tile + 2048 + c * 512 + lane * 16 + (h * 2 + rs) * 4, blk + 128 + c * 32 + l0, true, 0);
                    }
                }
            } else {  // Q8_0: eight 34-byte blocks per 256 inputs, stored as q + 128
                for (int b = 0; b < 8; ++b) {
                    const unsigned char* blk = live ? raw + (row * k_blocks_per_row + kb * 8 + b) * 34 : nullptr;
                    for (int h = 0; h < 2; ++h) {
                        unsigned char* dst = tile + b * 512 + lane * 16 + (rs * 2 + h) * 4;
                        if (live) put4(dst, blk + 2 + 16 * h + 4 * t, false, 0x80);
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

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kXPad = 32;  // halves of padding per activation column (64 bytes)

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg128(const unsigned char* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

struct Shared {
    __half* xh;     // [cols][K + kXPad]
    float* s16;     // [K / 16][4]
    float* s32;     // [K / 32][4]
    float* hdr;     // [kWarps][16][16]
    float* red;     // [kWarps][16][4]
    float* scale;   // [4] per-member output scale
};

constexpr uint32_t kLowMask = 0x000F000Fu;   // nibble in mantissa bits 0..3: q * 2^-24
constexpr uint32_t kHighMask = 0x00F000F0u;  // nibble in mantissa bits 4..7: q * 2^-20
constexpr uint32_t kTopMask = 0x00300030u;   // Q6_K high two bits in mantissa bits 4..5
constexpr float kTwo24 = 16777216.0f;
constexpr float kTwo20 = 1048576.0f;

__device__ __forceinline__ float byte_of(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xffu); }

// B fragment of column `g` for the 16 inputs that start at k0: inputs
// 4t..4t+3 in natural order are exactly (b0, b1).
__device__ __forceinline__ uint2 load_b(const Shared& sh, int stride, int g, int t, int cols, int k0) {
    if (g < cols) return *reinterpret_cast<const uint2*>(sh.xh + (size_t)g * stride + k0 + 4 * t);
    return make_uint2(0u, 0u);
}

// ---- Q4_K -----------------------------------------------------------------
__device__ __forceinline__ void tile_q4k(const unsigned char* tile, const Shared& sh, int stride, int cols, int kb,
                                         int warp, int lane, float (&acc)[2]) {
    const int g = lane >> 2, t = lane & 3;
    uint4 qv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) qv[j] = ldg128(tile + j * 512 + lane * 16);
    float* hdr = sh.hdr + warp * 256;
    {
        // lane -> (row, scales | minima): eight six-bit values each
        const int row = lane >> 1, sel = lane & 1;
        const uint4 h = ldg128(tile + 2048 + row * 16);
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        uint32_t lo4, hi4;
        if (sel == 0) {
            lo4 = h.y & 0x3F3F3F3Fu;
            hi4 = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
        } else {
            lo4 = h.z & 0x3F3F3F3Fu;
            hi4 = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
        }
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[i] = byte_of(lo4, i); f[4 + i] = byte_of(hi4, i); }
        if (sel == 0) {
            // even groups are low nibbles (2^-24), odd groups high nibbles (2^-20)
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = d * f[i] * ((i & 1) ? kTwo20 : kTwo24);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = -(dmin * f[i]);
        }
        float4* dst = reinterpret_cast<float4*>(hdr + row * 16 + sel * 8);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncwarp();
    const float* h0 = hdr + g * 16;
    const float* h1 = hdr + (g + 8) * 16;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t r0a = qv[j].x, r0b = qv[j].y, r1a = qv[j].z, r1b = qv[j].w;
        const int ke = kb * 256 + (2 * j) * 32, ko = ke + 32;
        float ce[4] = {0.f, 0.f, 0.f, 0.f}, co[4] = {0.f, 0.f, 0.f, 0.f};
        uint2 b = load_b(sh, stride, g, t, cols, ke);
        mma16816(ce, r0a & kLowMask, r1a & kLowMask, (r0a >> 8) & kLowMask, (r1a >> 8) & kLowMask, b.x, b.y);
        b = load_b(sh, stride, g, t, cols, ke + 16);
        mma16816(ce, r0b & kLowMask, r1b & kLowMask, (r0b >> 8) & kLowMask, (r1b >> 8) & kLowMask, b.x, b.y);
        b = load_b(sh, stride, g, t, cols, ko);
        mma16816(co, r0a & kHighMask, r1a & kHighMask, (r0a >> 8) & kHighMask, (r1a >> 8) & kHighMask, b.x, b.y);
        b = load_b(sh, stride, g, t, cols, ko + 16);
        mma16816(co, r0b & kHighMask, r1b & kHighMask, (r0b >> 8) & kHighMask, (r1b >> 8) & kHighMask, b.x, b.y);
        const float se = sh.s32[(kb * 8 + 2 * j) * 4 + t], so = sh.s32[(kb * 8 + 2 * j + 1) * 4 + t];
        acc[0] = fmaf(h0[2 * j], ce[0] + ce[1], acc[0]);
        acc[0] = fmaf(h0[8 + 2 * j], se, acc[0]);
        acc[0] = fmaf(h0[2 * j + 1], co[0] + co[1], acc[0]);
        acc[0] = fmaf(h0[8 + 2 * j + 1], so, acc[0]);
        acc[1] = fmaf(h1[2 * j], ce[2] + ce[3], acc[1]);
        acc[1] = fmaf(h1[8 + 2 * j], se, acc[1]);
        acc[1] = fmaf(h1[2 * j + 1], co[2] + co[3], acc[1]);
        acc[1] = fmaf(h1[8 + 2 * j + 1], so, acc[1]);
    }
    __syncwarp();
}

// ---- Q6_K -----------------------------------------------------------------
__device__ __forceinline__ void tile_q6k(const unsigned char* tile, const Shared& sh, int stride, int cols, int kb,
                                         int warp, int lane, float (&acc)[2]) {
    const int g = lane >> 2, t = lane & 3;
    uint4 ql[4], qh[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) ql[i] = ldg128(tile + i * 512 + lane * 16);
#pragma unroll
    for (int c = 0; c < 2; ++c) qh[c] = ldg128(tile + 2048 + c * 512 + lane * 16);
    float* hdr = sh.hdr + warp * 256;
    {
        const int row = lane >> 1, half = lane & 1;
        const uint2 s8 = __ldg(reinterpret_cast<const uint2*>(tile + 3072 + row * 16 + half * 8));
        const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(tile + 3328 + row * 2)))) * kTwo24;
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[i] = d * (float)(signed char)((s8.x >> (8 * i)) & 0xffu);
            f[4 + i] = d * (float)(signed char)((s8.y >> (8 * i)) & 0xffu);
        }
        float4* dst = reinterpret_cast<float4*>(hdr + row * 16 + half * 8);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncwarp();
    const float* h0 = hdr + g * 16;
    const float* h1 = hdr + (g + 8) * 16;
    constexpr float kOffset = -32.0f / kTwo24;  // (q - 32): subtract 32 * sum(x) in the 2^-24 units of C
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 w = ql[c * 2 + h];
            const uint32_t la0 = w.x, lb0 = w.y, la1 = w.z, lb1 = w.w;
            const uint32_t wh0 = h == 0 ? qh[c].x : qh[c].z;
            const uint32_t wh1 = h == 0 ? qh[c].y : qh[c].w;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint32_t l0 = (v & 1) ? lb0 : la0, l1 = (v & 1) ? lb1 : la1;
                const int ls = (v < 2) ? 0 : 4;
                // high bits of variant v sit at bits 2v..2v+1 of each byte; move them to bits 4..5
                uint32_t a0, a1, a2, a3;
                if (v == 0) {
                    a0 = ((l0 >> ls) & kLowMask) | ((wh0 << 4) & kTopMask);
                    a1 = ((l1 >> ls) & kLowMask) | ((wh1 << 4) & kTopMask);
                    a2 = ((l0 >> (ls + 8)) & kLowMask) | ((wh0 >> 4) & kTopMask);
                    a3 = ((l1 >> (ls + 8)) & kLowMask) | ((wh1 >> 4) & kTopMask);
                } else if (v == 1) {
                    a0 = ((l0 >> ls) & kLowMask) | ((wh0 << 2) & kTopMask);
                    a1 = ((l1 >> ls) & kLowMask) | ((wh1 << 2) & kTopMask);
                    a2 = ((l0 >> (ls + 8)) & kLowMask) | ((wh0 >> 6) & kTopMask);
                    a3 = ((l1 >> (ls + 8)) & kLowMask) | ((wh1 >> 6) & kTopMask);
                } else if (v == 2) {
                    a0 = ((l0 >> ls) & kLowMask) | (wh0 & kTopMask);
                    a1 = ((l1 >> ls) & kLowMask) | (wh1 & kTopMask);
                    a2 = ((l0 >> (ls + 8)) & kLowMask) | ((wh0 >> 8) & kTopMask);
                    a3 = ((l1 >> (ls + 8)) & kLowMask) | ((wh1 >> 8) & kTopMask);
                } else {
                    a0 = ((l0 >> ls) & kLowMask) | ((wh0 >> 2) & kTopMask);
                    a1 = ((l1 >> ls) & kLowMask) | ((wh1 >> 2) & kTopMask);
                    a2 = ((l0 >> (ls + 8)) & kLowMask) | ((wh0 >> 10) & kTopMask);
                    a3 = ((l1 >> (ls + 8)) & kLowMask) | ((wh1 >> 10) & kTopMask);
                }
                const int group = c * 4 + v, sub = group * 2 + h;
                const int k0 = kb * 256 + group * 32 + 16 * h;
                float cc[4] = {0.f, 0.f, 0.f, 0.f};
                const uint2 b = load_b(sh, stride, g, t, cols, k0);
                mma16816(cc, a0, a1, a2, a3, b.x, b.y);
                const float s = sh.s16[(kb * 16 + sub) * 4 + t] * kOffset;
                acc[0] = fmaf(h0[sub], (cc[0] + cc[1]) + s, acc[0]);
                acc[1] = fmaf(h1[sub], (cc[2] + cc[3]) + s, acc[1]);
            }
        }
    }
    __syncwarp();
}

// ---- Q8_0 -----------------------------------------------------------------
__device__ __forceinline__ void tile_q8_0(const unsigned char* tile, const Shared& sh, int stride, int cols, int kb,
                                          int warp, int lane, float (&acc)[2]) {
    const int g = lane >> 2, t = lane & 3;
    float* hdr = sh.hdr + warp * 256;
    {
        const int row = lane >> 1, half = lane & 1;
        const uint2 d4 = __ldg(reinterpret_cast<const uint2*>(tile + 4096 + row * 16 + half * 8));
        float4 f;
        f.x = __half2float(__ushort_as_half((unsigned short)(d4.x & 0xffffu))) * kTwo24;
        f.y = __half2float(__ushort_as_half((unsigned short)(d4.x >> 16))) * kTwo24;
        f.z = __half2float(__ushort_as_half((unsigned short)(d4.y & 0xffffu))) * kTwo24;
        f.w = __half2float(__ushort_as_half((unsigned short)(d4.y >> 16))) * kTwo24;
        *reinterpret_cast<float4*>(hdr + row * 16 + half * 4) = f;
    }
    __syncwarp();
    const float* h0 = hdr + g * 16;
    const float* h1 = hdr + (g + 8) * 16;
    constexpr float kOffset = -128.0f / kTwo24;  // stored bytes are q + 128
#pragma unroll
    for (int b8 = 0; b8 < 8; ++b8) {
        const uint4 w = ldg128(tile + b8 * 512 + lane * 16);
        const int k0 = kb * 256 + b8 * 32;
        float cc[4] = {0.f, 0.f, 0.f, 0.f};
        uint2 b = load_b(sh, stride, g, t, cols, k0);
        mma16816(cc, __byte_perm(w.x, 0u, 0x4140), __byte_perm(w.z, 0u, 0x4140), __byte_perm(w.x, 0u, 0x4342),
                 __byte_perm(w.z, 0u, 0x4342), b.x, b.y);
        b = load_b(sh, stride, g, t, cols, k0 + 16);
        mma16816(cc, __byte_perm(w.y, 0u, 0x4140), __byte_perm(w.w, 0u, 0x4140), __byte_perm(w.y, 0u, 0x4342),
                 __byte_perm(w.w, 0u, 0x4342), b.x, b.y);
        const float s = sh.s32[(kb * 8 + b8) * 4 + t] * kOffset;
        acc[0] = fmaf(h0[b8], (cc[0] + cc[1]) + s, acc[0]);
        acc[1] = fmaf(h1[b8], (cc[2] + cc[3]) + s, acc[1]);
    }
    __syncwarp();
}

__device__ __forceinline__ float block_reduce_sum(float v, float* tmp) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) total += tmp[w];
    return total;
}

__device__ __forceinline__ float block_reduce_max(float v, float* tmp) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) total = fmaxf(total, tmp[w]);
    return total;
}

// Build the B operand: optional RMSNorm, power-of-two scaling, hi/lo binary16
// split, and the per-16 / per-32 sums of the reconstructed inputs.
__device__ void stage_activations(const GemvArgs& a, const Shared& sh, int stride) {
    const int K = a.k;
    float* tmp = sh.red;  // reused before the main loop
    for (int m = 0; m < a.members; ++m) {
        const float* x = a.x + (size_t)m * K;
        float ss = 0.0f, amax = 0.0f;
        for (int i = threadIdx.x; i < K; i += kThreads) {
            const float v = x[i];
            ss = fmaf(v, v, ss);
            amax = fmaxf(amax, fabsf(a.norm_weight ? v * a.norm_weight[i] : v));
        }
        float inv = 1.0f;
        if (a.norm_weight != nullptr) {
            const float total = block_reduce_sum(ss, tmp);
            inv = 1.0f / sqrtf(total / (float)K + a.eps);
        }
        amax = block_reduce_max(amax, tmp) * inv;
        // amax * s lies in [2^14, 2^15): inside binary16 range with room for rounding.
        int ex = 0;
        float s = 1.0f;
        if (amax > 0.0f && amax < INFINITY) {
            frexpf(amax, &ex);
            s = ldexpf(1.0f, max(-100, min(100, 15 - ex)));
        }
        if (threadIdx.x == 0) sh.scale[m] = 1.0f / s;
        __half* hi = sh.xh + (size_t)(2 * m) * stride;
        __half* lo = sh.xh + (size_t)(2 * m + 1) * stride;
        for (int sub = threadIdx.x; sub < K / 16; sub += kThreads) {
            float sum = 0.0f;
            __align__(16) __half hbuf[16];
            __align__(16) __half lbuf[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int k = sub * 16 + i;
                float v = x[k];
                if (a.norm_weight != nullptr) v = v * inv * a.norm_weight[k];
                v *= s;
                const __half h = __float2half_rn(v);
                const float hf = __half2float(h);
                const __half l = __float2half_rn(v - hf);
                hbuf[i] = h;
                lbuf[i] = l;
                sum += hf + __half2float(l);
            }
            uint4* hd = reinterpret_cast<uint4*>(hi + sub * 16);
            uint4* ld = reinterpret_cast<uint4*>(lo + sub * 16);
            hd[0] = reinterpret_cast<const uint4*>(hbuf)[0];
            hd[1] = reinterpret_cast<const uint4*>(hbuf)[1];
            ld[0] = reinterpret_cast<const uint4*>(lbuf)[0];
            ld[1] = reinterpret_cast<const uint4*>(lbuf)[1];
            sh.s16[sub * 4 + m] = sum;
        }
    }
    for (int m = a.members; m < 4; ++m) {
        for (int sub = threadIdx.x; sub < K / 16; sub += kThreads) sh.s16[sub * 4 + m] = 0.0f;
        if (threadIdx.x == 0) sh.scale[m] = 0.0f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (K / 32) * 4; i += kThreads) {
        const int grp = i >> 2, m = i & 3;
        sh.s32[i] = sh.s16[(2 * grp) * 4 + m] + sh.s16[(2 * grp + 1) * 4 + m];
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kThreads) gemv_mma_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = a.k, stride = K + kXPad, cols = 2 * a.members;
    Shared sh;
    sh.xh = reinterpret_cast<__half*>(smem_raw);
    sh.s16 = reinterpret_cast<float*>(smem_raw + (size_t)cols * stride * sizeof(__half));
    sh.s32 = sh.s16 + (K / 16) * 4;
    sh.hdr = sh.s32 + (K / 32) * 4;
    sh.red = sh.hdr + kWarps * 256;
    sh.scale = sh.red + kWarps * 64;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool swiglu = a.epilogue == kSwiGLU;
    // SwiGLU: warps 0..3 take the gate tile, warps 4..7 the matching up tile.
    int seg = 0, rt = blockIdx.x;
    if (swiglu) {
        seg = warp >> 2;
    } else {
        while (seg + 1 < a.n_segments && rt >= a.seg[seg].row_tiles) { rt -= a.seg[seg].row_tiles; ++seg; }
    }
    const GemvSegment s = a.seg[seg];
    const int k_tiles = K / kTileCols;
    const int split = swiglu ? 4 : kWarps, part = swiglu ? (warp & 3) : warp;
    const size_t tile_bytes = (size_t)packed_tile_bytes(s.type);
    const unsigned char* base = s.data + (size_t)rt * k_tiles * tile_bytes;

    stage_activations(a, sh, stride);

    float acc[2] = {0.0f, 0.0f};
    for (int kb = part; kb < k_tiles; kb += split) {
        const unsigned char* tile = base + (size_t)kb * tile_bytes;
        if (s.type == kQ4_K) tile_q4k(tile, sh, stride, cols, kb, warp, lane, acc);
        else if (s.type == kQ6_K) tile_q6k(tile, sh, stride, cols, kb, warp, lane, acc);
        else tile_q8_0(tile, sh, stride, cols, kb, warp, lane, acc);
    }
    const int g = lane >> 2, t = lane & 3;
    sh.red[warp * 64 + g * 4 + t] = acc[0];
    sh.red[warp * 64 + (g + 8) * 4 + t] = acc[1];
    __syncthreads();
    if (threadIdx.x < 64) {
        const int row = threadIdx.x >> 2, m = threadIdx.x & 3;
        const int n_index = rt * kTileRows + row;
        if (m < a.members && n_index < s.n) {
            if (swiglu) {
                float gate = 0.0f, up = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w) { gate += sh.red[w * 64 + row * 4 + m]; up += sh.red[(w + 4) * 64 + row * 4 + m]; }
                gate *= sh.scale[m];
                up *= sh.scale[m];
                a.seg[0].y[(size_t)m * a.seg[0].n + n_index] = gate / (1.0f + expf(-gate)) * up;
            } else {
                float total = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) total += sh.red[w * 64 + row * 4 + m];
                total *= sh.scale[m];
                float* dst = s.y + (size_t)m * s.n + n_index;
                *dst = a.epilogue == kResidual ? *dst + total : total;
            }
        }
    }
}

}  // namespace

cudaError_t launch_gemv_mma(cudaStream_t stream, const GemvArgs& args, bool dependent_launch) {
    (void)dependent_launch;
    if (args.members < 1 || args.members > kGemvMaxMembers || args.k % kTileCols != 0) return cudaErrorInvalidValue;
    int grid = 0;
    if (args.epilogue == kSwiGLU) {
        if (args.n_segments != 2 || args.seg[0].row_tiles != args.seg[1].row_tiles) return cudaErrorInvalidValue;
        grid = args.seg[0].row_tiles;
    } else {
        for (int i = 0; i < args.n_segments; ++i) grid += args.seg[i].row_tiles;
    }
    if (grid <= 0) return cudaSuccess;
    const int K = args.k, cols = 2 * args.members;
    const size_t smem = (size_t)cols * (K + kXPad) * sizeof(__half) + (size_t)(K / 16) * 4 * sizeof(float) +
                        (size_t)(K / 32) * 4 * sizeof(float) + (size_t)kWarps * 256 * sizeof(float) +
                        (size_t)kWarps * 64 * sizeof(float) + 4 * sizeof(float);
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    gemv_mma_kernel<<<grid, kThreads, smem, stream>>>(args);
    return cudaGetLastError();
}

}  // namespace ribn
