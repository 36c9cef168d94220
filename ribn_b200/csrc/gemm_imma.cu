// Batched decode projection (3..64 rows): the same integer tensor-core arithmetic as the GEMV,
// organised as a small GEMM so that weights are read once per batch.
//
// A CTA owns 4 row tiles (64 output rows) and walks the k tiles.  Per k tile the weights of its
// row tiles and the activations' digit chunk for that k tile arrive by bulk (TMA) copies into a
// two-deep shared-memory ring.  The eight warps split the *members* (8 each, four MMA column
// tiles), so every warp reuses its B fragments across the CTA's row tiles and the activation
// chunk is read from shared memory once per warp.  Block scales are folded per 32 (Q4_K, Q8_0)
// or 16 (Q6_K) inputs exactly as in the GEMV; here each member has ONE activation scale for its
// whole vector (applied in the epilogue), so the fold factor does not depend on the column.
// The formats' offsets are removed with per-16-input digit sums supplied with the activations.
// Per-member work is independent of the other members and all sums are ordered: deterministic.
#include <cuda_fp16.h>

#include <algorithm>

#include "blocks.cuh"
#include "gemv.cuh"

namespace ribn {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRowTiles = 4;            // row tiles per CTA
constexpr int kMembersPerWarp = 8;      // 4 MMA column tiles of 2 members x (3 digits + pad)
constexpr int kMaxMembers = kWarps * kMembersPerWarp;
constexpr int kHdrStride = 36;          // floats per header row: 16 scales, 16 offset coefficients, pad
constexpr int kPlane = kBatchPlaneBytes; // bytes per (member, digit) plane of one k tile: 256 digits + bank padding
constexpr uint32_t kNibbles = 0x0F0F0F0Fu;
constexpr uint32_t kTopBits = 0x30303030u;
constexpr int kMagicInt = 0x4B400000;
constexpr float kMagic = 12582912.0f;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (error_flag != nullptr) atomicExch(error_flag, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void imma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(kMagicInt));
}
__device__ __forceinline__ void imma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(kMagicInt));
}
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t other) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(other));
    return r;
}
__device__ __forceinline__ float byte_f32(uint32_t w, int i) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (uint32_t)i)) - 8388608.0f;
}
__device__ __forceinline__ void fold(float (&a)[4], const int (&c)[4], float s0, float s1) {
    a[0] = fmaf(s0, __int_as_float(c[0]) - kMagic, a[0]);
    a[1] = fmaf(s0, __int_as_float(c[1]) - kMagic, a[1]);
    a[2] = fmaf(s1, __int_as_float(c[2]) - kMagic, a[2]);
    a[3] = fmaf(s1, __int_as_float(c[3]) - kMagic, a[3]);
}

// Header of one tile -> per row: 16 fold scales (one per 16 inputs; the 32-input formats repeat
// theirs) and 16 offset coefficients (multiplying the per-16 digit sums).  lane -> (row, half).
__device__ __forceinline__ void decode_header(int type, const unsigned char* tile, float* hdr, int lane) {
    const int row = lane >> 1, half = lane & 1;
    float* out = hdr + row * kHdrStride + half * 8;
    float sc[8], co[8];
    if (type == kQ4_K) {
        const uint4 h = *reinterpret_cast<const uint4*>(tile + 2048 + row * 16);
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        const uint32_t s4 = half ? ((h.w & kNibbles) | ((h.y >> 2) & kTopBits)) : (h.y & 0x3F3F3F3Fu);
        const uint32_t m4 = half ? (((h.w >> 4) & kNibbles) | ((h.z >> 2) & kTopBits)) : (h.z & 0x3F3F3F3Fu);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sc[2 * i] = sc[2 * i + 1] = d * byte_f32(s4, i);
            co[2 * i] = co[2 * i + 1] = -(dmin * byte_f32(m4, i));
        }
    } else if (type == kQ6_K) {
        const uint2 s8 = *reinterpret_cast<const uint2*>(tile + 3072 + row * 16 + half * 8);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(tile + 3328 + row * 2)));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sc[i] = d * (byte_f32(s8.x ^ 0x80808080u, i) - 128.0f);
            sc[4 + i] = d * (byte_f32(s8.y ^ 0x80808080u, i) - 128.0f);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) co[i] = -32.0f * sc[i];
    } else {
        const uint2 d4 = *reinterpret_cast<const uint2*>(tile + 4096 + row * 16 + half * 8);
        const float d0 = __half2float(__ushort_as_half((unsigned short)(d4.x & 0xffffu)));
        const float d1 = __half2float(__ushort_as_half((unsigned short)(d4.x >> 16)));
        const float d2 = __half2float(__ushort_as_half((unsigned short)(d4.y & 0xffffu)));
        const float d3 = __half2float(__ushort_as_half((unsigned short)(d4.y >> 16)));
        sc[0] = sc[1] = d0; sc[2] = sc[3] = d1; sc[4] = sc[5] = d2; sc[6] = sc[7] = d3;
#pragma unroll
        for (int i = 0; i < 8; ++i) co[i] = -128.0f * sc[i];
    }
    *reinterpret_cast<float4*>(out) = make_float4(sc[0], sc[1], sc[2], sc[3]);
    *reinterpret_cast<float4*>(out + 4) = make_float4(sc[4], sc[5], sc[6], sc[7]);
    *reinterpret_cast<float4*>(out + 16) = make_float4(co[0], co[1], co[2], co[3]);
    *reinterpret_cast<float4*>(out + 20) = make_float4(co[4], co[5], co[6], co[7]);
}

struct StageLayout {
    int w_bytes;      // kRowTiles weight tiles
    int x_bytes;      // members_padded * 3 digit planes
    int s_bytes;      // members_padded * 16 floats of per-16 digit sums
    int stage_bytes;
};

__global__ void __launch_bounds__(kThreads, 1) gemm_imma_kernel(const GemmArgs a, const StageLayout lay) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int K = a.k, k_tiles = K / kTileCols;
    unsigned char* stage[2] = {smem, smem + lay.stage_bytes};
    float* hdr = reinterpret_cast<float*>(smem + 2 * lay.stage_bytes);              // [kRowTiles][16][kHdrStride]
    const uint32_t bars = smem_u32(hdr + kRowTiles * 16 * kHdrStride);               // full[2]
    const bool swiglu = a.epilogue == kSwiGLU;

    // This CTA's row tiles: kRowTiles consecutive tiles of one segment (SwiGLU: 2 gate + the 2 matching up tiles).
    int seg = 0, unit = blockIdx.x;
    if (!swiglu) {
        while (seg + 1 < a.n_segments && unit >= (a.seg[seg].row_tiles + kRowTiles - 1) / kRowTiles) {
            unit -= (a.seg[seg].row_tiles + kRowTiles - 1) / kRowTiles;
            ++seg;
        }
    }
    const int rows_per_unit = swiglu ? kRowTiles / 2 : kRowTiles;
    auto tile_of = [&](int r, const GemvSegment*& s, int& rt) -> bool {
        s = &a.seg[swiglu ? (r & 1) : seg];
        rt = unit * rows_per_unit + (swiglu ? (r >> 1) : r);
        return rt < s->row_tiles;
    };

    int tile_type[kRowTiles];              // -1: beyond the segment's last row tile
    const unsigned char* tile_src[kRowTiles];
#pragma unroll
    for (int r = 0; r < kRowTiles; ++r) {
        const GemvSegment* s; int rt;
        const bool ok = tile_of(r, s, rt);
        tile_type[r] = ok ? s->type : -1;
        tile_src[r] = s->data + (size_t)rt * k_tiles * packed_tile_bytes(s->type);
    }

    if (threadIdx.x == 0) {
        mbar_init(bars, 1);
        mbar_init(bars + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto issue = [&](int kb) {  // thread 0: fill stage kb & 1 with the weights and activations of k tile kb
        const int b = kb & 1;
        const uint32_t bar = bars + b * 8;
        uint32_t bytes = (uint32_t)(lay.x_bytes + lay.s_bytes);
#pragma unroll
        for (int r = 0; r < kRowTiles; ++r)
            if (tile_type[r] >= 0) bytes += (uint32_t)packed_tile_bytes(tile_type[r]);
        mbar_expect_tx(bar, bytes);
#pragma unroll
        for (int r = 0; r < kRowTiles; ++r) {
            if (tile_type[r] >= 0) {
                const uint32_t tb = (uint32_t)packed_tile_bytes(tile_type[r]);
                bulk_g2s(smem_u32(stage[b] + r * (lay.w_bytes / kRowTiles)), tile_src[r] + (size_t)kb * tb, tb, bar);
            }
        }
        bulk_g2s(smem_u32(stage[b] + lay.w_bytes), a.dig + (size_t)kb * lay.x_bytes, (uint32_t)lay.x_bytes, bar);
        bulk_g2s(smem_u32(stage[b] + lay.w_bytes + lay.x_bytes), a.sum16 + (size_t)kb * (lay.s_bytes / 4),
                 (uint32_t)lay.s_bytes, bar);
    };
    if (threadIdx.x == 0) {
        issue(0);
        if (k_tiles > 1) issue(1);
    }

    float acc[kRowTiles][4][4];  // [row tile][column tile][c fragment]
#pragma unroll
    for (int r = 0; r < kRowTiles; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[r][j][0] = acc[r][j][1] = acc[r][j][2] = acc[r][j][3] = 0.0f;

    bool alive = true;
    const int member0 = warp * kMembersPerWarp;  // this warp's first member
    // Warps whose members lie beyond the (padded) batch only help with headers and barriers:
    // the stage holds digits for the padded member count and nothing further.
    const bool warp_live = member0 < (a.members + kMembersPerWarp - 1) / kMembersPerWarp * kMembersPerWarp;
    for (int kb = 0; kb < k_tiles; ++kb) {
        const int b = kb & 1;
        if (alive) alive = mbar_wait(bars + b * 8, (kb >> 1) & 1, a.error_flag, 4);
        const unsigned char* wst = stage[b];
        const signed char* xst = reinterpret_cast<const signed char*>(stage[b] + lay.w_bytes);
        const float* sst = reinterpret_cast<const float*>(stage[b] + lay.w_bytes + lay.x_bytes);
#pragma unroll
        for (int r = 0; r < kRowTiles; ++r)
            if (warp == r && tile_type[r] >= 0)
                decode_header(tile_type[r], wst + r * (lay.w_bytes / kRowTiles), hdr + r * 16 * kHdrStride, lane);
        __syncthreads();
        // B fragments: MMA column tile j holds members member0 + 2j (cols 0..2) and + 2j + 1 (cols 4..6).
        const bool col_live = (g & 3) < 3;
        const signed char* xcol[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = member0 + 2 * j + (g >> 2);
            xcol[j] = xst + ((size_t)m * 3 + (g & 3)) * kPlane + 8 * t;
        }
#pragma unroll
        for (int r = 0; r < kRowTiles; ++r) {
            const int type = warp_live ? tile_type[r] : -1;
            if (type < 0) continue;
            const unsigned char* tile = wst + r * (lay.w_bytes / kRowTiles);
            const float* h0 = hdr + (r * 16 + g) * kHdrStride;
            const float* h1 = h0 + 8 * kHdrStride;
            if (type == kQ6_K) {
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    const uint4 qh = *reinterpret_cast<const uint4*>(tile + 2048 + c * 512 + lane * 16);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint4 w = *reinterpret_cast<const uint4*>(tile + (c * 2 + h) * 512 + lane * 16);
                        const uint32_t wh0 = h == 0 ? qh.x : qh.z, wh1 = h == 0 ? qh.y : qh.w;
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const uint32_t l0 = (v & 1) ? w.y : w.x, l1 = (v & 1) ? w.w : w.z;
                            uint32_t t0, t1;
                            if (v == 0) { t0 = wh0 << 4; t1 = wh1 << 4; }
                            else if (v == 1) { t0 = wh0 << 2; t1 = wh1 << 2; }
                            else if (v == 2) { t0 = wh0; t1 = wh1; }
                            else { t0 = wh0 >> 2; t1 = wh1 >> 2; }
                            const uint32_t a0 = and_or(v < 2 ? l0 : l0 >> 4, kNibbles, t0 & kTopBits);
                            const uint32_t a1 = and_or(v < 2 ? l1 : l1 >> 4, kNibbles, t1 & kTopBits);
                            const int group = c * 4 + v, sub = group * 2 + h;
                            const float s0 = h0[sub], s1 = h1[sub];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint2 bb = col_live ? *reinterpret_cast<const uint2*>(xcol[j] + group * 32) : make_uint2(0u, 0u);
                                int cc[4];
                                imma_k16(cc, a0, a1, h == 0 ? bb.x : bb.y);
                                fold(acc[r][j], cc, s0, s1);
                            }
                        }
                    }
                }
            } else if (type == kQ4_K) {
#pragma unroll 1
                for (int jj = 0; jj < 4; ++jj) {
                    const uint4 w = *reinterpret_cast<const uint4*>(tile + jj * 512 + lane * 16);
                    const float se0 = h0[4 * jj], se1 = h1[4 * jj], so0 = h0[4 * jj + 2], so1 = h1[4 * jj + 2];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint2 be = col_live ? *reinterpret_cast<const uint2*>(xcol[j] + (2 * jj) * 32) : make_uint2(0u, 0u);
                        const uint2 bo = col_live ? *reinterpret_cast<const uint2*>(xcol[j] + (2 * jj + 1) * 32) : make_uint2(0u, 0u);
                        int ce[4], co[4];
                        imma_k32(ce, w.x & kNibbles, w.z & kNibbles, w.y & kNibbles, w.w & kNibbles, be.x, be.y);
                        imma_k32(co, (w.x >> 4) & kNibbles, (w.z >> 4) & kNibbles, (w.y >> 4) & kNibbles,
                                 (w.w >> 4) & kNibbles, bo.x, bo.y);
                        fold(acc[r][j], ce, se0, se1);
                        fold(acc[r][j], co, so0, so1);
                    }
                }
            } else {
#pragma unroll 1
                for (int b8 = 0; b8 < 8; ++b8) {
                    const uint4 w = *reinterpret_cast<const uint4*>(tile + b8 * 512 + lane * 16);
                    const float s0 = h0[2 * b8], s1 = h1[2 * b8];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint2 bb = col_live ? *reinterpret_cast<const uint2*>(xcol[j] + b8 * 32) : make_uint2(0u, 0u);
                        int cc[4];
                        imma_k32(cc, w.x, w.z, w.y, w.w, bb.x, bb.y);
                        fold(acc[r][j], cc, s0, s1);
                    }
                }
            }
            // Offsets: lanes with even t own digit 1 of member member0 + 2j + t/2; add coef[row][sub] * sum16[sub][member].
            if ((t & 1) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float* sums = sst + (size_t)(member0 + 2 * j + (t >> 1)) * 16;
                    float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float4 sv = *reinterpret_cast<const float4*>(sums + 4 * q4);
                        const float4 c0 = *reinterpret_cast<const float4*>(h0 + 16 + 4 * q4);
                        const float4 c1 = *reinterpret_cast<const float4*>(h1 + 16 + 4 * q4);
                        o0 = fmaf(c0.x, sv.x, o0); o0 = fmaf(c0.y, sv.y, o0); o0 = fmaf(c0.z, sv.z, o0); o0 = fmaf(c0.w, sv.w, o0);
                        o1 = fmaf(c1.x, sv.x, o1); o1 = fmaf(c1.y, sv.y, o1); o1 = fmaf(c1.z, sv.z, o1); o1 = fmaf(c1.w, sv.w, o1);
                    }
                    acc[r][j][0] += o0;
                    acc[r][j][2] += o1;
                }
            }
        }
        __syncthreads();  // everyone has left stage b and the headers
        if (threadIdx.x == 0 && kb + 2 < k_tiles) issue(kb + 2);
    }

    // Epilogue: even-t lanes hold (rows g, g + 8) x member (member0 + 2j + t/2) once the digits are combined.
#pragma unroll
    for (int r = 0; r < kRowTiles; ++r) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float d3a = __shfl_down_sync(0xffffffffu, acc[r][j][0], 1);
            const float d3b = __shfl_down_sync(0xffffffffu, acc[r][j][2], 1);
            acc[r][j][0] = acc[r][j][0] + acc[r][j][1] * (1.0f / 128.0f) + d3a * (1.0f / 16384.0f);
            acc[r][j][2] = acc[r][j][2] + acc[r][j][3] * (1.0f / 128.0f) + d3b * (1.0f / 16384.0f);
        }
    }
    if ((t & 1) != 0) return;
#pragma unroll
    for (int r = 0; r < (swiglu ? kRowTiles / 2 : kRowTiles); ++r) {
        // SwiGLU pairs accumulators (2r, 2r + 1) = (gate, up) of the same rows.
        const int ra = swiglu ? 2 * r : r;
        const GemvSegment* s; int rt;
        if (!tile_of(ra, s, rt)) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = member0 + 2 * j + (t >> 1);
            if (m >= a.members) continue;
            const float mult = a.member_scale[m];
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int n_index = rt * kTileRows + g + 8 * hrow;
                if (n_index >= s->n) continue;
                const float v = acc[ra][j][2 * hrow] * mult;
                float* y = a.seg[swiglu ? 0 : seg].y + (size_t)m * s->n + n_index;
                if (swiglu) {
                    const float u = acc[ra + 1][j][2 * hrow] * mult;
                    *y = v / (1.0f + expf(-v)) * u;
                } else if (a.epilogue == kResidual) {
                    *y += v;
                } else {
                    *y = v;
                }
            }
        }
    }
}

// ---- activations -> batch operand form -----------------------------------------------------
// Pass 1: per member, max |x * w| and sum of squares (one block per member).
__global__ void batch_scale_kernel(const float* x, const int32_t* index, const float* norm_weight, int k, float eps,
                                   float* digit_inv, float* member_scale) {
    __shared__ float red_max[32], red_sum[32];
    const int m = blockIdx.x;
    const float* row = x + (size_t)(index ? index[m] : m) * k;
    float amax = 0.0f, ss = 0.0f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const float v = row[i];
        ss = fmaf(v, v, ss);
        amax = fmaxf(amax, fabsf(norm_weight ? v * norm_weight[i] : v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    if ((threadIdx.x & 31) == 0) { red_max[threadIdx.x >> 5] = amax; red_sum[threadIdx.x >> 5] = ss; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float top = 0.0f, total = 0.0f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { top = fmaxf(top, red_max[w]); total += red_sum[w]; }
        const float inv_norm = norm_weight ? 1.0f / sqrtf(total / (float)k + eps) : 1.0f;
        digit_inv[m] = top > 0.0f ? 127.0f / top : 0.0f;
        member_scale[m] = (top / 127.0f) * inv_norm;  // digit scale times the RMSNorm factor
    }
}

// Pass 2: digits and per-16 digit sums, laid out per k tile: dig[kt][member][digit][kBatchPlaneBytes], sum16[kt][member][16].
__global__ void batch_digits_kernel(const float* x, const int32_t* index, const float* norm_weight, int members,
                                    int members_padded, int k, const float* digit_inv, signed char* dig, float* sum16) {
    const int lane = threadIdx.x & 31;
    const long long span_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int spans_per_member = k / 32;
    if (span_id >= (long long)members_padded * spans_per_member) return;
    const int m = (int)(span_id / spans_per_member), span = (int)(span_id % spans_per_member);
    const int kk = span * 32 + lane, kt = kk >> 8, in_tile = kk & 255;
    float v = 0.0f, inv = 0.0f;
    if (m < members) {
        v = x[(size_t)(index ? index[m] : m) * k + kk];
        if (norm_weight != nullptr) v *= norm_weight[kk];
        inv = digit_inv[m];
    }
    const float r0 = v * inv;
    const float f1 = fminf(fmaxf(rintf(r0), -127.0f), 127.0f);
    const float r1 = (r0 - f1) * 128.0f;
    const float f2 = fminf(fmaxf(rintf(r1), -127.0f), 127.0f);
    const float r2 = (r1 - f2) * 128.0f;
    const float f3 = fminf(fmaxf(rintf(r2), -127.0f), 127.0f);
    float value = f1 + f2 * (1.0f / 128.0f) + f3 * (1.0f / 16384.0f);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) value += __shfl_xor_sync(0xffffffffu, value, o);
    signed char* base = dig + (((size_t)kt * members_padded + m) * 3) * kPlane + operand_position(in_tile);
    base[0] = (signed char)(int)f1;
    base[kPlane] = (signed char)(int)f2;
    base[2 * kPlane] = (signed char)(int)f3;
    if ((lane & 15) == 0) sum16[((size_t)kt * members_padded + m) * 16 + (in_tile >> 4)] = value;
}

StageLayout layout_for(const GemmArgs& a) {
    StageLayout l{};
    int tile = 0;
    for (int i = 0; i < a.n_segments; ++i) tile = std::max(tile, packed_tile_bytes(a.seg[i].type));
    const int members_padded = (a.members + kMembersPerWarp - 1) / kMembersPerWarp * kMembersPerWarp;
    l.w_bytes = kRowTiles * tile;
    l.x_bytes = members_padded * 3 * kPlane;
    l.s_bytes = members_padded * 16 * 4;
    l.stage_bytes = (l.w_bytes + l.x_bytes + l.s_bytes + 127) / 128 * 128;
    return l;
}

}  // namespace

size_t batch_operand_digit_bytes(int members, int k) {
    const int mp = (members + kMembersPerWarp - 1) / kMembersPerWarp * kMembersPerWarp;
    return (size_t)(k / 256) * mp * 3 * kPlane;
}
size_t batch_operand_sum_floats(int members, int k) {
    const int mp = (members + kMembersPerWarp - 1) / kMembersPerWarp * kMembersPerWarp;
    return (size_t)(k / 256) * mp * 16;
}

cudaError_t launch_to_batch_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                                    int members, int k, float eps, BatchOperand out) {
    if (members <= 0 || members > kMaxMembers || k % 256 != 0) return cudaErrorInvalidValue;
    const int mp = (members + kMembersPerWarp - 1) / kMembersPerWarp * kMembersPerWarp;
    batch_scale_kernel<<<members, 256, 0, stream>>>(x, index, norm_weight, k, eps, out.digit_inv, out.member_scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const long long warps = (long long)mp * (k / 32);
    batch_digits_kernel<<<(unsigned int)((warps + 7) / 8), 256, 0, stream>>>(x, index, norm_weight, members, mp, k,
                                                                           out.digit_inv, out.dig, out.sum16);
    return cudaGetLastError();
}

cudaError_t launch_gemm_imma(cudaStream_t stream, const GemmArgs& args) {
    if (args.members < 1 || args.members > kMaxMembers || args.k % kTileCols != 0) return cudaErrorInvalidValue;
    const bool swiglu = args.epilogue == kSwiGLU;
    int units = 0;
    if (swiglu) {
        if (args.n_segments != 2 || args.seg[0].row_tiles != args.seg[1].row_tiles) return cudaErrorInvalidValue;
        units = (args.seg[0].row_tiles + kRowTiles / 2 - 1) / (kRowTiles / 2);
    } else {
        for (int i = 0; i < args.n_segments; ++i) units += (args.seg[i].row_tiles + kRowTiles - 1) / kRowTiles;
    }
    if (units <= 0) return cudaSuccess;
    const StageLayout lay = layout_for(args);
    const size_t smem = (size_t)2 * lay.stage_bytes + (size_t)kRowTiles * 16 * kHdrStride * 4 + 16;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_imma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured = 200 * 1024;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    gemm_imma_kernel<<<units, kThreads, smem, stream>>>(args, lay);
    return cudaGetLastError();
}

}  // namespace ribn
