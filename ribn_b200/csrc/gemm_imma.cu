// Batched decode projection (3..64 rows): the same integer tensor-core arithmetic as the GEMV,
// organised as a small GEMM so that weights are read once per batch.
//
// A CTA owns 4 row tiles (64 output rows) and walks the k tiles.  Per k tile the weights of its
// row tiles and the activations' digit chunk for that k tile arrive by bulk (TMA) copies into a
// two-deep shared-memory ring.  The MMA columns are the flat list of (member, digit) pairs
// (column 3 m + d), so 64 members fill 24 column tiles with no padding; the twelve warps take two
// column tiles each and reuse their B fragments across the CTA's row tiles.  Block scales are
// folded per 32 (Q4_K, Q8_0) or 16 (Q6_K) inputs exactly as in the GEMV; here each member has ONE
// activation scale for its whole vector (applied in the epilogue), so the fold factor does not
// depend on the column.  The formats' offsets (Q4_K minimum, Q6_K -32, Q8_0 -128) are removed with
// per-16-input digit sums supplied with the activations: a second role of the same threads
// accumulates sum_sub coef[row][sub] * sum16[sub][member] over the whole K loop.  At the end the
// accumulators and the offset totals meet in shared memory, the three digits of each member are
// combined, and outputs are written with consecutive threads on consecutive output rows.
// Per-member work is independent of the other members and all sums are ordered: deterministic.
#include <cuda_fp16.h>

#include <algorithm>

#include "blocks.cuh"
#include "gemv.cuh"

// Measurement aid (0 in the shipped build): 1 = no MMA part, 2 = neither MMAs nor offsets, 3 = no offsets.
#ifndef RIBN_GEMM_PROBE
#define RIBN_GEMM_PROBE 0
#endif

namespace ribn {

namespace {

constexpr int kWarps = 12;              // MMA warps; two more serve them: one issues the copies, one decodes headers
constexpr int kProducerWarp = kWarps, kHeaderWarp = kWarps + 1;
constexpr int kThreads = (kWarps + 2) * 32;
constexpr int kColTiles = 2;            // MMA column tiles (8 columns each) per warp
constexpr int kMaxMembers = kGemmMaxMembers;
constexpr int kMemberPad = 8;           // members are padded to a multiple of this: 3 * 8 columns = 3 column tiles
constexpr int kQuadFloats = 8 * 8 * 4;  // fold scales of one row tile: [pair of scales 8][g 8][4]
constexpr int kPlane = kBatchPlaneBytes; // bytes per (member, digit) plane of one k tile: 256 digits + bank padding
constexpr int kCoefStride = 20;         // floats per row of offset coefficients (16 + bank spread)
constexpr int kExchStride = 3 * kMaxMembers + 1;  // floats per row of the accumulator exchange
constexpr int kOffStride = kMaxMembers + 1;       // floats per row of the offset exchange
constexpr uint32_t kNibbles = 0x0F0F0F0Fu;
constexpr uint32_t kTopBits = 0x30303030u;
constexpr int kMagicInt = 0x4B400000;
constexpr float kMagic = 12582912.0f;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

// Header of one tile, decoded by one warp (lane -> row lane / 2, half lane % 2 of the row's scales):
//   quads[pair][g][4] = {s(g, 2 pair), s(g, 2 pair + 1), s(g + 8, 2 pair), s(g + 8, 2 pair + 1)}
//       fold scales as the MMA lanes read them (one 128-bit load per pair): 8 scales per row for the
//       32-input formats (pairs 0..3), 16 for Q6_K (pairs 0..7);
//   coef[row][16] offset coefficients multiplying the per-16-input digit sums.
__device__ __forceinline__ void decode_header(int type, const unsigned char* tile, float* quads, float* coef, int lane) {
    const int row = lane >> 1, half = lane & 1;
    float* q = quads + (row & 7) * 4 + (row >> 3) * 2;
    float* co = coef + row * kCoefStride + half * 8;
    if (type == kQ4_K) {
        const uint4 h = *reinterpret_cast<const uint4*>(tile + 2048 + row * 16);
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        const uint32_t s4 = half ? ((h.w & kNibbles) | ((h.y >> 2) & kTopBits)) : (h.y & 0x3F3F3F3Fu);
        const uint32_t m4 = half ? (((h.w >> 4) & kNibbles) | ((h.z >> 2) & kTopBits)) : (h.z & 0x3F3F3F3Fu);
        float sc[4], mn[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { sc[i] = d * byte_f32(s4, i); mn[i] = -(dmin * byte_f32(m4, i)); }
        *reinterpret_cast<float2*>(q + (half * 2) * 32) = make_float2(sc[0], sc[1]);
        *reinterpret_cast<float2*>(q + (half * 2 + 1) * 32) = make_float2(sc[2], sc[3]);
        *reinterpret_cast<float4*>(co) = make_float4(mn[0], mn[0], mn[1], mn[1]);
        *reinterpret_cast<float4*>(co + 4) = make_float4(mn[2], mn[2], mn[3], mn[3]);
    } else if (type == kQ6_K) {
        const uint2 s8 = *reinterpret_cast<const uint2*>(tile + 3072 + row * 16 + half * 8);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(tile + 3328 + row * 2)));
        float sc[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sc[i] = d * (byte_f32(s8.x ^ 0x80808080u, i) - 128.0f);
            sc[4 + i] = d * (byte_f32(s8.y ^ 0x80808080u, i) - 128.0f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<float2*>(q + (half * 4 + i) * 32) = make_float2(sc[2 * i], sc[2 * i + 1]);
        *reinterpret_cast<float4*>(co) = make_float4(-32.0f * sc[0], -32.0f * sc[1], -32.0f * sc[2], -32.0f * sc[3]);
        *reinterpret_cast<float4*>(co + 4) = make_float4(-32.0f * sc[4], -32.0f * sc[5], -32.0f * sc[6], -32.0f * sc[7]);
    } else {
        const uint2 d4 = *reinterpret_cast<const uint2*>(tile + 4096 + row * 16 + half * 8);
        const float d0 = __half2float(__ushort_as_half((unsigned short)(d4.x & 0xffffu)));
        const float d1 = __half2float(__ushort_as_half((unsigned short)(d4.x >> 16)));
        const float d2 = __half2float(__ushort_as_half((unsigned short)(d4.y & 0xffffu)));
        const float d3 = __half2float(__ushort_as_half((unsigned short)(d4.y >> 16)));
        *reinterpret_cast<float2*>(q + (half * 2) * 32) = make_float2(d0, d1);
        *reinterpret_cast<float2*>(q + (half * 2 + 1) * 32) = make_float2(d2, d3);
        *reinterpret_cast<float4*>(co) = make_float4(-128.0f * d0, -128.0f * d0, -128.0f * d1, -128.0f * d1);
        *reinterpret_cast<float4*>(co + 4) = make_float4(-128.0f * d2, -128.0f * d2, -128.0f * d3, -128.0f * d3);
    }
}

struct StageLayout {
    int w_bytes;      // the row tiles of the CTA
    int x_bytes;      // members_padded * 3 digit planes
    int s_bytes;      // members_padded * 16 floats of per-16 digit sums
    int stage_bytes;
};

// MMA part of one k tile for the CTA's row tiles of one format.  B fragments are loaded once and
// reused across the row tiles.  MASKED: tiles of another format or absent tiles have their bit in
// `mask` clear and are skipped; otherwise all four row tiles are processed without branches (an
// absent tile then computes on stale shared memory into accumulators that are never stored), which
// lets the compiler interleave the independent MMA -> fold chains.
template <int RT, bool MASKED>
__device__ __forceinline__ void mma_q4k(const unsigned char* wst, int tile_stride, const float* quads, int mask,
                                        const signed char* const (&xcol)[kColTiles], int lane, int g,
                                        float (&acc)[RT][kColTiles][4]) {
#pragma unroll 1
    for (int jj = 0; jj < 4; ++jj) {
        uint2 be[kColTiles], bo[kColTiles];
#pragma unroll
        for (int j = 0; j < kColTiles; ++j) {
            be[j] = *reinterpret_cast<const uint2*>(xcol[j] + (2 * jj) * 32);
            bo[j] = *reinterpret_cast<const uint2*>(xcol[j] + (2 * jj + 1) * 32);
        }
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            if (MASKED && !(mask >> r & 1)) continue;
            const uint4 w = *reinterpret_cast<const uint4*>(wst + r * tile_stride + jj * 512 + lane * 16);
            const float4 sc = *reinterpret_cast<const float4*>(quads + r * kQuadFloats + jj * 32 + g * 4);
            const uint32_t e0 = w.x & kNibbles, e1 = w.z & kNibbles, e2 = w.y & kNibbles, e3 = w.w & kNibbles;
            const uint32_t o0 = (w.x >> 4) & kNibbles, o1 = (w.z >> 4) & kNibbles, o2 = (w.y >> 4) & kNibbles,
                           o3 = (w.w >> 4) & kNibbles;
#pragma unroll
            for (int j = 0; j < kColTiles; ++j) {
                int ce[4], co[4];
                imma_k32(ce, e0, e1, e2, e3, be[j].x, be[j].y);
                imma_k32(co, o0, o1, o2, o3, bo[j].x, bo[j].y);
                fold(acc[r][j], ce, sc.x, sc.z);
                fold(acc[r][j], co, sc.y, sc.w);
            }
        }
    }
}

template <int RT, bool MASKED>
__device__ __forceinline__ void mma_q8_0(const unsigned char* wst, int tile_stride, const float* quads, int mask,
                                         const signed char* const (&xcol)[kColTiles], int lane, int g,
                                         float (&acc)[RT][kColTiles][4]) {
#pragma unroll 1
    for (int jj = 0; jj < 4; ++jj) {
        uint2 be[kColTiles], bo[kColTiles];
#pragma unroll
        for (int j = 0; j < kColTiles; ++j) {
            be[j] = *reinterpret_cast<const uint2*>(xcol[j] + (2 * jj) * 32);
            bo[j] = *reinterpret_cast<const uint2*>(xcol[j] + (2 * jj + 1) * 32);
        }
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            if (MASKED && !(mask >> r & 1)) continue;
            const uint4 we = *reinterpret_cast<const uint4*>(wst + r * tile_stride + (2 * jj) * 512 + lane * 16);
            const uint4 wo = *reinterpret_cast<const uint4*>(wst + r * tile_stride + (2 * jj + 1) * 512 + lane * 16);
            const float4 sc = *reinterpret_cast<const float4*>(quads + r * kQuadFloats + jj * 32 + g * 4);
#pragma unroll
            for (int j = 0; j < kColTiles; ++j) {
                int ce[4], co[4];
                imma_k32(ce, we.x, we.z, we.y, we.w, be[j].x, be[j].y);
                imma_k32(co, wo.x, wo.z, wo.y, wo.w, bo[j].x, bo[j].y);
                fold(acc[r][j], ce, sc.x, sc.z);
                fold(acc[r][j], co, sc.y, sc.w);
            }
        }
    }
}

template <int RT, bool MASKED>
__device__ __forceinline__ void mma_q6k(const unsigned char* wst, int tile_stride, const float* quads, int mask,
                                        const signed char* const (&xcol)[kColTiles], int lane, int g,
                                        float (&acc)[RT][kColTiles][4]) {
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
        uint2 bb[4][kColTiles];
#pragma unroll
        for (int v = 0; v < 4; ++v)
#pragma unroll
            for (int j = 0; j < kColTiles; ++j) bb[v][j] = *reinterpret_cast<const uint2*>(xcol[j] + (c * 4 + v) * 32);
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            if (MASKED && !(mask >> r & 1)) continue;
            const unsigned char* tile = wst + r * tile_stride + lane * 16;
            const uint4 qh = *reinterpret_cast<const uint4*>(tile + 2048 + c * 512);
            const uint4 w0 = *reinterpret_cast<const uint4*>(tile + (c * 2) * 512);       // inputs 0..15 of each group
            const uint4 w1 = *reinterpret_cast<const uint4*>(tile + (c * 2 + 1) * 512);   // inputs 16..31
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                // scales of 16-input halves 2 (4 c + v), + 1 for rows g and g + 8
                const float4 sc = *reinterpret_cast<const float4*>(quads + r * kQuadFloats + (c * 4 + v) * 32 + g * 4);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint4 w = h == 0 ? w0 : w1;
                    const uint32_t wh0 = h == 0 ? qh.x : qh.z, wh1 = h == 0 ? qh.y : qh.w;
                    const uint32_t l0 = (v & 1) ? w.y : w.x, l1 = (v & 1) ? w.w : w.z;
                    // the variant's two high bits sit at bits 2v..2v+1 of each high-bit byte: move them to bits 4..5
                    uint32_t t0, t1;
                    if (v == 0) { t0 = wh0 << 4; t1 = wh1 << 4; }
                    else if (v == 1) { t0 = wh0 << 2; t1 = wh1 << 2; }
                    else if (v == 2) { t0 = wh0; t1 = wh1; }
                    else { t0 = wh0 >> 2; t1 = wh1 >> 2; }
                    const uint32_t a0 = and_or(v < 2 ? l0 : l0 >> 4, kNibbles, t0 & kTopBits);
                    const uint32_t a1 = and_or(v < 2 ? l1 : l1 >> 4, kNibbles, t1 & kTopBits);
#pragma unroll
                    for (int j = 0; j < kColTiles; ++j) {
                        int cc[4];
                        imma_k16(cc, a0, a1, h == 0 ? bb[v][j].x : bb[v][j].y);
                        fold(acc[r][j], cc, h == 0 ? sc.x : sc.y, h == 0 ? sc.z : sc.w);
                    }
                }
            }
        }
    }
}

template <int RT>
__global__ void __launch_bounds__(kThreads, 1) gemm_imma_kernel(const GemmArgs a, const StageLayout lay) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int K = a.k, k_tiles = K / kTileCols;
    const int mp = (a.members + kMemberPad - 1) / kMemberPad * kMemberPad;
    unsigned char* stage[2] = {smem, smem + lay.stage_bytes};
    // per stage: fold scales [RT][kQuadFloats] and offset coefficients [(RT * 16)][kCoefStride]
    float* quads = reinterpret_cast<float*>(smem + 2 * lay.stage_bytes);
    float* coef = quads + 2 * RT * kQuadFloats;
    // mbarriers: full[2] (copies landed), ready[2] (headers decoded), empty[2] (MMA warps left the stage)
    const uint32_t bars = smem_u32(coef + 2 * (RT * 16) * kCoefStride);
    const uint32_t bar_full = bars, bar_ready = bars + 16, bar_empty = bars + 32;
    const bool swiglu = a.epilogue == kSwiGLU;

    // This CTA's row tiles: RT consecutive tiles of one segment (SwiGLU: 2 gate + the 2 matching up tiles).
    int seg = 0, unit = blockIdx.x;
    if (!swiglu) {
        while (seg + 1 < a.n_segments && unit >= (a.seg[seg].row_tiles + RT - 1) / RT) {
            unit -= (a.seg[seg].row_tiles + RT - 1) / RT;
            ++seg;
        }
    }
    const int rows_per_unit = swiglu ? RT / 2 : RT;
    auto tile_of = [&](int r, const GemvSegment*& s, int& rt) -> bool {
        s = &a.seg[swiglu ? (r & 1) : seg];
        rt = unit * rows_per_unit + (swiglu ? (r >> 1) : r);
        return rt < s->row_tiles;
    };

    int tile_type[RT];              // -1: beyond the segment's last row tile
    const unsigned char* tile_src[RT];
    int mask_q4k = 0, mask_q6k = 0, mask_q8 = 0;
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const GemvSegment* s; int rt;
        const bool ok = tile_of(r, s, rt);
        tile_type[r] = ok ? s->type : -1;
        tile_src[r] = s->data + (size_t)rt * k_tiles * packed_tile_bytes(s->type);
        if (tile_type[r] == kQ4_K) mask_q4k |= 1 << r;
        if (tile_type[r] == kQ6_K) mask_q6k |= 1 << r;
        if (tile_type[r] == kQ8_0) mask_q8 |= 1 << r;
    }
    // One format across the present row tiles (the usual case): the branch-free MMA path serves.
    const int uniform_type = (mask_q6k | mask_q8) == 0 ? kQ4_K : (mask_q4k | mask_q8) == 0 ? kQ6_K
                           : (mask_q4k | mask_q6k) == 0 ? kQ8_0 : -1;

    if (threadIdx.x == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_full + 8 * b, 1);
            mbar_init(bar_ready + 8 * b, 1);
            mbar_init(bar_empty + 8 * b, kWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Coefficients of absent row tiles read as zero (their offset sums are computed but never stored).
    for (int i = threadIdx.x; i < 2 * (RT * 16) * kCoefStride; i += kThreads) coef[i] = 0.0f;
    __syncthreads();

    const int tile_stride = lay.w_bytes / RT;
    float acc[RT][kColTiles][4];  // [row tile][column tile][c fragment]
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < kColTiles; ++j) acc[r][j][0] = acc[r][j][1] = acc[r][j][2] = acc[r][j][3] = 0.0f;
    // Offset role: row groups of four rows, `warp` and (for the first four warps) `warp + 12`;
    // members lane and lane + 32.
    float off[2][4][2];
#pragma unroll
    for (int p = 0; p < 2; ++p)
#pragma unroll
        for (int i = 0; i < 4; ++i) off[p][i][0] = off[p][i][1] = 0.0f;
    // Column tiles 2 warp, 2 warp + 1 of the 3 mp / 8 in use; warps beyond them skip the MMA part
    // (the stage holds digit planes for the padded member count and nothing further).
    const int col_tiles = 3 * mp / 8;

    if (warp == kProducerWarp) {
        // ---- copies: stage kb & 1 receives the weights and activations of k tile kb -------------------
        if (lane == 0) {
            bool alive = true;
            for (int kb = 0; kb < k_tiles; ++kb) {
                const int b = kb & 1;
                if (kb >= 2 && alive) alive = mbar_wait(bar_empty + 8 * b, ((kb >> 1) - 1) & 1, a.error_flag, 5);
                const uint32_t bar = bar_full + 8 * b;
                uint32_t bytes = (uint32_t)(lay.x_bytes + lay.s_bytes);
#pragma unroll
                for (int r = 0; r < RT; ++r)
                    if (tile_type[r] >= 0) bytes += (uint32_t)packed_tile_bytes(tile_type[r]);
                mbar_expect_tx(bar, bytes);
                // digits and sums of a k tile are adjacent in memory: one copy
                bulk_g2s(smem_u32(stage[b] + lay.w_bytes), a.chunks + (size_t)kb * (lay.x_bytes + lay.s_bytes),
                         (uint32_t)(lay.x_bytes + lay.s_bytes), bar);
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    if (tile_type[r] >= 0) {
                        const uint32_t tb = (uint32_t)packed_tile_bytes(tile_type[r]);
                        bulk_g2s(smem_u32(stage[b] + r * tile_stride), tile_src[r] + (size_t)kb * tb, tb, bar);
                    }
                }
            }
        }
    } else if (warp == kHeaderWarp) {
        // ---- headers: one stage ahead of the MMA warps ----------------------------------------------------
        bool alive = true;
        for (int kb = 0; kb < k_tiles; ++kb) {
            const int b = kb & 1;
            if (alive) alive = mbar_wait(bar_full + 8 * b, (kb >> 1) & 1, a.error_flag, 4);
#pragma unroll
            for (int r = 0; r < RT; ++r)
                if (tile_type[r] >= 0)
                    decode_header(tile_type[r], stage[b] + r * tile_stride, quads + (b * RT + r) * kQuadFloats,
                                  coef + (b * (RT * 16) + r * 16) * kCoefStride, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_ready + 8 * b);
        }
    } else {
        const bool off_live0 = lane < mp, off_live1 = lane + 32 < mp;
        const bool warp_live = kColTiles * warp < col_tiles;
        bool alive = true;
        for (int kb = 0; kb < k_tiles; ++kb) {
            const int b = kb & 1;
            if (alive) alive = mbar_wait(bar_ready + 8 * b, (kb >> 1) & 1, a.error_flag, 6);
            const unsigned char* wst = stage[b];
            const signed char* xst = reinterpret_cast<const signed char*>(stage[b] + lay.w_bytes);
            const float4* sst = reinterpret_cast<const float4*>(stage[b] + lay.w_bytes + lay.x_bytes);  // [4][mp]
            const float* qd = quads + b * RT * kQuadFloats;
            // ---- offsets ---------------------------------------------------------------------------
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                if (RIBN_GEMM_PROBE == 2 || RIBN_GEMM_PROBE == 3) break;
                const int group = warp + p * kWarps;
                if (group >= (RT * 16) / 4) break;                                         // warp-uniform
                const float* cf = coef + (size_t)(b * (RT * 16) + 4 * group) * kCoefStride;   // broadcast reads
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const float4 s0 = off_live0 ? sst[q4 * mp + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 s1 = off_live1 ? sst[q4 * mp + lane + 32] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 c = *reinterpret_cast<const float4*>(cf + i * kCoefStride + 4 * q4);
                        off[p][i][0] = fmaf(c.x, s0.x, off[p][i][0]); off[p][i][0] = fmaf(c.y, s0.y, off[p][i][0]);
                        off[p][i][0] = fmaf(c.z, s0.z, off[p][i][0]); off[p][i][0] = fmaf(c.w, s0.w, off[p][i][0]);
                        off[p][i][1] = fmaf(c.x, s1.x, off[p][i][1]); off[p][i][1] = fmaf(c.y, s1.y, off[p][i][1]);
                        off[p][i][1] = fmaf(c.z, s1.z, off[p][i][1]); off[p][i][1] = fmaf(c.w, s1.w, off[p][i][1]);
                    }
                }
            }
            // ---- integer MMAs: column 8 (2 warp + j) + g is digit plane number `column` of the stage ----
            if (warp_live && RIBN_GEMM_PROBE != 1 && RIBN_GEMM_PROBE != 2) {
                const signed char* xcol[kColTiles];
#pragma unroll
                for (int j = 0; j < kColTiles; ++j) {
                    // an odd count of column tiles leaves the last warp's second tile empty: it re-reads the first
                    const int ct = min(kColTiles * warp + j, col_tiles - 1);
                    xcol[j] = xst + (size_t)(8 * ct + g) * kPlane + 8 * t;
                }
                if (uniform_type == kQ4_K) mma_q4k<RT, false>(wst, tile_stride, qd, 0, xcol, lane, g, acc);
                else if (uniform_type == kQ6_K) mma_q6k<RT, false>(wst, tile_stride, qd, 0, xcol, lane, g, acc);
                else if (uniform_type == kQ8_0) mma_q8_0<RT, false>(wst, tile_stride, qd, 0, xcol, lane, g, acc);
                else {
                    if (mask_q4k) mma_q4k<RT, true>(wst, tile_stride, qd, mask_q4k, xcol, lane, g, acc);
                    if (mask_q6k) mma_q6k<RT, true>(wst, tile_stride, qd, mask_q6k, xcol, lane, g, acc);
                    if (mask_q8) mma_q8_0<RT, true>(wst, tile_stride, qd, mask_q8, xcol, lane, g, acc);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * b);
        }
    }
    __syncthreads();  // every copy has landed and every warp has left the stages

    // Accumulators and offset totals meet in shared memory (the stages are free now).
    float* exch = reinterpret_cast<float*>(smem);                  // [(RT * 16)][kExchStride]: column 3 m + digit
    float* offx = exch + (RT * 16) * kExchStride;                   // [(RT * 16)][kOffStride]
    if (warp < kWarps) {
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int j = 0; j < kColTiles; ++j) {
                const int ct = kColTiles * warp + j;
                if (ct < col_tiles) {
                    float* e = exch + (size_t)(r * 16 + g) * kExchStride + 8 * ct + 2 * t;
                    e[0] = acc[r][j][0]; e[1] = acc[r][j][1];
                    e[8 * kExchStride] = acc[r][j][2]; e[8 * kExchStride + 1] = acc[r][j][3];
                }
            }
    }
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const int group = warp + p * kWarps;
        if (warp >= kWarps || group >= (RT * 16) / 4) break;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            offx[(4 * group + i) * kOffStride + lane] = off[p][i][0];
            offx[(4 * group + i) * kOffStride + lane + 32] = off[p][i][1];
        }
    }
    __syncthreads();

    // Epilogue: consecutive threads take consecutive output rows of one member.
    const int out_rows = swiglu ? (RT * 16) / 2 : (RT * 16);
    for (int idx = threadIdx.x; idx < out_rows * a.members; idx += kThreads) {
        const int m = idx / out_rows, o = idx % out_rows;
        // SwiGLU: output row o of the unit is gate row (o / 16) * 32 + o % 16 of the CTA, its up row 16 further
        const int row = swiglu ? (o >> 4) * 32 + (o & 15) : o;
        const GemvSegment& s = a.seg[swiglu ? 0 : seg];
        const int n_index = unit * out_rows + o;
        if (n_index >= s.n) continue;
        const float mult = a.member_scale[m];
        auto value = [&](int rr) {
            const float* e = exch + (size_t)rr * kExchStride + 3 * m;
            return (e[0] + e[1] * (1.0f / 128.0f) + e[2] * (1.0f / 16384.0f) + offx[rr * kOffStride + m]) * mult;
        };
        const float v = value(row);
        float* y = s.y + (size_t)m * s.n + n_index;
        if (swiglu) {
            const float u = value(row + 16);
            *y = v / (1.0f + expf(-v)) * u;
        } else if (a.epilogue == kResidual) {
            *y += v;
        } else {
            *y = v;
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

// Pass 2: digits and per-16 digit sums, one chunk per k tile:
// [member][digit][kBatchPlaneBytes] digits, then [sub / 4][member][sub % 4] F32 sums.
__global__ void batch_digits_kernel(const float* x, const int32_t* index, const float* norm_weight, int members,
                                    int members_padded, int k, const float* digit_inv, signed char* chunks) {
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
    const size_t digit_bytes = (size_t)members_padded * 3 * kPlane, chunk_bytes = digit_bytes + (size_t)members_padded * 64;
    signed char* chunk = chunks + (size_t)kt * chunk_bytes;
    signed char* base = chunk + ((size_t)m * 3) * kPlane + operand_position(in_tile);
    base[0] = (signed char)(int)f1;
    base[kPlane] = (signed char)(int)f2;
    base[2 * kPlane] = (signed char)(int)f3;
    if ((lane & 15) == 0) {
        const int sub = in_tile >> 4;
        reinterpret_cast<float*>(chunk + digit_bytes)[((size_t)(sub >> 2) * members_padded + m) * 4 + (sub & 3)] = value;
    }
}

size_t exchange_bytes(int row_tiles) { return (size_t)row_tiles * 16 * (kExchStride + kOffStride) * 4; }

StageLayout layout_for(const GemmArgs& a, int row_tiles) {
    StageLayout l{};
    int tile = 0;
    for (int i = 0; i < a.n_segments; ++i) tile = std::max(tile, packed_tile_bytes(a.seg[i].type));
    const int members_padded = (a.members + kMemberPad - 1) / kMemberPad * kMemberPad;
    l.w_bytes = row_tiles * tile;
    l.x_bytes = members_padded * 3 * kPlane;
    l.s_bytes = members_padded * 16 * 4;
    l.stage_bytes = (l.w_bytes + l.x_bytes + l.s_bytes + 127) / 128 * 128;
    // the epilogue's exchange arrays reuse the two stages
    const int exchange = (int)exchange_bytes(row_tiles);
    if (2 * l.stage_bytes < exchange) l.stage_bytes = (exchange / 2 + 127) / 128 * 128;
    return l;
}

size_t smem_for(const StageLayout& lay, int row_tiles) {
    return (size_t)2 * lay.stage_bytes + (size_t)2 * (row_tiles * kQuadFloats + row_tiles * 16 * kCoefStride) * 4 + 64;
}

}  // namespace

size_t batch_operand_bytes(int members, int k) {
    const int mp = (members + kMemberPad - 1) / kMemberPad * kMemberPad;
    return (size_t)(k / 256) * mp * (3 * kPlane + 64);
}

cudaError_t launch_to_batch_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                                    int members, int k, float eps, BatchOperand out) {
    if (members <= 0 || members > kMaxMembers || k % 256 != 0) return cudaErrorInvalidValue;
    const int mp = (members + kMemberPad - 1) / kMemberPad * kMemberPad;
    batch_scale_kernel<<<members, 256, 0, stream>>>(x, index, norm_weight, k, eps, out.digit_inv, out.member_scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const long long warps = (long long)mp * (k / 32);
    batch_digits_kernel<<<(unsigned int)((warps + 7) / 8), 256, 0, stream>>>(x, index, norm_weight, members, mp, k,
                                                                           out.digit_inv, out.chunks);
    return cudaGetLastError();
}

namespace {

int units_for(const GemmArgs& args, int row_tiles) {
    if (args.epilogue == kSwiGLU) return (args.seg[0].row_tiles + row_tiles / 2 - 1) / (row_tiles / 2);
    int units = 0;
    for (int i = 0; i < args.n_segments; ++i) units += (args.seg[i].row_tiles + row_tiles - 1) / row_tiles;
    return units;
}

template <int RT>
cudaError_t launch_rt(cudaStream_t stream, const GemmArgs& args, int units) {
    const StageLayout lay = layout_for(args, RT);
    const size_t smem = smem_for(lay, RT);
    static bool configured[kMaxDevices] = {false};  // function attributes are per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_imma_kernel<RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    gemm_imma_kernel<RT><<<units, kThreads, smem, stream>>>(args, lay);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm_imma(cudaStream_t stream, const GemmArgs& args) {
    if (args.members < 1 || args.members > kMaxMembers || args.k % kTileCols != 0) return cudaErrorInvalidValue;
    if (args.epilogue == kSwiGLU && (args.n_segments != 2 || args.seg[0].row_tiles != args.seg[1].row_tiles)) {
        return cudaErrorInvalidValue;
    }
    static int sm_counts[kMaxDevices] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (sm_counts[dev] == 0) {
        if (cudaDeviceGetAttribute(&sm_counts[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_counts[dev] <= 0) sm_counts[dev] = 148;
    }
    const int sm_count = sm_counts[dev];
    const int units4 = units_for(args, 4);
    if (units4 <= 0) return cudaSuccess;
    // Four row tiles per CTA reuse each activation chunk most; when that leaves SMs idle and half-size
    // CTAs still fit in one wave, two row tiles per CTA finish sooner.
    const int units2 = units_for(args, 2);
    if (units4 < sm_count && units2 <= sm_count) return launch_rt<2>(stream, args, units2);
    return launch_rt<4>(stream, args, units4);
}

}  // namespace ribn
