// Dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for batches of 3..128 rows:
// chunked prefill and batched decode.
//
//   y[m][n] = sum_k deq(W[n][k]) x[m][k]
//
// The weights stay in their tile-major GGUF repack (16 rows x 256 inputs per tile).  A CTA owns
// 128 output rows at a time and walks K:
//   * a producer warp brings the 8 packed tiles of a k tile (bulk copies) and, per 64 inputs, the
//     activations' operand chunk into shared-memory rings;
//   * eight dequant warps decode the blocks with the reference's own arithmetic
//     (w = fl(fl(d * sc) * q) - fl(dmin * m) for Q4_K, two products for Q6_K, one for Q8_0) and split
//     every F32 weight into two binary16 numbers hi + lo (22 significant bits), stored in the
//     K-major core-matrix layout `tcgen05.mma` reads;
//   * one thread issues `tcgen05.mma.kind::f16`: hi x [x_hi | x_lo] and lo x x_hi, F32 accumulation
//     over the whole K in tensor memory (activations are likewise hi + lo pairs scaled per row by a
//     power of two, so no product or sum is rounded below F32);
//   * four epilogue warps read the accumulators back with `tcgen05.ld`, add the two column halves,
//     apply the row scale (and RMSNorm factor) and store or add into the residual stream, while
//     the next 128 rows already accumulate in the other half of tensor memory.
// Every column (batch row) is computed independently of the others and every sum has a fixed
// order: a row's result does not depend on what it is batched with.  All waits are bounded and
// raise the caller's error word.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "blocks.cuh"
#include "gemv.cuh"

namespace ribn {

namespace {

constexpr int kRows = 128;                 // output rows per unit (UMMA M)
constexpr int kRowTilesPerUnit = kRows / kTileRows;
constexpr int kChunkK = 64;                // inputs per operand chunk
constexpr int kChunksPerTile = kTileCols / kChunkK;
constexpr int kEpilogueWarps = 4;          // warps 0..3: TMEM lane quadrant = warp index
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kDequantWarp0 = 6;
constexpr int kDequantWarps = 2 * kRowTilesPerUnit;  // two per row tile: rows g and rows g + 8 of the MMA-fragment order
constexpr int kThreads = (kDequantWarp0 + kDequantWarps) * 32;
constexpr int kAHalfBytes = kRows * kChunkK * 2;   // one of hi / lo for a chunk: 16 KB
constexpr int kABytes = 2 * kAHalfBytes;
constexpr int kALbo = (kRows / 8) * 128;           // bytes between the 8-input column blocks of A
constexpr int kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 22;   // bounded waits: default number of polls before giving up

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
// Bounded wait; on expiry raises the error word and reports false (the caller stops waiting but
// keeps arriving, so nobody else is left hanging on it).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (error_flag != nullptr) atomicExch(error_flag, code);
    return false;
}
// The same for waits that usually last microseconds (a whole K loop, a ring turn): sleeps between
// polls so the waiting warp does not take issue slots from the dequant warps.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, int* error_flag, int code, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(100);
    }
    if (error_flag != nullptr) atomicExch(error_flag, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// ---- tcgen05 ---------------------------------------------------------------------------------
// Shared-memory operand descriptor, K-major, no swizzle: 8 rows x 16 bytes core matrices; `lbo` =
// bytes between the two 8-element column blocks of one MMA's K = 16, `sbo` = bytes between
// successive groups of 8 rows.  Bits 46..47 carry the descriptor version (1).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// Instruction descriptor for kind::f16: F32 accumulate, F16 x F16, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- dequant to hi + lo binary16 ---------------------------------------------------------------
// Four consecutive inputs of one row: 8 bytes into the hi plane and 8 into the lo plane.
// hi = w with its significand cut to 11 bits (exact in binary16), lo = w - hi rounded to binary16.
__device__ __forceinline__ void store_split4(unsigned char* hi, float w0, float w1, float w2, float w3) {
    const float h0 = __uint_as_float(__float_as_uint(w0) & 0xFFFFE000u), h1 = __uint_as_float(__float_as_uint(w1) & 0xFFFFE000u);
    const float h2 = __uint_as_float(__float_as_uint(w2) & 0xFFFFE000u), h3 = __uint_as_float(__float_as_uint(w3) & 0xFFFFE000u);
    const __half2 h01 = __floats2half2_rn(h0, h1), h23 = __floats2half2_rn(h2, h3);
    const __half2 l01 = __floats2half2_rn(w0 - h0, w1 - h1), l23 = __floats2half2_rn(w2 - h2, w3 - h3);
    uint2 a, b;
    a.x = *reinterpret_cast<const uint32_t*>(&h01); a.y = *reinterpret_cast<const uint32_t*>(&h23);
    b.x = *reinterpret_cast<const uint32_t*>(&l01); b.y = *reinterpret_cast<const uint32_t*>(&l23);
    *reinterpret_cast<uint2*>(hi) = a;
    *reinterpret_cast<uint2*>(hi + kAHalfBytes) = b;
}
// Small unsigned integer (< 2^23) to float without the conversion pipe.
__device__ __forceinline__ float small_uint_f32(uint32_t v) { return __uint_as_float(v | 0x4B000000u) - 8388608.0f; }
// Byte offset inside a hi (or lo) plane of input k0 (multiple of 4) of row `r` of the unit.
__device__ __forceinline__ int a_offset(int r, int k0) { return (k0 >> 3) * kALbo + (r >> 3) * 128 + (r & 7) * 16 + (k0 & 7) * 2; }

__device__ __forceinline__ float byte_of(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xffu); }

// One 64-input chunk `c` of one packed tile, decoded with the reference's arithmetic: lane (g, t) holds rows g and
// g + 8 of the tile (`rr` selects which) in the byte order of the GEMV kernel's MMA fragments, and hands
// `emit(row, k, w0, w1, w2, w3)` the four consecutive weights k .. k + 3 (k inside the chunk) of tile row `row`.
template <typename Emit>
__device__ __forceinline__ void decode_chunk(int type, const unsigned char* tile, int c, int rr, int lane, Emit emit) {
    const int g = lane >> 2, t = lane & 3;
    const int row = g + 8 * rr;
    if (type == kQ4_K) {
        const uint4 w = *reinterpret_cast<const uint4*>(tile + c * 512 + lane * 16);
        const uint4 h = *reinterpret_cast<const uint4*>(tile + 2048 + row * 16);
        const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        const uint32_t sc4 = c < 2 ? (h.y & 0x3F3F3F3Fu) : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
        const uint32_t mn4 = c < 2 ? (h.z & 0x3F3F3F3Fu) : (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u));
        const int b0 = (2 * c) & 3;  // byte of the even group inside its half
        const float gs_e = __fmul_rn(d, byte_of(sc4, b0)), gs_o = __fmul_rn(d, byte_of(sc4, b0 + 1));
        const float gm_e = __fmul_rn(dmin, byte_of(mn4, b0)), gm_o = __fmul_rn(dmin, byte_of(mn4, b0 + 1));
        // fl(gs * q) from the integer's float pattern 2^23 + q in one fused step: gs * 2^23 is exact,
        // so fma(gs, 2^23 + q, -(gs * 2^23)) rounds the exact product gs * q once, as the multiplication does.
        const float ce = -(gs_e * 8388608.0f), co = -(gs_o * 8388608.0f);
        const uint32_t lo16 = rr == 0 ? w.x : w.z, hi16 = rr == 0 ? w.y : w.w;  // inputs 4t.. and 16 + 4t.. of both groups
#pragma unroll
        for (int part = 0; part < 2; ++part) {
            const uint32_t word = part == 0 ? lo16 : hi16;
            float e[4], o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float fe = __uint_as_float(((word >> (8 * i)) & 15u) | 0x4B000000u);
                const float fo = __uint_as_float(((word >> (8 * i + 4)) & 15u) | 0x4B000000u);
                e[i] = __fsub_rn(__fmaf_rn(gs_e, fe, ce), gm_e);
                o[i] = __fsub_rn(__fmaf_rn(gs_o, fo, co), gm_o);
            }
            const int k_e = part * 16 + 4 * t, k_o = 32 + part * 16 + 4 * t;
            emit(row, k_e, e[0], e[1], e[2], e[3]);
            emit(row, k_o, o[0], o[1], o[2], o[3]);
        }
    } else if (type == kQ6_K) {
        // chunk c covers groups 2c, 2c + 1: super-half cc = c / 2, variants v = 2 (c % 2), + 1
        const int cc = c >> 1, v0 = (c & 1) * 2;
        const uint4 qh = *reinterpret_cast<const uint4*>(tile + 2048 + cc * 512 + lane * 16);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 w = *reinterpret_cast<const uint4*>(tile + (cc * 2 + h) * 512 + lane * 16);
            const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(tile + 3328 + row * 2)));
            const signed char* scales = reinterpret_cast<const signed char*>(tile + 3072 + row * 16);
            const uint32_t high = rr == 0 ? (h == 0 ? qh.x : qh.z) : (h == 0 ? qh.y : qh.w);
#pragma unroll
            for (int vv = 0; vv < 2; ++vv) {
                const int v = v0 + vv, group = cc * 4 + v;
                const uint32_t low = rr == 0 ? ((v & 1) ? w.y : w.x) : ((v & 1) ? w.w : w.z);
                const float gs = __fmul_rn(d, (float)scales[group * 2 + h]);
                float q[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t lb = (low >> (8 * i)) & 0xffu, hb = (high >> (8 * i)) & 0xffu;
                    const uint32_t nib = v < 2 ? (lb & 15u) : (lb >> 4);
                    q[i] = __fmul_rn(gs, small_uint_f32(nib | (((hb >> (2 * v)) & 3u) << 4)) - 32.0f);
                }
                emit(row, vv * 32 + h * 16 + 4 * t, q[0], q[1], q[2], q[3]);
            }
        }
    } else {
        // Q8_0: chunk c covers blocks 2c, 2c + 1; stored byte = q + 128
#pragma unroll
        for (int bb = 0; bb < 2; ++bb) {
            const int block = 2 * c + bb;
            const uint4 w = *reinterpret_cast<const uint4*>(tile + block * 512 + lane * 16);
            const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(tile + 4096 + row * 16 + block * 2)));
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                const uint32_t word = rr == 0 ? (part == 0 ? w.x : w.y) : (part == 0 ? w.z : w.w);
                float q[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) q[i] = __fmul_rn(d, small_uint_f32((word >> (8 * i)) & 0xffu) - 128.0f);
                emit(row, bb * 32 + part * 16 + 4 * t, q[0], q[1], q[2], q[3]);
            }
        }
    }
}

// The same chunk -> rows [row0, row0 + 16) of the A operand chunk, as binary16 hi + lo planes.
__device__ __forceinline__ void dequant_chunk(int type, const unsigned char* tile, int c, unsigned char* a_hi, int row0, int rr, int lane) {
    decode_chunk(type, tile, c, rr, lane, [&](int row, int k, float w0, float w1, float w2, float w3) {
        store_split4(a_hi + a_offset(row0 + row, 0) + (k >> 3) * kALbo + (k & 7) * 2, w0, w1, w2, w3);
    });
}

// Packed tiles -> F32 [rows][cols], through decode_chunk: what the tensor-core kernels see of a repacked matrix.
__global__ void unpack_packed_kernel(int type, const unsigned char* packed, long long rows, int k_tiles, float* out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;   // 8 warps: (chunk c, row half rr)
    const long long tile_index = blockIdx.x;                      // row tile * k_tiles + k tile
    const long long rt = tile_index / k_tiles;
    const int kb = (int)(tile_index % k_tiles);
    const unsigned char* tile = packed + (size_t)tile_index * packed_tile_bytes(type);
    const long long cols = (long long)k_tiles * kTileCols;
    decode_chunk(type, tile, warp >> 1, warp & 1, lane, [&](int row, int k, float w0, float w1, float w2, float w3) {
        const long long r = rt * kTileRows + row;
        if (r < rows) {
            float* dst = out + r * cols + (long long)kb * kTileCols + (warp >> 1) * kChunkK + k;
            dst[0] = w0; dst[1] = w1; dst[2] = w2; dst[3] = w3;
        }
    });
}

// Rows [row0, row0 + 8) of both planes: 8 column blocks x 128 bytes per plane.
__device__ __forceinline__ void zero_rows(unsigned char* a_hi, int row0, int lane) {
    for (int i = lane; i < 2 * 8 * 8; i += 32) {
        const int plane = i >> 6, kblock = (i >> 3) & 7, q16 = i & 7;
        *reinterpret_cast<uint4*>(a_hi + plane * kAHalfBytes + kblock * kALbo + (row0 >> 3) * 128 + q16 * 16) =
            make_uint4(0u, 0u, 0u, 0u);
    }
}

// Rows [row0, row0 + 8) of one plane.
__device__ __forceinline__ void zero_rows_plane(unsigned char* plane, int row0, int lane) {
    for (int i = lane; i < 8 * 8; i += 32) {
        *reinterpret_cast<uint4*>(plane + (i >> 3) * kALbo + (row0 >> 3) * 128 + (i & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
}

struct TcLayout {
    int w_stage_bytes, w_stages, b_bytes, b_stages;  // per stage / per chunk
    int cols;                              // MMA N of the first product: 2 * padded members
    int members_padded;
};

// Work list shared by all roles: unit u of the launch -> segment, first row tile.
struct UnitRef { int seg, rt0; };
__device__ __forceinline__ UnitRef unit_of(const GemmArgs& a, int u) {
    UnitRef r{0, u * kRowTilesPerUnit};
    while (r.seg + 1 < a.n_segments) {
        const int units = (a.seg[r.seg].row_tiles + kRowTilesPerUnit - 1) / kRowTilesPerUnit;
        if (r.rt0 < units * kRowTilesPerUnit) break;
        r.rt0 -= units * kRowTilesPerUnit;
        ++r.seg;
    }
    return r;
}

__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const GemmArgs a, const TcLayout lay, const int units) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = a.k / kTileCols;
    const uint32_t spin_limit = a.spin_limit ? a.spin_limit : kSpinLimit;
    unsigned char* w_ring = smem;
    unsigned char* a_buf = w_ring + (size_t)lay.w_stages * lay.w_stage_bytes;   // [2][hi | lo]
    unsigned char* b_buf = a_buf + 2 * kABytes;                                  // [b_stages][b_bytes]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_buf + (size_t)lay.b_stages * lay.b_bytes);
    const uint32_t bars = smem_u32(tmem_slot + 4);
    const uint32_t w_full = bars, w_empty = bars + 32, a_full = bars + 64, a_empty = bars + 80, t_full = bars + 96,
                   t_empty = bars + 112, b_full = bars + 128, b_empty = bars + 192;

    if (threadIdx.x == 0) {
        for (int i = 0; i < lay.w_stages; ++i) { mbar_init(w_full + 8 * i, 1); mbar_init(w_empty + 8 * i, kDequantWarps); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(a_full + 8 * i, kDequantWarps);
            mbar_init(a_empty + 8 * i, 1);
            mbar_init(t_full + 8 * i, 1);
            mbar_init(t_empty + 8 * i, kEpilogueWarps);
        }
        for (int i = 0; i < lay.b_stages; ++i) { mbar_init(b_full + 8 * i, 1); mbar_init(b_empty + 8 * i, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const int acc_cols = kTmemCols / 2;  // two accumulator buffers

    if (warp == kProducerWarp) {
        // ---------------- copies: packed weight tiles two k tiles ahead, one activation chunk at a time ----------------
        bool alive = true;
        uint32_t w_count = 0, b_count = 0;
        // position of the next weight stage to issue
        int wu = blockIdx.x, wkb = 0;
        auto issue_w = [&]() {
            if (wu >= units) return;
            const UnitRef ur = unit_of(a, wu);
            const GemvSegment& s = a.seg[ur.seg];
            const uint32_t tb = (uint32_t)packed_tile_bytes(s.type);
            const uint32_t stage = w_count % (uint32_t)lay.w_stages;
            if (lane == 0) {
                if (w_count >= (uint32_t)lay.w_stages && alive) {
                    alive = mbar_wait_relaxed(w_empty + 8 * stage, ((w_count / (uint32_t)lay.w_stages) - 1u) & 1u, a.error_flag, 11, spin_limit);
                }
                const int present = min(kRowTilesPerUnit, s.row_tiles - ur.rt0);
                mbar_expect_tx(w_full + 8 * stage, (uint32_t)present * tb);
            }
            __syncwarp();
            if (lane < kRowTilesPerUnit && ur.rt0 + lane < s.row_tiles) {
                bulk_g2s(smem_u32(w_ring + (size_t)stage * lay.w_stage_bytes + (size_t)lane * tb),
                         s.data + ((size_t)(ur.rt0 + lane) * k_tiles + wkb) * tb, tb, w_full + 8 * stage);
            }
            ++w_count;
            if (++wkb == k_tiles) { wkb = 0; wu += gridDim.x; }
        };
        issue_w();
        if (lay.w_stages > 2) issue_w();
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            for (int kb = 0; kb < k_tiles; ++kb) {
                if (lane == 0) {
                    for (int c = 0; c < kChunksPerTile; ++c, ++b_count) {
                        const uint32_t nb = (uint32_t)lay.b_stages, bs = b_count % nb;
                        if (b_count >= nb && alive) alive = mbar_wait_relaxed(b_empty + 8 * bs, ((b_count / nb) - 1u) & 1u, a.error_flag, 12, spin_limit);
                        mbar_expect_tx(b_full + 8 * bs, (uint32_t)lay.b_bytes);
                        bulk_g2s(smem_u32(b_buf + (size_t)bs * lay.b_bytes),
                                 a.chunks + ((size_t)kb * kChunksPerTile + c) * lay.b_bytes, (uint32_t)lay.b_bytes, b_full + 8 * bs);
                    }
                }
                __syncwarp();
                issue_w();
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issue (one thread) ----------------
        if (lane == 0) {
            bool alive = true;
            uint32_t count = 0, unit_count = 0;
            const uint32_t idesc_full = umma_idesc(lay.cols), idesc_half = umma_idesc(lay.members_padded);
            const uint32_t b_lbo = (uint32_t)(lay.cols / 8) * 128u;
            for (int u = blockIdx.x; u < units; u += gridDim.x, ++unit_count) {
                const uint32_t tb = unit_count & 1u;
                if (unit_count >= 2u && alive) alive = mbar_wait_relaxed(t_empty + 8 * tb, ((unit_count >> 1) - 1u) & 1u, a.error_flag, 13, spin_limit);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + tb * (uint32_t)acc_cols;
                for (int kc = 0; kc < k_tiles * kChunksPerTile; ++kc, ++count) {
                    const uint32_t st = count & 1u, parity = (count >> 1) & 1u;
                    const uint32_t nb = (uint32_t)lay.b_stages, bs = count % nb;
                    if (alive) alive = mbar_wait(a_full + 8 * st, parity, a.error_flag, 14, spin_limit);
                    if (alive) alive = mbar_wait(b_full + 8 * bs, (count / nb) & 1u, a.error_flag, 15, spin_limit);
                    tc_fence_after();
                    const uint32_t a_hi = smem_u32(a_buf + (size_t)st * kABytes), a_lo = a_hi + kAHalfBytes;
                    const uint32_t b_addr = smem_u32(b_buf + (size_t)bs * lay.b_bytes);
#pragma unroll
                    for (int s16 = 0; s16 < kChunkK / 16; ++s16) {
                        const uint64_t da_hi = umma_desc(a_hi + s16 * 2 * kALbo, kALbo, 128);
                        const uint64_t da_lo = umma_desc(a_lo + s16 * 2 * kALbo, kALbo, 128);
                        const uint64_t db = umma_desc(b_addr + s16 * 2 * b_lbo, b_lbo, 128);
                        umma_f16(d_tmem, da_hi, db, idesc_full, (kc | s16) != 0 ? 1u : 0u);   // hi x [x_hi | x_lo]
                        umma_f16(d_tmem, da_lo, db, idesc_half, 1u);                          // lo x x_hi
                    }
                    umma_commit(a_empty + 8 * st);   // arrive when these MMAs have read the buffers
                    umma_commit(b_empty + 8 * bs);
                }
                umma_commit(t_full + 8 * tb);        // ... and when the unit's accumulators are complete
            }
        }
    } else if (warp >= kDequantWarp0) {
        // ---------------- dequant: warps 2 i, 2 i + 1 decode rows g and g + 8 of row tile i of the unit ----------------
        const int rt_local = (warp - kDequantWarp0) >> 1, rr = (warp - kDequantWarp0) & 1;
        bool alive = true;
        uint32_t w_count = 0, a_count = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            const UnitRef ur = unit_of(a, u);
            const GemvSegment& s = a.seg[ur.seg];
            const int type = s.type;
            const bool present = ur.rt0 + rt_local < s.row_tiles;
            const int tb = packed_tile_bytes(type);
            for (int kb = 0; kb < k_tiles; ++kb, ++w_count) {
                const uint32_t stage = w_count % (uint32_t)lay.w_stages;
                if (alive) alive = mbar_wait(w_full + 8 * stage, (w_count / (uint32_t)lay.w_stages) & 1u, a.error_flag, 16, spin_limit);
                const unsigned char* tile = w_ring + (size_t)stage * lay.w_stage_bytes + (size_t)rt_local * tb;
                for (int c = 0; c < kChunksPerTile; ++c, ++a_count) {
                    const uint32_t st = a_count & 1u;
                    if (a_count >= 2u && alive) alive = mbar_wait(a_empty + 8 * st, ((a_count >> 1) - 1u) & 1u, a.error_flag, 17, spin_limit);
                    unsigned char* a_hi = a_buf + (size_t)st * kABytes;
                    if (present) dequant_chunk(type, tile, c, a_hi, rt_local * kTileRows, rr, lane);
                    else zero_rows(a_hi, rt_local * kTileRows + 8 * rr, lane);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic stores -> tensor-core reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(a_full + 8 * st);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(w_empty + 8 * stage);
            }
        }
    } else {
        // ---------------- epilogue: warp q reads TMEM lanes 32 q .. 32 q + 31 (one output row per thread) ----------------
        bool alive = true;
        uint32_t unit_count = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++unit_count) {
            const uint32_t tb = unit_count & 1u;
            const UnitRef ur = unit_of(a, u);
            const GemvSegment& s = a.seg[ur.seg];
            if (alive) alive = mbar_wait_relaxed(t_full + 8 * tb, (unit_count >> 1) & 1u, a.error_flag, 18, spin_limit);
            tc_fence_after();
            const int n_index = ur.rt0 * kTileRows + warp * 32 + lane;
            const bool valid = n_index < s.n;
            const uint32_t taddr = tmem_base + tb * (uint32_t)acc_cols + ((uint32_t)(warp * 32) << 16);
            for (int m0 = 0; m0 < lay.members_padded; m0 += 16) {
                float hi[16], lo[16];
                tmem_ld16(taddr + (uint32_t)m0, hi);
                tmem_ld16(taddr + (uint32_t)(lay.members_padded + m0), lo);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int m = m0 + i;
                    if (valid && m < a.members) {
                        const float v = (hi[i] + lo[i]) * a.member_scale[m];
                        float* y = s.y + (size_t)m * s.n + n_index;
                        if (a.epilogue == kResidual) *y += v; else *y = v;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(t_empty + 8 * tb);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// =====================================================================================================
// K-quant form (Q4_K, Q6_K; up to 64 members): the tensor core multiplies exact small integers.
//
// Q4_K:  w = d * (sc * q) - dmin * m      sc, m 6-bit and q 4-bit integers, d and dmin one binary16
// Q6_K:  w = d * (sc * (q - 32))          sc 8-bit, q 6-bit                   pair per row and 256 inputs
//
// The A operand is the integer sc * q (at most 945, exact in binary16), made from the packed nibbles
// with two instructions per pair of weights (byte permute into the pattern 1024 + q, one fused
// multiply-add).  For Q6_K sc * (q - 32) can reach 4096, so sc = 16 sh + sl is split into two exact
// planes, sl * v and (16 sh) * v, accumulated into the same tensor-memory columns.  The Q4_K minimum
// enters as one more K = 16 MMA per 256 inputs: the eight group minima m against the eight group sums
// of the activations.  Tensor memory then holds, per 256 inputs, exact-integer-weighted sums; four
// epilogue warps fold them into F32 registers with the row's d (and dmin) once per k tile, in order,
// with round-to-nearest FMAs - so the only roundings below F32 are the activations' hi + lo split.
constexpr int kKqMaxMembers = 64;
constexpr int kKqDequantWarps = kRowTilesPerUnit;   // one per row tile (the operand conversion is cheap)
constexpr int kKqChunkWarp0 = kDequantWarp0 + kKqDequantWarps;   // two warps that only copy activation chunks
constexpr int kKqThreads = (kKqChunkWarp0 + 2) * 32;
constexpr int kA2Bytes = kRows * 16 * 2;   // the minima operand: 128 rows x 16 (8 groups + 8 zeros) halves

struct KqLayout {
    int w_stage_bytes, w_stages, b_bytes, b2_bytes;
    int cols, members_padded, a_stages, a_planes, chunk_k;
    int k_slices, total_n;                 // split-K: slices per unit, and the rows of all segments together
    int groups;                            // row groups per launch (work items: unit, then group, then K slice)
    size_t group_bytes;                    // bytes between the operands of consecutive groups
};

// 4 bytes (each < 64) -> the binary16 pairs (1024 + b0, 1024 + b1) and (1024 + b2, 1024 + b3)
__device__ __forceinline__ void bytes_to_half_pairs(uint32_t b, __half2& p01, __half2& p23) {
    const uint32_t x = __byte_perm(b, 0x64646464u, 0x4140), y = __byte_perm(b, 0x64646464u, 0x4342);
    p01 = *reinterpret_cast<const __half2*>(&x);
    p23 = *reinterpret_cast<const __half2*>(&y);
}
__device__ __forceinline__ void store_half4(unsigned char* dst, __half2 a, __half2 b) {
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&a);
    v.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(dst) = v;
}

// One 64-input piece `c` of one packed tile for the row g + 8 rr of each lane -> integer operand planes.
// At piece 0 the lane with t == 0 also leaves the row's d (and dmin) in `row_scales` and, for Q4_K,
// lanes t = 0..3 write the row's eight group minima into the A2 operand.
__device__ __forceinline__ void kq_chunk(int type, const unsigned char* tile, int c, int k_base, unsigned char* a_planes,
                                         unsigned char* a2, float2* row_scales, int row0, int rr, int lane) {
    const int g = lane >> 2, t = lane & 3, row = g + 8 * rr, unit_row = row0 + row;
    // k_base: where this 64-input piece sits inside the operand stage (stages hold 64 or 128 inputs)
    unsigned char* base = a_planes + (k_base >> 3) * kALbo + (unit_row >> 3) * 128 + (unit_row & 7) * 16;
    if (type == kQ4_K) {
        const uint4 w = *reinterpret_cast<const uint4*>(tile + c * 512 + lane * 16);
        const uint4 h = *reinterpret_cast<const uint4*>(tile + 2048 + row * 16);
        const uint32_t sc4 = c < 2 ? (h.y & 0x3F3F3F3Fu) : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
        const int b0 = (2 * c) & 3;
        const float sce = (float)((sc4 >> (8 * b0)) & 0xffu), sco = (float)((sc4 >> (8 * b0 + 8)) & 0xffu);
        const __half2 se = __float2half2_rn(sce), so = __float2half2_rn(sco);
        const __half2 be = __float2half2_rn(-1024.0f * sce), bo = __float2half2_rn(-1024.0f * sco);
        if (c == 0) {
            if (t == 0) {
                row_scales[unit_row] = make_float2(__half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu))),
                                                   __half2float(__ushort_as_half((unsigned short)(h.x >> 16))));
            }
            // minima of groups 2 t, 2 t + 1 as binary16, into the first 8-input block of A2
            const uint32_t mlo = h.z & 0x3F3F3F3Fu, mhi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
            const uint32_t m4 = t < 2 ? mlo : mhi;
            const int mb = (2 * t) & 3;
            const __half2 mm = __floats2half2_rn((float)((m4 >> (8 * mb)) & 0xffu), (float)((m4 >> (8 * mb + 8)) & 0xffu));
            *reinterpret_cast<__half2*>(a2 + (unit_row >> 3) * 128 + (unit_row & 7) * 16 + 4 * t) = mm;
        }
        const uint32_t lo16 = rr == 0 ? w.x : w.z, hi16 = rr == 0 ? w.y : w.w;
#pragma unroll
        for (int part = 0; part < 2; ++part) {
            const uint32_t word = part == 0 ? lo16 : hi16;
            __half2 e01, e23, o01, o23;
            bytes_to_half_pairs(word & 0x0F0F0F0Fu, e01, e23);
            bytes_to_half_pairs((word >> 4) & 0x0F0F0F0Fu, o01, o23);
            const int k_e = part * 16 + 4 * t, k_o = 32 + k_e;
            store_half4(base + (k_e >> 3) * kALbo + (k_e & 7) * 2, __hfma2(e01, se, be), __hfma2(e23, se, be));
            store_half4(base + (k_o >> 3) * kALbo + (k_o & 7) * 2, __hfma2(o01, so, bo), __hfma2(o23, so, bo));
        }
    } else {
        const int cc = c >> 1, v0 = (c & 1) * 2;
        const uint4 qh = *reinterpret_cast<const uint4*>(tile + 2048 + cc * 512 + lane * 16);
        const signed char* scales = reinterpret_cast<const signed char*>(tile + 3072 + row * 16);
        if (c == 0 && t == 0) {
            row_scales[unit_row] = make_float2(__half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(tile + 3328 + row * 2))), 0.0f);
        }
        const __half2 bias = __float2half2_rn(1056.0f);  // 1024 + 32
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 w = *reinterpret_cast<const uint4*>(tile + (cc * 2 + h) * 512 + lane * 16);
            const uint32_t high = rr == 0 ? (h == 0 ? qh.x : qh.z) : (h == 0 ? qh.y : qh.w);
#pragma unroll
            for (int vv = 0; vv < 2; ++vv) {
                const int v = v0 + vv, group = cc * 4 + v;
                const uint32_t low = rr == 0 ? ((v & 1) ? w.y : w.x) : ((v & 1) ? w.w : w.z);
                const uint32_t q4 = ((v < 2 ? low : low >> 4) & 0x0F0F0F0Fu) | (((high >> (2 * v)) & 0x03030303u) << 4);
                const int sc = scales[group * 2 + h];
                const __half2 sl = __float2half2_rn((float)(sc & 15)), sh = __float2half2_rn((float)((sc >> 4) * 16));
                __half2 p01, p23;
                bytes_to_half_pairs(q4, p01, p23);
                const __half2 v01 = __hsub2(p01, bias), v23 = __hsub2(p23, bias);
                const int k = vv * 32 + h * 16 + 4 * t;
                unsigned char* dst = base + (k >> 3) * kALbo + (k & 7) * 2;
                store_half4(dst, __hmul2(v01, sl), __hmul2(v23, sl));
                store_half4(dst + kAHalfBytes, __hmul2(v01, sh), __hmul2(v23, sh));
            }
        }
    }
}

// The Q4_K form of kq_chunk for a whole 128-input operand stage (64-input pieces 2 c and 2 c + 1, both row halves
// of the lane): every shared-memory load is issued before the first use, the 6-bit scales become binary16 through
// the same byte permute as the quants (no conversion pipe), and the four (piece, row half) conversions are
// independent instruction streams the scheduler can interleave.
__device__ __forceinline__ void kq_stage_q4k(const unsigned char* __restrict__ tile, int c, unsigned char* __restrict__ a_planes,
                                             unsigned char* __restrict__ a2, float2* __restrict__ row_scales, int row0, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint4 w0 = *reinterpret_cast<const uint4*>(tile + (2 * c) * 512 + lane * 16);
    const uint4 w1 = *reinterpret_cast<const uint4*>(tile + (2 * c + 1) * 512 + lane * 16);
    const uint4 ha = *reinterpret_cast<const uint4*>(tile + 2048 + g * 16);
    const uint4 hb = *reinterpret_cast<const uint4*>(tile + 2048 + (g + 8) * 16);
    const __half2 k1024 = __float2half2_rn(1024.0f), kneg = __float2half2_rn(-1024.0f);
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const uint4 h = rr == 0 ? ha : hb;
        const int unit_row = row0 + g + 8 * rr;
        // scales of groups 4 c .. 4 c + 3 of this row, as binary16 (exact)
        const uint32_t sc4 = c == 0 ? (h.y & 0x3F3F3F3Fu) : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
        __half2 s01, s23;
        bytes_to_half_pairs(sc4, s01, s23);
        s01 = __hsub2(s01, k1024);
        s23 = __hsub2(s23, k1024);
        if (c == 0) {
            if (t == 0) {
                row_scales[unit_row] = make_float2(__half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu))),
                                                   __half2float(__ushort_as_half((unsigned short)(h.x >> 16))));
            }
            // minima of groups 2 t, 2 t + 1 as binary16, into the first 8-input block of A2
            const uint32_t mlo = h.z & 0x3F3F3F3Fu, mhi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
            const uint32_t m4 = t < 2 ? mlo : mhi;
            __half2 m01, m23;
            bytes_to_half_pairs(m4, m01, m23);
            const __half2 mm = __hsub2((t & 1) ? m23 : m01, k1024);
            *reinterpret_cast<__half2*>(a2 + (unit_row >> 3) * 128 + (unit_row & 7) * 16 + 4 * t) = mm;
        }
        unsigned char* row_base = a_planes + (unit_row >> 3) * 128 + (unit_row & 7) * 16;
#pragma unroll
        for (int piece = 0; piece < 2; ++piece) {
            const uint4 w = piece == 0 ? w0 : w1;
            const __half2 sp = piece == 0 ? s01 : s23;               // (even group's scale, odd group's scale)
            const __half2 se = __low2half2(sp), so = __high2half2(sp);
            const __half2 be = __hmul2(se, kneg), bo = __hmul2(so, kneg);
            unsigned char* base = row_base + ((piece * kChunkK) >> 3) * kALbo;
            const uint32_t lo16 = rr == 0 ? w.x : w.z, hi16 = rr == 0 ? w.y : w.w;
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                const uint32_t word = part == 0 ? lo16 : hi16;
                __half2 e01, e23, o01, o23;
                bytes_to_half_pairs(word & 0x0F0F0F0Fu, e01, e23);
                bytes_to_half_pairs((word >> 4) & 0x0F0F0F0Fu, o01, o23);
                const int k_e = part * 16 + 4 * t, k_o = 32 + k_e;
                store_half4(base + (k_e >> 3) * kALbo + (k_e & 7) * 2, __hfma2(e01, se, be), __hfma2(e23, se, be));
                store_half4(base + (k_o >> 3) * kALbo + (k_o & 7) * 2, __hfma2(o01, so, bo), __hfma2(o23, so, bo));
            }
        }
    }
}

__global__ void __launch_bounds__(kKqThreads, 1) gemm_tcq_kernel(const GemmArgs a, const KqLayout lay, const int units) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = a.k / kTileCols;
    const uint32_t spin_limit = a.spin_limit ? a.spin_limit : kSpinLimit;
    // Operand stages hold lay.chunk_k inputs: 128 when every unit is Q4_K (half as many hand-offs per k tile), else 64.
    const int pieces = lay.chunk_k / kChunkK, chunks_per_tile = kTileCols / lay.chunk_k;
    const int a_bytes = lay.a_planes * kAHalfBytes * pieces;
    const int b_stage_bytes = lay.b_bytes * pieces;
    const uint32_t na = (uint32_t)lay.a_stages;
    unsigned char* w_ring = smem;
    unsigned char* a_buf = w_ring + (size_t)lay.w_stages * lay.w_stage_bytes;        // [2][planes][16 KB]
    unsigned char* a2_buf = a_buf + (size_t)lay.a_stages * a_bytes;                   // [2][kA2Bytes]
    unsigned char* b_buf = a2_buf + 2 * kA2Bytes;                                     // [a_stages][b_bytes]
    unsigned char* b2_buf = b_buf + (size_t)lay.a_stages * b_stage_bytes;             // [2][b2_bytes]
    float2* row_scales = reinterpret_cast<float2*>(b2_buf + 2 * (size_t)lay.b2_bytes);  // [4][kRows]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(row_scales + 4 * kRows);
    const uint32_t bars = smem_u32(tmem_slot + 4);
    // One commit per chunk frees the A stage and the activation stage of the same index (a_empty); the
    // commit that completes a k tile (t_full) also frees that k tile's group-sum buffer.
    const uint32_t w_full = bars, w_empty = bars + 32, a_full = bars + 64, a_empty = bars + 96, t_full = bars + 128,
                   t_empty = bars + 144, b2_full = bars + 160, b_full = bars + 192;
    const int S = lay.k_slices, tps = (k_tiles + S - 1) / S, G = lay.groups, items = units * G * S;
    // work item -> (unit, row group, K slice), the slice innermost: the groups of a unit run side by side on
    // neighbouring CTAs, so the unit's weight tiles come from HBM once
    auto unit_index = [&](int item) { return item / (G * S); };
    auto group_index = [&](int item) { return (item / S) % G; };

    if (threadIdx.x == 0) {
        for (int i = 0; i < lay.w_stages; ++i) { mbar_init(w_full + 8 * i, 1); mbar_init(w_empty + 8 * i, kKqDequantWarps); }
        for (int i = 0; i < lay.a_stages; ++i) { mbar_init(a_full + 8 * i, kKqDequantWarps); mbar_init(a_empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(t_full + 8 * i, 1);
            mbar_init(t_empty + 8 * i, kEpilogueWarps);
            mbar_init(b2_full + 8 * i, 1);
        }
        for (int i = 0; i < lay.a_stages; ++i) mbar_init(b_full + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // The second 8-input block of the minima operand stays zero for the whole kernel.
    for (int i = threadIdx.x; i < 2 * kA2Bytes / 16; i += kKqThreads) reinterpret_cast<uint4*>(a2_buf)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    // tensor memory: main sums of k tile parity p at columns 128 p, minima sums at 256 + 128 p

    if (warp == kProducerWarp) {
        bool alive = true;
        uint32_t w_count = 0, kt_count = 0;
        int witem = blockIdx.x, wkb = (witem % S) * tps;   // next weight stage to issue: (work item, k tile)
        auto issue_w = [&]() {
            if (witem >= items) return;
            const UnitRef ur = unit_of(a, unit_index(witem));
            const GemvSegment& s = a.seg[ur.seg];
            const uint32_t tb = (uint32_t)packed_tile_bytes(s.type);
            const uint32_t stage = w_count % (uint32_t)lay.w_stages;
            if (lane == 0) {
                if (w_count >= (uint32_t)lay.w_stages && alive) {
                    alive = mbar_wait_relaxed(w_empty + 8 * stage, ((w_count / (uint32_t)lay.w_stages) - 1u) & 1u, a.error_flag, 21, spin_limit);
                }
                const int present = min(kRowTilesPerUnit, s.row_tiles - ur.rt0);
                mbar_expect_tx(w_full + 8 * stage, (uint32_t)present * tb);
            }
            __syncwarp();
            if (lane < kRowTilesPerUnit && ur.rt0 + lane < s.row_tiles) {
                bulk_g2s(smem_u32(w_ring + (size_t)stage * lay.w_stage_bytes + (size_t)lane * tb),
                         s.data + ((size_t)(ur.rt0 + lane) * k_tiles + wkb) * tb, tb, w_full + 8 * stage);
            }
            ++w_count;
            if (++wkb == min(k_tiles, ((witem % S) + 1) * tps)) { witem += gridDim.x; wkb = (witem % S) * tps; }
        };
        issue_w();
        if (lay.w_stages > 2) issue_w();
        const size_t tile_stride = (size_t)kChunksPerTile * lay.b_bytes + lay.b2_bytes;  // one k tile of activations
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const int kb0 = (item % S) * tps, kb1 = min(k_tiles, kb0 + tps);
            for (int kb = kb0; kb < kb1; ++kb, ++kt_count) {
                if (lane == 0) {
                    const uint32_t p = kt_count & 1u;
                    if (kt_count >= 2u && alive) alive = mbar_wait_relaxed(t_full + 8 * p, ((kt_count >> 1) - 1u) & 1u, a.error_flag, 23, spin_limit);
                    mbar_expect_tx(b2_full + 8 * p, (uint32_t)lay.b2_bytes);
                    bulk_g2s(smem_u32(b2_buf + (size_t)p * lay.b2_bytes),
                             a.chunks + (size_t)group_index(item) * lay.group_bytes + (size_t)kb * tile_stride + (size_t)kChunksPerTile * lay.b_bytes,
                             (uint32_t)lay.b2_bytes, b2_full + 8 * p);
                }
                __syncwarp();
                issue_w();
            }
        }
    } else if (warp >= kKqChunkWarp0) {
        // ---------------- activation chunks: a bulk copy keeps its issuing thread busy for a few hundred
        // nanoseconds, so the chunks of a k tile alternate between two copying warps ----------------
        if (lane == 0) {
            bool alive = true;
            const int which = warp - kKqChunkWarp0;
            const size_t tile_stride = (size_t)kChunksPerTile * lay.b_bytes + lay.b2_bytes;
            uint32_t b_count = 0;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int kb0 = (item % S) * tps, kb1 = min(k_tiles, kb0 + tps);
                for (int kb = kb0; kb < kb1; ++kb) {
                    const signed char* src = a.chunks + (size_t)group_index(item) * lay.group_bytes + (size_t)kb * tile_stride;
                    for (int c = 0; c < chunks_per_tile; ++c, ++b_count) {
                        if ((c & 1) != which) continue;
                        const uint32_t bs = b_count % na;
                        if (b_count >= na && alive) alive = mbar_wait_relaxed(a_empty + 8 * bs, ((b_count / na) - 1u) & 1u, a.error_flag, 22, spin_limit);
                        mbar_expect_tx(b_full + 8 * bs, (uint32_t)b_stage_bytes);
                        bulk_g2s(smem_u32(b_buf + (size_t)bs * b_stage_bytes), src + (size_t)c * b_stage_bytes, (uint32_t)b_stage_bytes, b_full + 8 * bs);
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            bool alive = true;
            uint32_t count = 0, kt_count = 0;
            const uint32_t idesc = umma_idesc(lay.cols);
            const uint32_t b_lbo = (uint32_t)(lay.cols / 8) * 128u;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const bool q4k = a.seg[unit_of(a, unit_index(item)).seg].type == kQ4_K;
                const int kb0 = (item % S) * tps, kb1 = min(k_tiles, kb0 + tps);
                for (int kb = kb0; kb < kb1; ++kb, ++kt_count) {
                    const uint32_t p = kt_count & 1u;
                    if (kt_count >= 2u && alive) alive = mbar_wait(t_empty + 8 * p, ((kt_count >> 1) - 1u) & 1u, a.error_flag, 24, spin_limit);
                    tc_fence_after();
                    const uint32_t d_main = tmem_base + p * 128u, d_min = tmem_base + 256u + p * 128u;
                    for (int c = 0; c < chunks_per_tile; ++c, ++count) {
                        const uint32_t st = count % na, bs = st;
                        if (alive) alive = mbar_wait(a_full + 8 * st, (count / na) & 1u, a.error_flag, 25, spin_limit);
                        if (alive) alive = mbar_wait(b_full + 8 * bs, (count / na) & 1u, a.error_flag, 26, spin_limit);
                        tc_fence_after();
                        const uint32_t a_addr = smem_u32(a_buf + (size_t)st * a_bytes);
                        const uint32_t b_addr = smem_u32(b_buf + (size_t)bs * b_stage_bytes);
                        // Descriptors of successive 16-input steps differ only in the start address field (bits 0..13,
                        // in 16-byte units; no carry leaves it inside one stage): one 64-bit add per step.
                        uint64_t da = umma_desc(a_addr, kALbo, 128), db = umma_desc(b_addr, b_lbo, 128);
                        const uint64_t da_step = (uint64_t)((2 * kALbo) >> 4), db_step = (uint64_t)((2 * b_lbo) >> 4);
                        const uint64_t da_plane = (uint64_t)(kAHalfBytes >> 4);
                        const int steps = lay.chunk_k / 16;
                        if (q4k) {
#pragma unroll 4
                            for (int s16 = 0; s16 < steps; ++s16, da += da_step, db += db_step) {
                                umma_f16(d_main, da, db, idesc, (c | s16) != 0 ? 1u : 0u);
                            }
                        } else {
#pragma unroll 4
                            for (int s16 = 0; s16 < steps; ++s16, da += da_step, db += db_step) {
                                umma_f16(d_main, da, db, idesc, (c | s16) != 0 ? 1u : 0u);
                                umma_f16(d_main, da + da_plane, db, idesc, 1u);
                            }
                        }
                        if (c == chunks_per_tile - 1) {
                            // Q4_K: group minima x group sums of the activations (the chunk's a_full covers A2 as well)
                            if (alive) alive = mbar_wait(b2_full + 8 * p, (kt_count >> 1) & 1u, a.error_flag, 27, spin_limit);
                            tc_fence_after();
                            if (q4k) {
                                umma_f16(d_min, umma_desc(smem_u32(a2_buf + (size_t)p * kA2Bytes), kALbo, 128),
                                         umma_desc(smem_u32(b2_buf + (size_t)p * lay.b2_bytes), b_lbo, 128), idesc, 0u);
                            }
                        }
                        umma_commit(a_empty + 8 * st);
                    }
                    umma_commit(t_full + 8 * p);
                }
            }
        }
    } else if (warp >= kDequantWarp0 && warp < kKqChunkWarp0) {
        const int rt_local = warp - kDequantWarp0;
        bool alive = true;
        uint32_t w_count = 0, a_count = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const UnitRef ur = unit_of(a, unit_index(item));
            const GemvSegment& s = a.seg[ur.seg];
            const int type = s.type;
            const bool present = ur.rt0 + rt_local < s.row_tiles;
            const int tb = packed_tile_bytes(type);
            const int kb0 = (item % S) * tps, kb1 = min(k_tiles, kb0 + tps);
            for (int kb = kb0; kb < kb1; ++kb, ++w_count) {
                const uint32_t stage = w_count % (uint32_t)lay.w_stages;
                if (alive) alive = mbar_wait(w_full + 8 * stage, (w_count / (uint32_t)lay.w_stages) & 1u, a.error_flag, 28, spin_limit);
                const unsigned char* tile = w_ring + (size_t)stage * lay.w_stage_bytes + (size_t)rt_local * tb;
                for (int c = 0; c < chunks_per_tile; ++c, ++a_count) {
                    const uint32_t st = a_count % na;
                    if (a_count >= na && alive) alive = mbar_wait(a_empty + 8 * st, ((a_count / na) - 1u) & 1u, a.error_flag, 29, spin_limit);
                    unsigned char* planes = a_buf + (size_t)st * a_bytes;
                    // A2 and the row scales of k tile w_count: written at chunk 0, consumed after chunk 3's MMAs.
                    // A2's previous reader (two k tiles back) was issued before the MMAs whose completion released this
                    // chunk's buffer (at most four chunks back), so it has finished too.
                    unsigned char* a2 = a2_buf + (size_t)(w_count & 1u) * kA2Bytes;
                    float2* scales = row_scales + (size_t)(w_count & 3u) * kRows;
                    if (present && type == kQ4_K && pieces == 2) {
                        kq_stage_q4k(tile, c, planes, a2, scales, rt_local * kTileRows, lane);
                    } else if (present) {
                        for (int piece = 0; piece < pieces; ++piece) {
                            kq_chunk(type, tile, c * pieces + piece, piece * kChunkK, planes, a2, scales, rt_local * kTileRows, 0, lane);
                            kq_chunk(type, tile, c * pieces + piece, piece * kChunkK, planes, a2, scales, rt_local * kTileRows, 1, lane);
                        }
                    } else {
                        for (int pl = 0; pl < (type == kQ4_K ? 1 : 2); ++pl) {
                            for (int piece = 0; piece < pieces; ++piece) {
                                unsigned char* at = planes + (size_t)pl * kAHalfBytes + (size_t)piece * (kChunkK / 8) * kALbo;
                                zero_rows_plane(at, rt_local * kTileRows, lane);
                                zero_rows_plane(at, rt_local * kTileRows + 8, lane);
                            }
                        }
                        if (c == 0 && lane < 16) {
                            const int unit_row = rt_local * kTileRows + lane;
                            scales[unit_row] = make_float2(0.0f, 0.0f);
                            *reinterpret_cast<uint4*>(a2 + (unit_row >> 3) * 128 + (unit_row & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(a_full + 8 * st);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(w_empty + 8 * stage);
            }
        }
    } else {
        // ---------------- epilogue warps: fold each k tile into registers, store at the end of the unit ----------------
        bool alive = true;
        uint32_t kt_count = 0;
        const int row = warp * 32 + lane;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const UnitRef ur = unit_of(a, unit_index(item));
            const GemvSegment& s = a.seg[ur.seg];
            const bool q4k = s.type == kQ4_K;
            const int slice = item % S, kb0 = slice * tps, kb1 = min(k_tiles, kb0 + tps);
            float acc[kKqMaxMembers];
#pragma unroll
            for (int i = 0; i < kKqMaxMembers; ++i) acc[i] = 0.0f;
            for (int kb = kb0; kb < kb1; ++kb, ++kt_count) {
                const uint32_t p = kt_count & 1u;
                if (alive) alive = mbar_wait(t_full + 8 * p, (kt_count >> 1) & 1u, a.error_flag, 30, spin_limit);
                tc_fence_after();
                const float2 ds = row_scales[(size_t)(kt_count & 3u) * kRows + row];
                const uint32_t t_main = tmem_base + p * 128u + ((uint32_t)(warp * 32) << 16), t_min = t_main + 256u;
#pragma unroll
                for (int m0 = 0; m0 < kKqMaxMembers; m0 += 16) {
                    if (m0 < lay.members_padded) {
                        float hi[16], lo[16];
                        tmem_ld16(t_main + (uint32_t)m0, hi);
                        tmem_ld16(t_main + (uint32_t)(lay.members_padded + m0), lo);
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[m0 + i] = fmaf(ds.x, hi[i] + lo[i], acc[m0 + i]);
                        if (q4k) {
                            tmem_ld16(t_min + (uint32_t)m0, hi);
                            tmem_ld16(t_min + (uint32_t)(lay.members_padded + m0), lo);
#pragma unroll
                            for (int i = 0; i < 16; ++i) acc[m0 + i] = fmaf(-ds.y, hi[i] + lo[i], acc[m0 + i]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(t_empty + 8 * p);
            }
            const int n_index = ur.rt0 * kTileRows + row;
            if (n_index < s.n) {
                if (S > 1) {
                    // this K slice's sums, unscaled: [slice][member][all segments' rows]; a second kernel adds the slices in order
                    int seg_offset = 0;
                    for (int i = 0; i < ur.seg; ++i) seg_offset += a.seg[i].n;
                    float* part = a.partial + ((size_t)slice * a.members) * lay.total_n + seg_offset + n_index;
#pragma unroll
                    for (int m = 0; m < kKqMaxMembers; ++m) {
                        if (m < a.members) part[(size_t)m * lay.total_n] = acc[m];
                    }
                } else {
#pragma unroll
                    for (int m = 0; m < kKqMaxMembers; ++m) {
                        if (m < a.members) {
                            const size_t member = (size_t)group_index(item) * a.members + m;
                            const float v = acc[m] * a.member_scale[member];
                            float* y = s.y + member * s.n + n_index;
                            if (a.epilogue == kResidual) *y += v; else *y = v;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- two row groups per work item ------------------------------------------------------------------
// Prefill steps and large batches bring several whole groups of 64 rows to a projection.  The kernel above
// converts every weight stage once per group; this one converts it once per PAIR of groups: the MMA thread
// multiplies each converted stage by both groups' activation chunks, into two tensor-memory regions (main sums
// of group g at columns 128 g, minima sums at 256 + 128 g: all 512 columns, one buffer per k tile: the fold
// of k tile t hides under the conversion of k tile t + 1's first stage, which the MMAs wait for anyway).  Eight
// epilogue warps (lane quadrant q = warp & 3, member half h = warp >> 2) fold 32 members of both groups each, so
// a thread still carries 64 accumulators.  Stages hold 64 inputs; whole groups only (64 members), no K split.
constexpr int kKq2EpilogueWarps = 8;
constexpr int kKq2ProducerWarp = 8;
constexpr int kKq2MmaWarp = 9;
constexpr int kKq2DequantWarp0 = 10;
constexpr int kKq2ChunkWarp0 = kKq2DequantWarp0 + kKqDequantWarps;
constexpr int kKq2Threads = (kKq2ChunkWarp0 + 2) * 32;

__global__ void __launch_bounds__(kKq2Threads, 1) gemm_tcq2_kernel(const GemmArgs a, const KqLayout lay, const int units) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = a.k / kTileCols;
    const uint32_t spin_limit = a.spin_limit ? a.spin_limit : kSpinLimit;
    constexpr int chunks_per_tile = kChunksPerTile;   // 64-input stages
    const int a_bytes = lay.a_planes * kAHalfBytes;
    const int b_group_bytes = lay.b_bytes;             // one group's chunk
    const int b_stage_bytes = 2 * b_group_bytes;       // both groups' chunks
    const uint32_t na = (uint32_t)lay.a_stages;
    unsigned char* w_ring = smem;
    unsigned char* a_buf = w_ring + (size_t)lay.w_stages * lay.w_stage_bytes;        // [a_stages][planes][16 KB]
    unsigned char* a2_buf = a_buf + (size_t)lay.a_stages * a_bytes;                   // [2][kA2Bytes]
    unsigned char* b_buf = a2_buf + 2 * kA2Bytes;                                     // [a_stages][2 groups][b_bytes]
    unsigned char* b2_buf = b_buf + (size_t)lay.a_stages * b_stage_bytes;             // [2][2 groups][b2_bytes]
    float2* row_scales = reinterpret_cast<float2*>(b2_buf + 4 * (size_t)lay.b2_bytes);  // [4][kRows]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(row_scales + 4 * kRows);
    const uint32_t bars = smem_u32(tmem_slot + 4);
    const uint32_t w_full = bars, w_empty = bars + 32, a_full = bars + 64, a_empty = bars + 96, t_full = bars + 128,
                   t_empty = bars + 144, b2_full = bars + 160, b_full = bars + 192;
    const int P = lay.groups / 2, items = units * P;   // work item -> (unit, pair of groups), the pair innermost
    auto unit_index = [&](int item) { return item / P; };
    auto pair_index = [&](int item) { return item % P; };

    if (threadIdx.x == 0) {
        for (int i = 0; i < lay.w_stages; ++i) { mbar_init(w_full + 8 * i, 1); mbar_init(w_empty + 8 * i, kKqDequantWarps); }
        for (int i = 0; i < lay.a_stages; ++i) { mbar_init(a_full + 8 * i, kKqDequantWarps); mbar_init(a_empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) {   // two barriers each, alternating by k tile, so that no wait is two phases behind
            mbar_init(t_full + 8 * i, 1);
            mbar_init(t_empty + 8 * i, kKq2EpilogueWarps);
            mbar_init(b2_full + 8 * i, 1);
        }
        for (int i = 0; i < lay.a_stages; ++i) mbar_init(b_full + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < 2 * kA2Bytes / 16; i += kKq2Threads) reinterpret_cast<uint4*>(a2_buf)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == kKq2MmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const size_t tile_stride = (size_t)kChunksPerTile * lay.b_bytes + lay.b2_bytes;  // one k tile of one group's activations

    if (warp == kKq2ProducerWarp) {
        bool alive = true;
        uint32_t w_count = 0, kt_count = 0;
        int witem = blockIdx.x, wkb = 0;   // next weight stage to issue: (work item, k tile)
        auto issue_w = [&]() {
            if (witem >= items) return;
            const UnitRef ur = unit_of(a, unit_index(witem));
            const GemvSegment& s = a.seg[ur.seg];
            const uint32_t tb = (uint32_t)packed_tile_bytes(s.type);
            const uint32_t stage = w_count % (uint32_t)lay.w_stages;
            if (lane == 0) {
                if (w_count >= (uint32_t)lay.w_stages && alive) {
                    alive = mbar_wait_relaxed(w_empty + 8 * stage, ((w_count / (uint32_t)lay.w_stages) - 1u) & 1u, a.error_flag, 41, spin_limit);
                }
                const int present = min(kRowTilesPerUnit, s.row_tiles - ur.rt0);
                mbar_expect_tx(w_full + 8 * stage, (uint32_t)present * tb);
            }
            __syncwarp();
            if (lane < kRowTilesPerUnit && ur.rt0 + lane < s.row_tiles) {
                bulk_g2s(smem_u32(w_ring + (size_t)stage * lay.w_stage_bytes + (size_t)lane * tb),
                         s.data + ((size_t)(ur.rt0 + lane) * k_tiles + wkb) * tb, tb, w_full + 8 * stage);
            }
            ++w_count;
            if (++wkb == k_tiles) { witem += gridDim.x; wkb = 0; }
        };
        issue_w();
        if (lay.w_stages > 2) issue_w();
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            for (int kb = 0; kb < k_tiles; ++kb, ++kt_count) {
                if (lane == 0) {
                    // the group sums of k tile kt go where those of k tile kt - 2 were: its minima MMAs ended before
                    // the commit that completed k tile kt - 2, which the epilogue of kt - 2 and so the MMAs of kt - 1 followed
                    const uint32_t p = kt_count & 1u;
                    if (kt_count >= 2u && alive) alive = mbar_wait_relaxed(t_full + 8 * p, ((kt_count >> 1) - 1u) & 1u, a.error_flag, 43, spin_limit);
                    mbar_expect_tx(b2_full + 8 * p, 2u * (uint32_t)lay.b2_bytes);
                    for (int g = 0; g < 2; ++g) {
                        bulk_g2s(smem_u32(b2_buf + (size_t)(2 * p + g) * lay.b2_bytes),
                                 a.chunks + (size_t)(2 * pair_index(item) + g) * lay.group_bytes + (size_t)kb * tile_stride + (size_t)kChunksPerTile * lay.b_bytes,
                                 (uint32_t)lay.b2_bytes, b2_full + 8 * p);
                    }
                }
                __syncwarp();
                issue_w();
            }
        }
    } else if (warp >= kKq2ChunkWarp0) {
        if (lane == 0) {
            bool alive = true;
            const int which = warp - kKq2ChunkWarp0;
            uint32_t b_count = 0;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                for (int kb = 0; kb < k_tiles; ++kb) {
                    for (int c = 0; c < chunks_per_tile; ++c, ++b_count) {
                        if ((c & 1) != which) continue;
                        const uint32_t bs = b_count % na;
                        if (b_count >= na && alive) alive = mbar_wait_relaxed(a_empty + 8 * bs, ((b_count / na) - 1u) & 1u, a.error_flag, 42, spin_limit);
                        mbar_expect_tx(b_full + 8 * bs, (uint32_t)b_stage_bytes);
                        for (int g = 0; g < 2; ++g) {
                            const signed char* src = a.chunks + (size_t)(2 * pair_index(item) + g) * lay.group_bytes + (size_t)kb * tile_stride;
                            bulk_g2s(smem_u32(b_buf + (size_t)bs * b_stage_bytes + (size_t)g * b_group_bytes), src + (size_t)c * b_group_bytes,
                                     (uint32_t)b_group_bytes, b_full + 8 * bs);
                        }
                    }
                }
            }
        }
    } else if (warp == kKq2MmaWarp) {
        if (lane == 0) {
            bool alive = true;
            uint32_t count = 0, kt_count = 0;
            const uint32_t idesc = umma_idesc(lay.cols);
            const uint32_t b_lbo = (uint32_t)(lay.cols / 8) * 128u;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const bool q4k = a.seg[unit_of(a, unit_index(item)).seg].type == kQ4_K;
                for (int kb = 0; kb < k_tiles; ++kb, ++kt_count) {
                    const uint32_t p = kt_count & 1u;
                    // the one accumulator buffer: the epilogue has folded the previous k tile
                    if (kt_count >= 1u && alive) alive = mbar_wait(t_empty + 8 * ((kt_count - 1u) & 1u), ((kt_count - 1u) >> 1) & 1u, a.error_flag, 44, spin_limit);
                    tc_fence_after();
                    for (int c = 0; c < chunks_per_tile; ++c, ++count) {
                        const uint32_t st = count % na;
                        if (alive) alive = mbar_wait(a_full + 8 * st, (count / na) & 1u, a.error_flag, 45, spin_limit);
                        if (alive) alive = mbar_wait(b_full + 8 * st, (count / na) & 1u, a.error_flag, 46, spin_limit);
                        tc_fence_after();
                        const uint32_t a_addr = smem_u32(a_buf + (size_t)st * a_bytes);
                        const uint64_t da_step = (uint64_t)((2 * kALbo) >> 4), db_step = (uint64_t)((2 * b_lbo) >> 4);
                        const uint64_t da_plane = (uint64_t)(kAHalfBytes >> 4);
                        for (int g = 0; g < 2; ++g) {
                            const uint32_t b_addr = smem_u32(b_buf + (size_t)st * b_stage_bytes + (size_t)g * b_group_bytes);
                            uint64_t da = umma_desc(a_addr, kALbo, 128), db = umma_desc(b_addr, b_lbo, 128);
                            const uint32_t d_main = tmem_base + 128u * (uint32_t)g;
                            if (q4k) {
#pragma unroll
                                for (int s16 = 0; s16 < kChunkK / 16; ++s16, da += da_step, db += db_step) {
                                    umma_f16(d_main, da, db, idesc, (c | s16) != 0 ? 1u : 0u);
                                }
                            } else {
#pragma unroll
                                for (int s16 = 0; s16 < kChunkK / 16; ++s16, da += da_step, db += db_step) {
                                    umma_f16(d_main, da, db, idesc, (c | s16) != 0 ? 1u : 0u);
                                    umma_f16(d_main, da + da_plane, db, idesc, 1u);
                                }
                            }
                        }
                        if (c == chunks_per_tile - 1) {
                            // Q4_K: group minima x group sums of the activations (the chunk's a_full covers A2 as well)
                            if (alive) alive = mbar_wait(b2_full + 8 * p, (kt_count >> 1) & 1u, a.error_flag, 47, spin_limit);
                            tc_fence_after();
                            if (q4k) {
                                for (int g = 0; g < 2; ++g) {
                                    umma_f16(tmem_base + 256u + 128u * (uint32_t)g, umma_desc(smem_u32(a2_buf + (size_t)p * kA2Bytes), kALbo, 128),
                                             umma_desc(smem_u32(b2_buf + (size_t)(2 * p + g) * lay.b2_bytes), b_lbo, 128), idesc, 0u);
                                }
                            }
                        }
                        umma_commit(a_empty + 8 * st);
                    }
                    umma_commit(t_full + 8 * p);
                }
            }
        }
    } else if (warp >= kKq2DequantWarp0 && warp < kKq2ChunkWarp0) {
        const int rt_local = warp - kKq2DequantWarp0;
        bool alive = true;
        uint32_t w_count = 0, a_count = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const UnitRef ur = unit_of(a, unit_index(item));
            const GemvSegment& s = a.seg[ur.seg];
            const int type = s.type;
            const bool present = ur.rt0 + rt_local < s.row_tiles;
            const int tb = packed_tile_bytes(type);
            for (int kb = 0; kb < k_tiles; ++kb, ++w_count) {
                const uint32_t stage = w_count % (uint32_t)lay.w_stages;
                if (alive) alive = mbar_wait(w_full + 8 * stage, (w_count / (uint32_t)lay.w_stages) & 1u, a.error_flag, 48, spin_limit);
                const unsigned char* tile = w_ring + (size_t)stage * lay.w_stage_bytes + (size_t)rt_local * tb;
                for (int c = 0; c < chunks_per_tile; ++c, ++a_count) {
                    const uint32_t st = a_count % na;
                    if (a_count >= na && alive) alive = mbar_wait(a_empty + 8 * st, ((a_count / na) - 1u) & 1u, a.error_flag, 49, spin_limit);
                    unsigned char* planes = a_buf + (size_t)st * a_bytes;
                    unsigned char* a2 = a2_buf + (size_t)(w_count & 1u) * kA2Bytes;
                    float2* scales = row_scales + (size_t)(w_count & 3u) * kRows;
                    if (present) {
                        kq_chunk(type, tile, c, 0, planes, a2, scales, rt_local * kTileRows, 0, lane);
                        kq_chunk(type, tile, c, 0, planes, a2, scales, rt_local * kTileRows, 1, lane);
                    } else {
                        for (int pl = 0; pl < (type == kQ4_K ? 1 : 2); ++pl) {
                            unsigned char* at = planes + (size_t)pl * kAHalfBytes;
                            zero_rows_plane(at, rt_local * kTileRows, lane);
                            zero_rows_plane(at, rt_local * kTileRows + 8, lane);
                        }
                        if (c == 0 && lane < 16) {
                            const int unit_row = rt_local * kTileRows + lane;
                            scales[unit_row] = make_float2(0.0f, 0.0f);
                            *reinterpret_cast<uint4*>(a2 + (unit_row >> 3) * 128 + (unit_row & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(a_full + 8 * st);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(w_empty + 8 * stage);
            }
        }
    } else {
        // ---------------- epilogue warps: (lane quadrant, member half); fold each k tile of both groups ----------------
        bool alive = true;
        uint32_t kt_count = 0;
        const int quadrant = warp & 3, half = warp >> 2;
        const int row = quadrant * 32 + lane;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const UnitRef ur = unit_of(a, unit_index(item));
            const GemvSegment& s = a.seg[ur.seg];
            const bool q4k = s.type == kQ4_K;
            float acc[2][32];
#pragma unroll
            for (int g = 0; g < 2; ++g) {
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[g][i] = 0.0f;
            }
            for (int kb = 0; kb < k_tiles; ++kb, ++kt_count) {
                const uint32_t p = kt_count & 1u;
                if (alive) alive = mbar_wait(t_full + 8 * p, (kt_count >> 1) & 1u, a.error_flag, 50, spin_limit);
                tc_fence_after();
                const float2 ds = row_scales[(size_t)(kt_count & 3u) * kRows + row];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const uint32_t t_main = tmem_base + 128u * (uint32_t)g + ((uint32_t)(quadrant * 32) << 16), t_min = t_main + 256u;
#pragma unroll
                    for (int m0 = 0; m0 < 32; m0 += 16) {
                        float hi[16], lo[16];
                        tmem_ld16(t_main + (uint32_t)(32 * half + m0), hi);
                        tmem_ld16(t_main + (uint32_t)(64 + 32 * half + m0), lo);
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[g][m0 + i] = fmaf(ds.x, hi[i] + lo[i], acc[g][m0 + i]);
                        if (q4k) {
                            tmem_ld16(t_min + (uint32_t)(32 * half + m0), hi);
                            tmem_ld16(t_min + (uint32_t)(64 + 32 * half + m0), lo);
#pragma unroll
                            for (int i = 0; i < 16; ++i) acc[g][m0 + i] = fmaf(-ds.y, hi[i] + lo[i], acc[g][m0 + i]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(t_empty + 8 * p);
            }
            const int n_index = ur.rt0 * kTileRows + row;
            if (n_index < s.n) {
#pragma unroll
                for (int g = 0; g < 2; ++g) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const size_t member = (size_t)(2 * pair_index(item) + g) * 64 + 32 * half + i;
                        const float v = acc[g][i] * a.member_scale[member];
                        float* y = s.y + member * s.n + n_index;
                        if (a.epilogue == kResidual) *y += v; else *y = v;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kKq2MmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace

// ---- converted-operand cache ------------------------------------------------------------------------
// The kernels above convert every packed weight stage into the tensor core's operand form each time it is
// used.  With 180 GB of HBM the converted form can simply be kept: per unit (128 rows) and k tile, the four
// 64-input pieces of the A operand exactly as kq_chunk leaves them in shared memory (one binary16 plane of
// 16 KB per piece for Q4_K, two for Q6_K), and a 5 KB record with the rows' scales and the minima operand.
// gemm_tcqc_kernel is the K-quant GEMM without conversion warps: a producer thread brings the pieces in with bulk
// copies, everything downstream (MMA thread, tensor-memory sums, fold, outputs) is the arithmetic of the
// kernels above on identical operand bytes, so results are identical.  What a launch then streams per step is
// the converted bytes (2 or 4 per weight), which is what bounds it.
constexpr int kCachePieceBytes = kAHalfBytes;                        // one plane of one 64-input piece: 16 KB
constexpr int kCacheMetaBytes = kRows * (int)sizeof(float2) + kA2Bytes;   // row scales, then the minima operand

size_t tc_cache_a_bytes(int type, long long rows, long long cols) {
    const long long units = (rows + kRows - 1) / kRows, k_tiles = cols / kTileCols;
    return (size_t)units * k_tiles * kChunksPerTile * (type == kQ4_K ? 1 : 2) * kCachePieceBytes;
}
size_t tc_cache_meta_bytes(long long rows, long long cols) {
    const long long units = (rows + kRows - 1) / kRows, k_tiles = cols / kTileCols;
    return (size_t)units * k_tiles * kCacheMetaBytes;
}

namespace {

// One block per (unit, k tile): warp w converts row tile w of the unit with kq_chunk, straight into the cache.
__global__ void __launch_bounds__(kRowTilesPerUnit * 32) tcq_cache_kernel(int type, const unsigned char* packed, int row_tiles, int k_tiles,
                                                                          unsigned char* cache_a, unsigned char* cache_meta) {
    const int unit = blockIdx.x / k_tiles, kb = blockIdx.x % k_tiles, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int planes = type == kQ4_K ? 1 : 2, rt = unit * kRowTilesPerUnit + warp;
    unsigned char* a_tile = cache_a + ((size_t)unit * k_tiles + kb) * kChunksPerTile * planes * kCachePieceBytes;
    unsigned char* meta = cache_meta + ((size_t)unit * k_tiles + kb) * kCacheMetaBytes;
    float2* scales = reinterpret_cast<float2*>(meta);
    unsigned char* a2 = meta + kRows * sizeof(float2);
    // the minima operand: eight group minima per row, then eight zeros (all zero for Q6_K)
    for (int i = threadIdx.x; i < kA2Bytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(a2)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const bool present = rt < row_tiles;
    const unsigned char* tile = packed + ((size_t)rt * k_tiles + kb) * packed_tile_bytes(type);
    for (int c = 0; c < kChunksPerTile; ++c) {
        unsigned char* planes_at = a_tile + (size_t)c * planes * kCachePieceBytes;
        if (present) {
            kq_chunk(type, tile, c, 0, planes_at, a2, scales, warp * kTileRows, 0, lane);
            kq_chunk(type, tile, c, 0, planes_at, a2, scales, warp * kTileRows, 1, lane);
        } else {
            for (int pl = 0; pl < planes; ++pl) {
                zero_rows_plane(planes_at + (size_t)pl * kCachePieceBytes, warp * kTileRows, lane);
                zero_rows_plane(planes_at + (size_t)pl * kCachePieceBytes, warp * kTileRows + 8, lane);
            }
            if (c == 0 && lane < 16) {
                const int unit_row = warp * kTileRows + lane;
                scales[unit_row] = make_float2(0.0f, 0.0f);
                *reinterpret_cast<uint4*>(a2 + (unit_row >> 3) * 128 + (unit_row & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    }
}

constexpr int kKqcEpilogueWarps = 8;
constexpr int kKqcProducerWarp = 8;
constexpr int kKqcMmaWarp = 9;
constexpr int kKqcChunkWarp0 = 10;
constexpr int kKqcThreads = (kKqcChunkWarp0 + 2) * 32;

struct KqcLayout {
    int stages, pieces, m_slots, stage_bytes, b_bytes, b2_bytes, cols, members_padded;
    int k_slices, total_n, groups;
    size_t group_bytes;
};

// GROUPS row groups per work item (1: up to 64 members, K may be split; 2: whole groups of 64 in pairs).
template <int GROUPS>
__global__ void __launch_bounds__(kKqcThreads, 1) gemm_tcqc_kernel(const GemmArgs a, const KqcLayout lay, const int units) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = a.k / kTileCols;
    const uint32_t spin_limit = a.spin_limit ? a.spin_limit : kSpinLimit;
    // A ring of stages (`pieces` 64-input pieces of the operand with the activation chunks they meet; one commit
    // frees both), and a ring of the k tiles' records.
    const uint32_t na = (uint32_t)lay.stages, nm = (uint32_t)lay.m_slots;
    const int pieces = lay.pieces, stages_per_tile = kChunksPerTile / pieces;
    const int meta_slot = kCacheMetaBytes + GROUPS * lay.b2_bytes;
    const int b_stage_bytes = pieces * GROUPS * lay.b_bytes;
    unsigned char* a_buf = smem;                                                       // [stages][stage_bytes]
    unsigned char* b_buf = a_buf + (size_t)lay.stages * lay.stage_bytes;               // [stages][GROUPS][pieces][b_bytes]
    unsigned char* meta_buf = b_buf + (size_t)lay.stages * b_stage_bytes;              // [m_slots][scales | minima operand | GROUPS group sums]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(meta_buf + (size_t)lay.m_slots * meta_slot);
    const uint32_t bars = smem_u32(tmem_slot + 4);
    const uint32_t a_full = bars, a_empty = bars + 128, b_full = bars + 256, m_full = bars + 384, m_empty = bars + 416,
                   t_full = bars + 448, t_empty = bars + 464;   // at most 16 stages and 4 records
    const int S = lay.k_slices, tps = (k_tiles + S - 1) / S, G = GROUPS == 1 ? lay.groups : lay.groups / 2, items = units * G * S;
    auto unit_index = [&](int item) { return item / (G * S); };
    auto group_index = [&](int item) { return (item / S) % G; };   // GROUPS == 2: index of the pair
    constexpr uint32_t kLag = GROUPS == 1 ? 2u : 1u;   // accumulator buffers: two by k tile parity, or one per group
    const size_t tile_stride = (size_t)kChunksPerTile * lay.b_bytes + lay.b2_bytes;   // one k tile of one group's activations

    if (threadIdx.x == 0) {
        for (int i = 0; i < lay.stages; ++i) { mbar_init(a_full + 8 * i, 1); mbar_init(a_empty + 8 * i, 1); mbar_init(b_full + 8 * i, 1); }
        for (int i = 0; i < lay.m_slots; ++i) { mbar_init(m_full + 8 * i, 1); mbar_init(m_empty + 8 * i, kKqcEpilogueWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(t_full + 8 * i, 1); mbar_init(t_empty + 8 * i, kKqcEpilogueWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kKqcMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == kKqcProducerWarp) {
        if (lane == 0) {
            bool alive = true;
            uint32_t a_count = 0, kt_count = 0;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const UnitRef ur = unit_of(a, unit_index(item));
                const GemvSegment& s = a.seg[ur.seg];
                const uint32_t stage_bytes = (uint32_t)(s.type == kQ4_K ? 1 : 2) * kCachePieceBytes * (uint32_t)pieces;
                const size_t unit_local = (size_t)(ur.rt0 / kRowTilesPerUnit);
                const int kb0 = (item % S) * tps, kb1 = min(k_tiles, kb0 + tps);
                for (int kb = kb0; kb < kb1; ++kb, ++kt_count) {
                    const uint32_t ms = kt_count % nm;
                    // the record slot was last read by the minima MMAs and the fold of k tile kt - m_slots
                    if (kt_count >= nm && alive) alive = mbar_wait_relaxed(m_empty + 8 * ms, ((kt_count / nm) - 1u) & 1u, a.error_flag, 61, spin_limit);
                    unsigned char* slot = meta_buf + (size_t)ms * meta_slot;
                    mbar_expect_tx(m_full + 8 * ms, (uint32_t)meta_slot);
                    bulk_g2s(smem_u32(slot), s.op_meta + (unit_local * k_tiles + kb) * kCacheMetaBytes, (uint32_t)kCacheMetaBytes, m_full + 8 * ms);
                    for (int g = 0; g < GROUPS; ++g) {
                        bulk_g2s(smem_u32(slot + kCacheMetaBytes + (size_t)g * lay.b2_bytes),
                                 a.chunks + (size_t)(GROUPS * group_index(item) + g) * lay.group_bytes + (size_t)kb * tile_stride + (size_t)kChunksPerTile * lay.b_bytes,
                                 (uint32_t)lay.b2_bytes, m_full + 8 * ms);
                    }
                    for (int c = 0; c < stages_per_tile; ++c, ++a_count) {
                        const uint32_t st = a_count % na;
                        if (a_count >= na && alive) alive = mbar_wait_relaxed(a_empty + 8 * st, ((a_count / na) - 1u) & 1u, a.error_flag, 62, spin_limit);
                        mbar_expect_tx(a_full + 8 * st, stage_bytes);
                        bulk_g2s(smem_u32(a_buf + (size_t)st * lay.stage_bytes),
                                 s.op_a + ((unit_local * k_tiles + kb) * stages_per_tile + c) * stage_bytes, stage_bytes, a_full + 8 * st);
                    }
                }
            }
        }
    } else if (warp >= kKqcChunkWarp0) {
        if (lane == 0) {
            bool alive = true;
            const int which = warp - kKqcChunkWarp0;
            uint32_t b_count = 0;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int kb0 = (item % S) * tps, kb1 = min(k_tiles, kb0 + tps);
                for (int kb = kb0; kb < kb1; ++kb) {
                    for (int c = 0; c < stages_per_tile; ++c, ++b_count) {
                        if ((c & 1) != which) continue;
                        const uint32_t bs = b_count % na;
                        if (b_count >= na && alive) alive = mbar_wait_relaxed(a_empty + 8 * bs, ((b_count / na) - 1u) & 1u, a.error_flag, 63, spin_limit);
                        mbar_expect_tx(b_full + 8 * bs, (uint32_t)b_stage_bytes);
                        for (int g = 0; g < GROUPS; ++g) {
                            const signed char* src = a.chunks + (size_t)(GROUPS * group_index(item) + g) * lay.group_bytes + (size_t)kb * tile_stride;
                            bulk_g2s(smem_u32(b_buf + (size_t)bs * b_stage_bytes + (size_t)g * pieces * lay.b_bytes), src + (size_t)c * pieces * lay.b_bytes,
                                     (uint32_t)(pieces * lay.b_bytes), b_full + 8 * bs);
                        }
                    }
                }
            }
        }
    } else if (warp == kKqcMmaWarp) {
        if (lane == 0) {
            bool alive = true;
            uint32_t count = 0, kt_count = 0;
            const uint32_t idesc = umma_idesc(lay.cols);
            const uint32_t b_lbo = (uint32_t)(lay.cols / 8) * 128u;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const bool q4k = a.seg[unit_of(a, unit_index(item)).seg].type == kQ4_K;
                const int kb0 = (item % S) * tps, kb1 = min(k_tiles, kb0 + tps);
                for (int kb = kb0; kb < kb1; ++kb, ++kt_count) {
                    const uint32_t p = kt_count & 1u;
                    if (kt_count >= kLag && alive) {
                        const uint32_t before = kt_count - kLag;   // the k tile whose fold frees these accumulators
                        alive = mbar_wait(t_empty + 8 * (before & 1u), (before >> 1) & 1u, a.error_flag, 64, spin_limit);
                    }
                    tc_fence_after();
                    const uint32_t ms = kt_count % nm;
                    const unsigned char* slot = meta_buf + (size_t)ms * meta_slot;
                    for (int c = 0; c < stages_per_tile; ++c, ++count) {
                        const uint32_t st = count % na;
                        if (alive) alive = mbar_wait(a_full + 8 * st, (count / na) & 1u, a.error_flag, 65, spin_limit);
                        if (alive) alive = mbar_wait(b_full + 8 * st, (count / na) & 1u, a.error_flag, 66, spin_limit);
                        tc_fence_after();
                        const uint64_t da_step = (uint64_t)((2 * kALbo) >> 4), db_step = (uint64_t)((2 * b_lbo) >> 4);
                        const uint64_t da_plane = (uint64_t)(kAHalfBytes >> 4);
                        for (int piece = 0; piece < pieces; ++piece) {
                            // a stage of several pieces holds one plane each (Q4_K only)
                            const uint32_t a_addr = smem_u32(a_buf + (size_t)st * lay.stage_bytes + (size_t)piece * kCachePieceBytes);
                            for (int g = 0; g < GROUPS; ++g) {
                                const uint32_t b_addr = smem_u32(b_buf + (size_t)st * b_stage_bytes + (size_t)(g * pieces + piece) * lay.b_bytes);
                                uint64_t da = umma_desc(a_addr, kALbo, 128), db = umma_desc(b_addr, b_lbo, 128);
                                const uint32_t d_main = tmem_base + 128u * (GROUPS == 1 ? p : (uint32_t)g);
                                if (q4k) {
#pragma unroll
                                    for (int s16 = 0; s16 < kChunkK / 16; ++s16, da += da_step, db += db_step) {
                                        umma_f16(d_main, da, db, idesc, (c | piece | s16) != 0 ? 1u : 0u);
                                    }
                                } else {
#pragma unroll
                                    for (int s16 = 0; s16 < kChunkK / 16; ++s16, da += da_step, db += db_step) {
                                        umma_f16(d_main, da, db, idesc, (c | piece | s16) != 0 ? 1u : 0u);
                                        umma_f16(d_main, da + da_plane, db, idesc, 1u);
                                    }
                                }
                            }
                        }
                        if (c == stages_per_tile - 1) {
                            if (alive) alive = mbar_wait(m_full + 8 * ms, (kt_count / nm) & 1u, a.error_flag, 67, spin_limit);
                            tc_fence_after();
                            if (q4k) {
                                for (int g = 0; g < GROUPS; ++g) {
                                    umma_f16(tmem_base + 256u + 128u * (GROUPS == 1 ? p : (uint32_t)g),
                                             umma_desc(smem_u32(slot + kRows * sizeof(float2)), kALbo, 128),
                                             umma_desc(smem_u32(slot + kCacheMetaBytes + (size_t)g * lay.b2_bytes), b_lbo, 128), idesc, 0u);
                                }
                            }
                        }
                        umma_commit(a_empty + 8 * st);
                    }
                    umma_commit(t_full + 8 * p);
                }
            }
        }
    } else {
        // ---------------- epilogue warps: (lane quadrant, member half) ----------------
        bool alive = true;
        uint32_t kt_count = 0;
        const int quadrant = warp & 3, half = warp >> 2;
        const int row = quadrant * 32 + lane;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const UnitRef ur = unit_of(a, unit_index(item));
            const GemvSegment& s = a.seg[ur.seg];
            const bool q4k = s.type == kQ4_K;
            const int slice = item % S, kb0 = slice * tps, kb1 = min(k_tiles, kb0 + tps);
            float acc[GROUPS][32];
#pragma unroll
            for (int g = 0; g < GROUPS; ++g) {
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[g][i] = 0.0f;
            }
            for (int kb = kb0; kb < kb1; ++kb, ++kt_count) {
                const uint32_t p = kt_count & 1u;
                if (alive) alive = mbar_wait(t_full + 8 * p, (kt_count >> 1) & 1u, a.error_flag, 68, spin_limit);
                // the record's own barrier (complete by now: the minima MMAs followed it), for the copy's bytes
                const uint32_t ms = kt_count % nm;
                if (alive) alive = mbar_wait(m_full + 8 * ms, (kt_count / nm) & 1u, a.error_flag, 69, spin_limit);
                tc_fence_after();
                const float2 ds = reinterpret_cast<const float2*>(meta_buf + (size_t)ms * meta_slot)[row];
                // the record is free again: its scales are in registers, and the MMAs that read its operands are complete
                __syncwarp();
                if (lane == 0) mbar_arrive(m_empty + 8 * ms);
#pragma unroll
                for (int g = 0; g < GROUPS; ++g) {
                    const uint32_t t_main = tmem_base + 128u * (GROUPS == 1 ? p : (uint32_t)g) + ((uint32_t)(quadrant * 32) << 16), t_min = t_main + 256u;
#pragma unroll
                    for (int m0 = 0; m0 < 32; m0 += 16) {
                        if (32 * half + m0 < lay.members_padded) {
                            float hi[16], lo[16];
                            tmem_ld16(t_main + (uint32_t)(32 * half + m0), hi);
                            tmem_ld16(t_main + (uint32_t)(lay.members_padded + 32 * half + m0), lo);
#pragma unroll
                            for (int i = 0; i < 16; ++i) acc[g][m0 + i] = fmaf(ds.x, hi[i] + lo[i], acc[g][m0 + i]);
                            if (q4k) {
                                tmem_ld16(t_min + (uint32_t)(32 * half + m0), hi);
                                tmem_ld16(t_min + (uint32_t)(lay.members_padded + 32 * half + m0), lo);
#pragma unroll
                                for (int i = 0; i < 16; ++i) acc[g][m0 + i] = fmaf(-ds.y, hi[i] + lo[i], acc[g][m0 + i]);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(t_empty + 8 * p);
            }
            const int n_index = ur.rt0 * kTileRows + row;
            if (n_index < s.n) {
                if (GROUPS == 1 && S > 1) {
                    // this K slice's sums, unscaled: [slice][member][all segments' rows]; a second kernel adds the slices in order
                    int seg_offset = 0;
                    for (int i = 0; i < ur.seg; ++i) seg_offset += a.seg[i].n;
                    float* part = a.partial + ((size_t)slice * a.members) * lay.total_n + seg_offset + n_index;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int m = 32 * half + i;
                        if (m < a.members) part[(size_t)m * lay.total_n] = acc[0][i];
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < GROUPS; ++g) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int m = 32 * half + i;
                            if (m < a.members) {
                                const size_t member = (size_t)(GROUPS * group_index(item) + g) * a.members + m;
                                const float v = acc[g][i] * a.member_scale[member];
                                float* y = s.y + member * s.n + n_index;
                                if (a.epilogue == kResidual) *y += v; else *y = v;
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kKqcMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace

cudaError_t launch_tc_cache(cudaStream_t stream, int type, const unsigned char* packed, long long rows, long long cols,
                            unsigned char* cache_a, unsigned char* cache_meta) {
    if ((type != kQ4_K && type != kQ6_K) || !packable(type, rows, cols)) return cudaErrorInvalidValue;
    const int row_tiles = (int)((rows + kTileRows - 1) / kTileRows), k_tiles = (int)(cols / kTileCols);
    const int units = (row_tiles + kRowTilesPerUnit - 1) / kRowTilesPerUnit;
    tcq_cache_kernel<<<(unsigned)(units * k_tiles), kRowTilesPerUnit * 32, 0, stream>>>(type, packed, row_tiles, k_tiles, cache_a, cache_meta);
    return cudaGetLastError();
}

namespace {

// Adds the K slices of a split launch in slice order, applies the member scale and the epilogue.
__global__ void tcq_reduce_kernel(const GemmArgs a, int slices, int total_n) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (long long)a.members * total_n) return;
    const int m = (int)(id / total_n);
    int n = (int)(id % total_n), seg = 0;
    while (seg + 1 < a.n_segments && n >= a.seg[seg].n) { n -= a.seg[seg].n; ++seg; }
    float sum = 0.0f, part[8];  // at most eight slices: all requested before the first is added
#pragma unroll
    for (int sl = 0; sl < 8; ++sl) part[sl] = sl < slices ? a.partial[((size_t)sl * a.members + m) * total_n + (id % total_n)] : 0.0f;
#pragma unroll
    for (int sl = 0; sl < 8; ++sl) {
        if (sl < slices) sum += part[sl];
    }
    const float v = sum * a.member_scale[m];
    float* y = a.seg[seg].y + (size_t)m * a.seg[seg].n + n;
    if (a.epilogue == kResidual) *y += v; else *y = v;
}

// ---- activations -> hi + lo binary16 operand chunks ------------------------------------------------
// Pass 1 (one block per member): power-of-two scale that brings max |x * w| into [1, 2), and the
// epilogue factor (RMSNorm factor / that scale).
__global__ void tc_scale_kernel(const float* x, const int32_t* index, const float* norm_weight, int k, float eps,
                                float* scale_in, float* member_scale) {
    __shared__ float red_max[32], red_sum[32];
    const int m = blockIdx.x;
    const float4* row = reinterpret_cast<const float4*>(x + (size_t)(index ? index[m] : m) * k);
    const float4* nw = reinterpret_cast<const float4*>(norm_weight);
    float amax = 0.0f, ss = 0.0f;
    for (int i0 = threadIdx.x; i0 < k / 4; i0 += 4 * blockDim.x) {   // k is a multiple of 256; four loads in flight per trip
        float4 v[4], w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = i < k / 4 ? row[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            w[u] = (nw != nullptr && i < k / 4) ? nw[i] : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss); ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
            amax = fmaxf(fmaxf(amax, fabsf(v[u].x * w[u].x)), fmaxf(fabsf(v[u].y * w[u].y), fmaxf(fabsf(v[u].z * w[u].z), fabsf(v[u].w * w[u].w))));
        }
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
        int e = 0;
        if (top > 0.0f && isfinite(top)) frexpf(top, &e);   // top = f * 2^e, f in [0.5, 1)
        const float s = ldexpf(1.0f, 1 - e);                // top * s in [1, 2)
        scale_in[m] = s;
        member_scale[m] = inv_norm * ldexpf(1.0f, e - 1);
    }
}

// Pass 2: chunk c (64 inputs) = [k block 8][column group cols / 8][column 8][8 halves], columns
// [0, mp) the hi parts and [mp, 2 mp) the lo parts; padded members are zero.
__global__ void tc_chunks_kernel(const float* x, const int32_t* index, const float* norm_weight, int members, int mp,
                                 int k, const float* scale_in, __half* chunks) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (member, 8 inputs)
    const int kblocks = k / 8;
    if (id >= (long long)mp * kblocks) return;
    const int m = (int)(id / kblocks), kblk = (int)(id % kblocks);
    const int cols = 2 * mp;
    __half hi[8], lo[8];
    if (m < members) {
        const float* row = x + (size_t)(index ? index[m] : m) * k + (size_t)kblk * 8;
        const float s = scale_in[m];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float v = row[i];
            if (norm_weight != nullptr) v *= norm_weight[kblk * 8 + i];
            v *= s;
            hi[i] = __float2half_rn(v);
            lo[i] = __float2half_rn(v - __half2float(hi[i]));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) hi[i] = lo[i] = __float2half_rn(0.0f);
    }
    const int chunk = kblk / 8, kb8 = kblk % 8;
    __half* base = chunks + (size_t)chunk * (cols * kChunkK) + (size_t)kb8 * (cols * 8);
    *reinterpret_cast<uint4*>(base + (size_t)m * 8) = *reinterpret_cast<const uint4*>(hi);
    *reinterpret_cast<uint4*>(base + (size_t)(mp + m) * 8) = *reinterpret_cast<const uint4*>(lo);
}

// K-quant form of the activations: per k tile (256 inputs) four chunks as above, then the group sums
// [2 blocks][column][8 halves]: block 0 = sums of the eight 32-input groups, block 1 zeros.  blockIdx.y selects a
// group of `group` consecutive members (the last one may be shorter); each group gets its own operand,
// `group_halves` halves apart, laid out for its own padded member count.
// Both passes for the K-quant form in one launch: block (x = member within its group, y = group) first finds the
// member's scale as tc_scale_kernel does (same arithmetic and order), then writes the member's column of every
// chunk.  Columns past the group's member count (padding up to a multiple of 16) are zero.
__global__ void __launch_bounds__(512) tcq_operand_kernel(const float* x, const int32_t* index, const float* norm_weight,
                                                          int total_members, int group, int k, float eps, float* scale_in,
                                                          float* member_scale, __half* chunks, size_t group_halves) {
    __shared__ float red_max[32], red_sum[32];
    __shared__ float scale_slot;
    const int member0 = (int)blockIdx.y * group;
    const int members = min(group, total_members - member0);
    const int mp = (members + 15) / 16 * 16;
    const int m = blockIdx.x;
    if (m >= mp) return;
    const bool real = m < members;
    const float* row = real ? x + (size_t)(index ? index[member0 + m] : member0 + m) * k : nullptr;
    if (real) {
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const float4* nw = reinterpret_cast<const float4*>(norm_weight);
        float amax = 0.0f, ss = 0.0f;
        for (int i0 = threadIdx.x; i0 < k / 4; i0 += 4 * blockDim.x) {
            float4 v[4], w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * blockDim.x;
                v[u] = i < k / 4 ? row4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                w[u] = (nw != nullptr && i < k / 4) ? nw[i] : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                ss = fmaf(v[u].x, v[u].x, ss); ss = fmaf(v[u].y, v[u].y, ss); ss = fmaf(v[u].z, v[u].z, ss); ss = fmaf(v[u].w, v[u].w, ss);
                amax = fmaxf(fmaxf(amax, fabsf(v[u].x * w[u].x)), fmaxf(fabsf(v[u].y * w[u].y), fmaxf(fabsf(v[u].z * w[u].z), fabsf(v[u].w * w[u].w))));
            }
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
            int e = 0;
            if (top > 0.0f && isfinite(top)) frexpf(top, &e);
            const float sc = ldexpf(1.0f, 1 - e);
            scale_in[member0 + m] = sc;
            member_scale[member0 + m] = inv_norm * ldexpf(1.0f, e - 1);
            scale_slot = sc;
        }
        __syncthreads();
    }
    const float sc = real ? scale_slot : 0.0f;
    const int cols = 2 * mp, kblocks = k / 8;
    const size_t tile_halves = (size_t)kChunksPerTile * cols * kChunkK + (size_t)cols * 16;
    __half* out = chunks + (size_t)blockIdx.y * group_halves;
    for (int kblk = threadIdx.x; kblk < kblocks; kblk += blockDim.x) {   // kblocks is a multiple of 32: whole warps
        __half hi[8], lo[8];
        float sum = 0.0f;
        if (real) {
            const float* src = row + (size_t)kblk * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float v = src[i];
                if (norm_weight != nullptr) v *= norm_weight[kblk * 8 + i];
                v *= sc;
                hi[i] = __float2half_rn(v);
                lo[i] = __float2half_rn(v - __half2float(hi[i]));
                sum += __half2float(hi[i]) + __half2float(lo[i]);   // the sum of what the tensor core will see
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) hi[i] = lo[i] = __float2half_rn(0.0f);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);   // four consecutive threads hold one 32-input group
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int tile = kblk / 32, in_tile = kblk % 32, chunk = in_tile / 8, kb8 = in_tile % 8;
        __half* base = out + (size_t)tile * tile_halves;
        __half* cbase = base + (size_t)chunk * (cols * kChunkK) + (size_t)kb8 * (cols * 8);
        *reinterpret_cast<uint4*>(cbase + (size_t)m * 8) = *reinterpret_cast<const uint4*>(hi);
        *reinterpret_cast<uint4*>(cbase + (size_t)(mp + m) * 8) = *reinterpret_cast<const uint4*>(lo);
        __half* sums = base + (size_t)kChunksPerTile * cols * kChunkK;
        if ((in_tile & 3) == 0) {
            const int g = in_tile / 4;
            const __half sh = __float2half_rn(sum);
            sums[(size_t)m * 8 + g] = sh;
            sums[(size_t)(mp + m) * 8 + g] = __float2half_rn(sum - __half2float(sh));
        }
        if (in_tile == 0) {
            const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(sums + (size_t)cols * 8 + (size_t)m * 8) = zero;
            *reinterpret_cast<uint4*>(sums + (size_t)cols * 8 + (size_t)(mp + m) * 8) = zero;
        }
    }
}

int padded_members(int members) { return (members + 15) / 16 * 16; }

}  // namespace

size_t tc_operand_bytes(int members, int k) {
    const size_t cols = 2 * (size_t)padded_members(members);
    // chunks of 64 inputs, plus (K-quant form) 16 halves of group sums per column and k tile
    return ((size_t)(k / kChunkK) * cols * kChunkK + (size_t)(k / kTileCols) * cols * 16) * sizeof(__half);
}

bool gemm_tc_kquant(const GemvSegment* segments, int n_segments, int members) {
    if (members > kKqMaxMembers) return false;
    for (int i = 0; i < n_segments; ++i) {
        if (segments[i].type != kQ4_K && segments[i].type != kQ6_K) return false;
    }
    return true;
}

cudaError_t launch_to_tc_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                                 int members, int k, float eps, bool kquant, TcOperand out) {
    if (members <= 0 || members > (kquant ? kKqMaxMembers : kGemmTcMaxMembers) || k % kTileCols != 0) return cudaErrorInvalidValue;
    const int mp = padded_members(members);
    if (kquant) {
        tcq_operand_kernel<<<dim3((unsigned int)mp, 1), 512, 0, stream>>>(x, index, norm_weight, members, members, k, eps, out.scale_in,
                                                                          out.member_scale, out.chunks, 0);
        return cudaGetLastError();
    }
    tc_scale_kernel<<<members, 512, 0, stream>>>(x, index, norm_weight, k, eps, out.scale_in, out.member_scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const long long threads = (long long)mp * (k / 8);
    const unsigned int blocks = (unsigned int)((threads + 255) / 256);
    tc_chunks_kernel<<<blocks, 256, 0, stream>>>(x, index, norm_weight, members, mp, k, out.scale_in, out.chunks);
    return cudaGetLastError();
}

cudaError_t launch_to_tc_operand_groups(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                                        int members, int group, int k, float eps, TcOperand out) {
    if (members <= 0 || group <= 0 || group > kKqMaxMembers || k % kTileCols != 0) return cudaErrorInvalidValue;
    const int groups = (members + group - 1) / group;
    const dim3 grid((unsigned int)padded_members(std::min(group, members)), (unsigned int)groups);
    tcq_operand_kernel<<<grid, 512, 0, stream>>>(x, index, norm_weight, members, group, k, eps, out.scale_in, out.member_scale,
                                                 out.chunks, tc_operand_bytes(group, k) / sizeof(__half));
    return cudaGetLastError();
}

namespace {

thread_local int g_last_launches = 1;
constexpr size_t kTcSmemBudget = 220 * 1024;

// Function attributes are per device: the opt-in to large dynamic shared memory is made once on every device a
// process uses, and the SM count is kept per device ordinal.
cudaError_t device_setup(int& sm_count) {
    static int sms[kMaxDevices] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (sms[dev] == 0) {
        e = cudaFuncSetAttribute(gemm_tcq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBudget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBudget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcq2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBudget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcqc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBudget);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcqc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBudget);
        if (e != cudaSuccess) return e;
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0) count = 148;
        sms[dev] = count;
    }
    sm_count = sms[dev];
    return cudaSuccess;
}

// The K-quant GEMM over cached operands: every segment carries op_a / op_meta.
cudaError_t launch_gemm_tcqc(cudaStream_t stream, const GemmArgs& args, int units) {
    KqcLayout lay{};
    lay.members_padded = padded_members(args.members);
    lay.cols = 2 * lay.members_padded;
    lay.b_bytes = lay.cols * kChunkK * (int)sizeof(__half);
    lay.b2_bytes = lay.cols * 16 * (int)sizeof(__half);
    bool all_q4k = true;
    for (int i = 0; i < args.n_segments; ++i) all_q4k = all_q4k && args.seg[i].type == kQ4_K;
    // 32 KB of operand per stage: 128 inputs of the one Q4_K plane, or 64 inputs of two planes
    lay.pieces = all_q4k ? 2 : 1;
    lay.stage_bytes = 2 * kCachePieceBytes;
    lay.total_n = 0;
    for (int i = 0; i < args.n_segments; ++i) lay.total_n += args.seg[i].n;
    lay.k_slices = 1;
    lay.groups = std::max(1, args.groups);
    lay.group_bytes = args.group_chunk_bytes;
    int sm_count = 0;
    {
        cudaError_t e = device_setup(sm_count);
        if (e != cudaSuccess) return e;
    }
    // whole groups of 64 in pairs: one pass over the unit's operand stages (through L2 and shared memory) per pair
    const bool pairs = lay.groups >= 2 && args.members == kKqMaxMembers;
    const int per_item = pairs ? 2 : 1;
    lay.m_slots = 2;
    const size_t fixed = (size_t)lay.m_slots * (kCacheMetaBytes + (size_t)per_item * lay.b2_bytes) + 16 + 512;
    size_t per_stage = (size_t)lay.stage_bytes + (size_t)lay.pieces * per_item * lay.b_bytes;
    if (lay.pieces == 2 && (kTcSmemBudget - fixed) / per_stage < 3) {   // too few of the wide stages: 64 inputs per stage
        lay.pieces = 1;
        lay.stage_bytes = kCachePieceBytes;
        per_stage = (size_t)lay.stage_bytes + (size_t)per_item * lay.b_bytes;
    }
    lay.stages = (int)std::min<size_t>(16, (kTcSmemBudget - fixed) / per_stage);
    if (lay.stages < 2) return cudaErrorInvalidValue;
    const size_t smem = fixed + (size_t)lay.stages * per_stage;
    if (pairs) {
        KqcLayout two = lay;
        two.groups = lay.groups & ~1;
        gemm_tcqc_kernel<2><<<std::min(units * (two.groups / 2), sm_count), kKqcThreads, smem, stream>>>(args, two, units);
        cudaError_t e2 = cudaGetLastError();
        g_last_launches = 1;
        if (e2 != cudaSuccess || two.groups == lay.groups) return e2;
        // the odd group: its operand, scales and outputs follow the pairs'
        GemmArgs rest = args;
        rest.groups = 1;
        rest.chunks = args.chunks + (size_t)two.groups * lay.group_bytes;
        rest.member_scale = args.member_scale + (size_t)two.groups * args.members;
        for (int i = 0; i < rest.n_segments; ++i) rest.seg[i].y = args.seg[i].y + (size_t)two.groups * args.members * args.seg[i].n;
        rest.partial = nullptr;
        cudaError_t e3 = launch_gemm_tcqc(stream, rest, units);
        g_last_launches = 2;
        return e3;
    }
    // Split K when whole units would leave SMs idle (every SM then streams its own part of the operands).
    const int k_tiles = args.k / kTileCols;
    if (args.partial != nullptr && lay.groups == 1) {
        long long best = -1;
        for (int slices = 1; slices <= std::min(8, k_tiles); ++slices) {
            const int tps = (k_tiles + slices - 1) / slices;
            if ((slices - 1) * tps >= k_tiles) continue;  // an empty slice
            if ((size_t)slices * args.members * lay.total_n > args.partial_floats) break;
            const long long waves = ((long long)units * slices + sm_count - 1) / sm_count;
            const long long cost = waves * (tps + 1);
            if (best < 0 || cost < best) { best = cost; lay.k_slices = slices; }
        }
    }
    gemm_tcqc_kernel<1><<<std::min(units * lay.k_slices * lay.groups, sm_count), kKqcThreads, smem, stream>>>(args, lay, units);
    cudaError_t e = cudaGetLastError();
    g_last_launches = 1;
    if (e != cudaSuccess || lay.k_slices == 1) return e;
    g_last_launches = 2;
    const long long outputs = (long long)args.members * lay.total_n;
    tcq_reduce_kernel<<<(unsigned int)((outputs + 255) / 256), 256, 0, stream>>>(args, lay.k_slices, lay.total_n);
    return cudaGetLastError();
}

cudaError_t launch_gemm_tcq(cudaStream_t stream, const GemmArgs& args, int units, int tile) {
    {
        bool cached = true;
        for (int i = 0; i < args.n_segments; ++i) cached = cached && args.seg[i].op_a != nullptr && args.seg[i].op_meta != nullptr;
        if (cached) return launch_gemm_tcqc(stream, args, units);
    }
    KqLayout lay{};
    lay.members_padded = padded_members(args.members);
    lay.cols = 2 * lay.members_padded;
    lay.b_bytes = lay.cols * kChunkK * (int)sizeof(__half);
    lay.b2_bytes = lay.cols * 16 * (int)sizeof(__half);
    lay.w_stage_bytes = kRowTilesPerUnit * tile;
    const size_t budget = kTcSmemBudget;
    // 64 KB of A stages, two of them: 128 inputs of one plane when every unit is Q4_K, else 64 inputs of two planes
    bool all_q4k = true;
    for (int i = 0; i < args.n_segments; ++i) all_q4k = all_q4k && args.seg[i].type == kQ4_K;
    lay.a_planes = all_q4k ? 1 : 2;
    lay.a_stages = 2;
    lay.chunk_k = all_q4k ? 2 * kChunkK : kChunkK;
    size_t fixed = (size_t)4 * kAHalfBytes + (size_t)2 * kA2Bytes + (size_t)4 * lay.b_bytes + (size_t)2 * lay.b2_bytes +
                   (size_t)4 * kRows * sizeof(float2) + 16 + 384;
    lay.w_stages = (int)std::min<size_t>(3, (budget - fixed) / (size_t)lay.w_stage_bytes);
    if (lay.w_stages < 2) return cudaErrorInvalidValue;
    const size_t smem = fixed + (size_t)lay.w_stages * lay.w_stage_bytes;
    int sm_count = 0;
    {
        cudaError_t e = device_setup(sm_count);
        if (e != cudaSuccess) return e;
    }
    // Split K when whole units would leave SMs idle: pick the slice count with the fewest k tiles on the
    // busiest SM (each work item also pays about one k tile of pipeline fill).
    const int k_tiles = args.k / kTileCols;
    lay.total_n = 0;
    for (int i = 0; i < args.n_segments; ++i) lay.total_n += args.seg[i].n;
    lay.k_slices = 1;
    lay.groups = std::max(1, args.groups);
    lay.group_bytes = args.group_chunk_bytes;
    if (args.partial != nullptr && lay.groups == 1) {
        long long best = -1;
        for (int slices = 1; slices <= std::min(8, k_tiles); ++slices) {
            const int tps = (k_tiles + slices - 1) / slices;
            if ((slices - 1) * tps >= k_tiles) continue;  // an empty slice
            if ((size_t)slices * args.members * lay.total_n > args.partial_floats) break;
            const long long waves = ((long long)units * slices + sm_count - 1) / sm_count;
            const long long cost = waves * (tps + 1);
            if (best < 0 || cost < best) { best = cost; lay.k_slices = slices; }
        }
    }
    // Whole groups in pairs: one conversion of every weight stage per pair (an odd last group takes the kernel above).
    // A pair's item takes about 1.45 times a single group's, so pairs pay when they save waves of work items.
    const long long single_waves = ((long long)units * lay.groups + sm_count - 1) / sm_count;
    const long long pair_waves = ((long long)units * (lay.groups / 2) + sm_count - 1) / sm_count + (lay.groups & 1 ? (units + sm_count - 1) / sm_count : 0);
    if (lay.groups >= 2 && args.members == kKqMaxMembers && pair_waves * 29 < single_waves * 20) {
        KqLayout two = lay;
        two.a_stages = 2;
        two.chunk_k = kChunkK;
        two.groups = lay.groups & ~1;
        size_t fixed2 = (size_t)two.a_stages * two.a_planes * kAHalfBytes + (size_t)2 * kA2Bytes + (size_t)two.a_stages * 2 * two.b_bytes +
                        (size_t)4 * two.b2_bytes + (size_t)4 * kRows * sizeof(float2) + 16 + 384;
        two.w_stages = (int)std::min<size_t>(3, (budget - fixed2) / (size_t)two.w_stage_bytes);
        if (two.w_stages >= 2) {
            const size_t smem2 = fixed2 + (size_t)two.w_stages * two.w_stage_bytes;
            gemm_tcq2_kernel<<<std::min(units * (two.groups / 2), sm_count), kKq2Threads, smem2, stream>>>(args, two, units);
            cudaError_t e2 = cudaGetLastError();
            g_last_launches = 1;
            if (e2 != cudaSuccess || two.groups == lay.groups) return e2;
            // the odd group: its operand, scales and outputs follow the pairs'
            GemmArgs rest = args;
            rest.groups = 1;
            rest.chunks = args.chunks + (size_t)two.groups * lay.group_bytes;
            rest.member_scale = args.member_scale + (size_t)two.groups * args.members;
            for (int i = 0; i < rest.n_segments; ++i) rest.seg[i].y = args.seg[i].y + (size_t)two.groups * args.members * args.seg[i].n;
            rest.partial = nullptr;
            cudaError_t e3 = launch_gemm_tcq(stream, rest, units, tile);
            g_last_launches = 2;
            return e3;
        }
    }
    gemm_tcq_kernel<<<std::min(units * lay.k_slices * lay.groups, sm_count), kKqThreads, smem, stream>>>(args, lay, units);
    cudaError_t e = cudaGetLastError();
    g_last_launches = 1;
    if (e != cudaSuccess || lay.k_slices == 1) return e;
    g_last_launches = 2;
    const long long outputs = (long long)args.members * lay.total_n;
    tcq_reduce_kernel<<<(unsigned int)((outputs + 255) / 256), 256, 0, stream>>>(args, lay.k_slices, lay.total_n);
    return cudaGetLastError();
}

}  // namespace

int gemm_tc_last_launches() { return g_last_launches; }

cudaError_t launch_unpack_packed(cudaStream_t stream, int type, const unsigned char* packed, long long rows, long long cols,
                                 float* out) {
    if (!packable(type, rows, cols)) return cudaErrorInvalidValue;
    const long long tiles = ((rows + kTileRows - 1) / kTileRows) * (cols / kTileCols);
    unpack_packed_kernel<<<(unsigned int)tiles, 256, 0, stream>>>(type, packed, rows, (int)(cols / kTileCols), out);
    return cudaGetLastError();
}

cudaError_t launch_gemm_tc(cudaStream_t stream, const GemmArgs& args) {
    g_last_launches = 1;
    if (args.members < 1 || args.members > kGemmTcMaxMembers || args.k % kTileCols != 0) return cudaErrorInvalidValue;
    if (args.epilogue != kStore && args.epilogue != kResidual) return cudaErrorInvalidValue;
    int units = 0, tile = 0;
    for (int i = 0; i < args.n_segments; ++i) {
        units += (args.seg[i].row_tiles + kRowTilesPerUnit - 1) / kRowTilesPerUnit;
        const int b = packed_tile_bytes(args.seg[i].type);
        if (b == 0) return cudaErrorInvalidValue;
        tile = std::max(tile, b);
    }
    if (units <= 0) return cudaSuccess;
    if (args.kquant) {
        if (!gemm_tc_kquant(args.seg, args.n_segments, args.members)) return cudaErrorInvalidValue;
        return launch_gemm_tcq(stream, args, units, tile);
    }
    TcLayout lay{};
    lay.members_padded = padded_members(args.members);
    lay.cols = 2 * lay.members_padded;
    lay.b_bytes = lay.cols * kChunkK * (int)sizeof(__half);
    lay.w_stage_bytes = kRowTilesPerUnit * tile;
    // Two activation chunks at least; what is left after three weight stages deepens the activation ring
    // (its copies have a longer way than the tensor core needs for a chunk).
    const size_t budget = kTcSmemBudget;
    size_t fixed = (size_t)2 * kABytes + (size_t)2 * lay.b_bytes + 16 + 320;
    lay.w_stages = (int)std::min<size_t>(3, (budget - fixed) / (size_t)lay.w_stage_bytes);
    if (lay.w_stages < 2) return cudaErrorInvalidValue;
    lay.b_stages = 2 + (int)std::min<size_t>(6, (budget - fixed - (size_t)lay.w_stages * lay.w_stage_bytes) / (size_t)lay.b_bytes);
    fixed += (size_t)(lay.b_stages - 2) * lay.b_bytes;
    const size_t smem = fixed + (size_t)lay.w_stages * lay.w_stage_bytes;
    int sm_count = 0;
    {
        cudaError_t e = device_setup(sm_count);
        if (e != cudaSuccess) return e;
    }
    const int grid = std::min(units, sm_count);
    gemm_tc_kernel<<<grid, kThreads, smem, stream>>>(args, lay, units);
    return cudaGetLastError();
}

}  // namespace ribn
