// Gemma-4 text decoder for B200: the reference host decoder's arithmetic policy (BF16 storage, FP32
// arithmetic, one BF16 round-to-nearest-even after every operation; crates/gemma4/src/cpu) run as CUDA
// kernels over rows of any number of sequences at once, so every weight matrix is read once per step.
//
// All of this work is BF16 streaming: projections are row-tile GEMVs with 128-bit loads; normalisation,
// rotary, GeGLU and the per-layer-embedding steps are fused per row around them; attention reads each
// owner layer's cache once per (row, head).  Every FP32 sum keeps the reference's source order (see the
// note above the kernels), which is what keeps the BF16-rounded results equal to the reference's.  Rotary
// cos / sin factors are tabulated on the host with the same libm calls the reference makes, so they are
// bit-identical to its BF16 factors.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "../../include/ribn_b200_gemma.h"

namespace {

typedef uint16_t bf16_t;

__host__ __device__ __forceinline__ float bf_load(bf16_t bits) {
#ifdef __CUDA_ARCH__
    return __uint_as_float((uint32_t)bits << 16);
#else
    uint32_t u = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

// crates/gemma4/src/cpu/linear.rs:10-16
__host__ __device__ __forceinline__ bf16_t bf_round(float value) {
#ifdef __CUDA_ARCH__
    const uint32_t bits = __float_as_uint(value);
#else
    uint32_t bits;
    memcpy(&bits, &value, 4);
#endif
    if ((bits & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    return (bf16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

// The reference rounds to BF16 after every operation and leaves attention scores unscaled, so a single
// FP32 ULP in a sum can move a rounded score by a whole BF16 step and, through the softmax, the output by
// tens of percent.  Every FP32 sum below therefore adds its terms in the reference's own (source) order:
// one thread owns each sum, and parallelism comes from the many independent sums (output columns, keys,
// channels, rows), not from splitting one.  A product of two BF16 values is exact in FP32, so an FMA
// equals the reference's multiply-then-add.  Transcendentals are evaluated in double and rounded once,
// which is what the host libm's float routines return in all but rare cases.

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float m = scratch[0];
    for (int w = 1; w < warps; ++w) m = fmaxf(m, scratch[w]);
    return m;
}

// Sum of squares of values[0 .. n) in index order by thread 0, broadcast to the block.  `squares` is a
// shared staging array of n floats the whole block fills first (each square is exact).
__device__ __forceinline__ float ordered_energy(const float* squares, int n, float* slot) {
    __syncthreads();
    if (threadIdx.x == 0) {
        // 128-bit reads run ahead of the additions; the additions themselves stay in index order
        const float4* quads = reinterpret_cast<const float4*>(squares);
        float energy = 0.0f;
#pragma unroll 8
        for (int i = 0; i < n / 4; ++i) {
            const float4 v = quads[i];
            energy += v.x; energy += v.y; energy += v.z; energy += v.w;
        }
        for (int i = n & ~3; i < n; ++i) energy += squares[i];
        *slot = energy;
    }
    __syncthreads();
    return *slot;
}

// x^(-1/2) rounded once from double (norm.rs:66 calls powf(mean + eps, -0.5)).
__device__ __forceinline__ float inverse_root(float x) { return (float)(1.0 / sqrt((double)x)); }

// elementwise.rs:66-83
__device__ __forceinline__ bf16_t gelu_round(bf16_t v) {
    const float x = bf_load(v);
    // separately rounded operations, as the reference's source-order FP32 expression (no contraction to FMA)
    const float cubic = __fadd_rn(1.0f, __fmul_rn(__fmul_rn(0.044715f, x), x));
    const float inner = __fmul_rn(__fmul_rn(0.7978846f, x), cubic);
    const float hyperbolic = (float)tanh((double)inner);
    return bf_round(__fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, hyperbolic)));
}

// ---------------------------------------------------------------------------------------------
// Embedding rows: hidden = bf16(embed[token] * sqrt(H) as BF16), identity = bf16(ple_embed[token] * sqrt(P) as BF16)
// (decoder.rs:346-360).  One block per row.
// ---------------------------------------------------------------------------------------------
__global__ void gm_embed_kernel(const uint32_t* tokens, const bf16_t* embed, const bf16_t* ple_embed, int hidden, int packed,
                                float embed_scale, float ple_scale, bf16_t* out_hidden, bf16_t* out_identity) {
    const int row = blockIdx.x;
    const size_t token = tokens[row];
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        out_hidden[(size_t)row * hidden + i] = bf_round(bf_load(embed[token * hidden + i]) * embed_scale);
    }
    for (int i = threadIdx.x; i < packed; i += blockDim.x) {
        out_identity[(size_t)row * packed + i] = bf_round(bf_load(ple_embed[token * packed + i]) * ple_scale);
    }
}

// ---------------------------------------------------------------------------------------------
// Projection: out[r][n] = bf16(sum_k in[r][k] * w[n][k]) (linear.rs:23-66), the sum in k order.  One warp
// per block; a thread owns one output column for a tile of RT rows and keeps RT independent accumulation
// chains.  Weights and input rows arrive in 256-input tiles through a two- or three-stage cp.async pipeline: the
// warp copies 32 weight-row segments of 512 bytes each (coalesced, L2-only) plus the RT input segments,
// then each thread walks its own row of the tile in shared memory (rows are pitched by 528 bytes, so the
// 128-bit reads of a quarter-warp fall in distinct banks; the input segment is a broadcast read).
// ---------------------------------------------------------------------------------------------
constexpr int kProjectCols = 32;                        // output columns (= threads) per block
// 16-byte chunks per row per tile: 256 inputs, or 128 for eight-row tiles (prefill), whose stages then fit eight
// blocks per SM: those tiles are bound by instruction issue and want two warps per scheduler
__host__ __device__ constexpr int project_tile_chunks(int rt) { return rt >= 8 ? 16 : 32; }
__host__ __device__ constexpr int project_stages(int rt) { return rt >= 8 ? 2 : 3; }  // an 8-row tile spends longer per stage
__host__ __device__ constexpr int project_row_pitch(int rt) { return project_tile_chunks(rt) * 16 + 16; }  // bytes between weight rows of a tile

__host__ __device__ constexpr int project_stage_bytes(int rt) {
    return rt * project_tile_chunks(rt) * 16 + kProjectCols * project_row_pitch(rt);
}
// all stages, then the current tile's input rows expanded to FP32 (one conversion per value instead of one per column)
__host__ __device__ constexpr int project_smem_bytes(int rt) {
    return project_stages(rt) * project_stage_bytes(rt) + rt * project_tile_chunks(rt) * 32;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// Up to three matrices that read the same input rows share one launch (q | k | v, gate | up): their
// column blocks are laid side by side in the grid.
struct ProjectTargets {
    const bf16_t* w[3];
    bf16_t* out[3];
    int n[3];
    int first_block[3];  // first column block of each matrix
    int count;
};

template <int RT>
__global__ void __launch_bounds__(kProjectCols) gm_project_kernel(const bf16_t* __restrict__ in,
                                                                  const int* __restrict__ row_index, int rows,
                                                                  const ProjectTargets targets, int k) {
    extern __shared__ __align__(16) unsigned char project_smem[];
    constexpr int kStageBytes = project_stage_bytes(RT);
    constexpr int kProjectStages = project_stages(RT);
    constexpr int kTileChunks = project_tile_chunks(RT);
    constexpr int kRowPitch = project_row_pitch(RT);
    constexpr int kRowsPerIssue = 32 / kTileChunks;  // rows one warp-wide copy instruction covers
    const int lane = threadIdx.x;
    const int piece = lane % kTileChunks, sub_row = lane / kTileChunks;
    int which = 0;
    if (targets.count > 1 && (int)blockIdx.x >= targets.first_block[1]) which = 1;
    if (targets.count > 2 && (int)blockIdx.x >= targets.first_block[2]) which = 2;
    const bf16_t* __restrict__ w = targets.w[which];
    bf16_t* __restrict__ out = targets.out[which];
    const int n = targets.n[which];
    const int col0 = ((int)blockIdx.x - targets.first_block[which]) * kProjectCols, col = col0 + lane;
    const int r0 = blockIdx.y * RT;
    const int live_cols = min(kProjectCols, n - col0);
    const uint4* x[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const int row = min(r0 + r, rows - 1);
        x[r] = reinterpret_cast<const uint4*>(in + (size_t)(row_index ? row_index[row] : row) * k);
    }
    const uint4* wbase = reinterpret_cast<const uint4*>(w + (size_t)col0 * k);
    const int chunks = k / 8, row_chunks = chunks;  // 16-byte chunks per weight row
    const int tiles = (chunks + kTileChunks - 1) / kTileChunks;
    const uint32_t smem = (uint32_t)__cvta_generic_to_shared(project_smem);

    auto issue = [&](int tile) {
        if (tile < tiles) {
            const int c = tile * kTileChunks + piece;  // this lane's chunk of its row segments
            if (c < chunks) {
                const uint32_t stage = smem + (uint32_t)((tile % kProjectStages) * kStageBytes);
#pragma unroll
                for (int r = 0; r < RT; ++r) {  // static indices keep the row pointers in registers
                    if (r % kRowsPerIssue == sub_row) cp_async16(stage + (uint32_t)(r * kTileChunks * 16 + piece * 16), x[r] + c);
                }
                uint32_t wdst = stage + (uint32_t)(RT * kTileChunks * 16 + sub_row * kRowPitch + piece * 16);
                const uint4* src = wbase + (size_t)sub_row * row_chunks + c;
                for (int j = sub_row; j < live_cols; j += kRowsPerIssue, wdst += kRowsPerIssue * kRowPitch,
                         src += (size_t)kRowsPerIssue * row_chunks) {
                    cp_async16(wdst, src);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = 0.0f;
#pragma unroll
    for (int s = 0; s < kProjectStages - 1; ++s) issue(s);
    for (int tile = 0; tile < tiles; ++tile) {
        issue(tile + kProjectStages - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(kProjectStages - 1) : "memory");
        __syncwarp();
        const unsigned char* stage = project_smem + (size_t)(tile % kProjectStages) * kStageBytes;
        const uint4* ws = reinterpret_cast<const uint4*>(stage + RT * kTileChunks * 16 + lane * kRowPitch);
        const int count = min(kTileChunks, chunks - tile * kTileChunks);
        // lane l expands chunk l of every input row to FP32
        float4* xf = reinterpret_cast<float4*>(project_smem + kProjectStages * kStageBytes);
        if (lane < count) {
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                const uint4 xv = reinterpret_cast<const uint4*>(stage)[r * kTileChunks + lane];
                xf[(r * kTileChunks + lane) * 2] = make_float4(__uint_as_float(xv.x << 16), __uint_as_float(xv.x & 0xffff0000u),
                                                               __uint_as_float(xv.y << 16), __uint_as_float(xv.y & 0xffff0000u));
                xf[(r * kTileChunks + lane) * 2 + 1] = make_float4(__uint_as_float(xv.z << 16), __uint_as_float(xv.z & 0xffff0000u),
                                                                   __uint_as_float(xv.w << 16), __uint_as_float(xv.w & 0xffff0000u));
            }
        }
        __syncwarp();
        if (lane < live_cols) {
#pragma unroll 4
            for (int i = 0; i < count; ++i) {
                const uint4 wv = ws[i];
                const float w0 = __uint_as_float(wv.x << 16), w1 = __uint_as_float(wv.x & 0xffff0000u);
                const float w2 = __uint_as_float(wv.y << 16), w3 = __uint_as_float(wv.y & 0xffff0000u);
                const float w4 = __uint_as_float(wv.z << 16), w5 = __uint_as_float(wv.z & 0xffff0000u);
                const float w6 = __uint_as_float(wv.w << 16), w7 = __uint_as_float(wv.w & 0xffff0000u);
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    const float4 a = xf[(r * kTileChunks + i) * 2], b = xf[(r * kTileChunks + i) * 2 + 1];
                    acc[r] = fmaf(a.x, w0, acc[r]); acc[r] = fmaf(a.y, w1, acc[r]);
                    acc[r] = fmaf(a.z, w2, acc[r]); acc[r] = fmaf(a.w, w3, acc[r]);
                    acc[r] = fmaf(b.x, w4, acc[r]); acc[r] = fmaf(b.y, w5, acc[r]);
                    acc[r] = fmaf(b.z, w6, acc[r]); acc[r] = fmaf(b.w, w7, acc[r]);
                }
            }
        }
        __syncwarp();  // every lane has left this stage (and the expanded rows) before they are overwritten
    }
    if (lane < live_cols) {
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            if (r0 + r < rows) out[(size_t)(r0 + r) * n + col] = bf_round(acc[r]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same projection on the tensor cores, for passes of many rows when the model was created with
// RIBN_B200_GEMMA_FLAG_TENSOR_CORE_PREFILL: BF16 x BF16 products (exact in FP32) accumulated in FP32 by
// `mma.sync.m16n8k16`, one BF16 rounding of each output.  The sums are no longer in source order, so a result
// can differ from the host decoder's by a rounding step of the FP32 sum before the BF16 rounding; the
// ordered kernel above stays the default.  A block of four warps owns 64 rows x 64 columns; warp w owns rows
// 16 w .. 16 w + 15 against all 64 columns.  Inputs and weights arrive in 32-input stages (rows pitched by 80
// bytes: conflict-free matrix loads) through a two-stage cp.async pipeline.  k must be a multiple of 32.
// ---------------------------------------------------------------------------------------------
constexpr int kMmaTile = 64;           // rows and columns per block
constexpr int kMmaStageK = 32;         // inputs per stage
constexpr int kMmaPitch = kMmaStageK * 2 + 16;   // bytes between rows of a stage
constexpr int kMmaStageBytes = 2 * kMmaTile * kMmaPitch;  // input rows, then weight rows

__global__ void __launch_bounds__(128) gm_project_mma_kernel(const bf16_t* __restrict__ in, const int* __restrict__ row_index,
                                                             int rows, const ProjectTargets targets, int k) {
    __shared__ __align__(16) unsigned char stage_smem[2 * kMmaStageBytes];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int which = 0;
    if (targets.count > 1 && (int)blockIdx.x >= targets.first_block[1]) which = 1;
    if (targets.count > 2 && (int)blockIdx.x >= targets.first_block[2]) which = 2;
    const bf16_t* __restrict__ w = targets.w[which];
    bf16_t* __restrict__ out = targets.out[which];
    const int n = targets.n[which];
    const int col0 = ((int)blockIdx.x - targets.first_block[which]) * kMmaTile;
    const int r0 = blockIdx.y * kMmaTile;
    const uint32_t smem = (uint32_t)__cvta_generic_to_shared(stage_smem);
    // copies: a stage holds 64 + 64 rows of 64 bytes = 512 pieces of 16 bytes, four per thread
    const unsigned char* src[4];
    uint32_t dst[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int piece = (int)threadIdx.x + 128 * j, row = piece >> 2, part = piece & 3;   // rows 0..63 inputs, 64..127 weights
        if (row < kMmaTile) {
            const int r = min(r0 + row, rows - 1);
            src[j] = reinterpret_cast<const unsigned char*>(in + (size_t)(row_index ? row_index[r] : r) * k) + part * 16;
        } else {
            const int c = min(col0 + row - kMmaTile, n - 1);
            src[j] = reinterpret_cast<const unsigned char*>(w + (size_t)c * k) + part * 16;
        }
        dst[j] = (uint32_t)(row * kMmaPitch + part * 16);
    }
    const int stages = k / kMmaStageK;
    auto issue = [&](int st) {
        if (st < stages) {
#pragma unroll
            for (int j = 0; j < 4; ++j) cp_async16(smem + (uint32_t)((st & 1) * kMmaStageBytes) + dst[j], src[j] + (size_t)st * (kMmaStageK * 2));
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[8][4];
#pragma unroll
    for (int t = 0; t < 8; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f; }
    // matrix-load offsets: A = this warp's 16 input rows; B = weight rows (the MMA's columns), two column tiles per load
    const uint32_t a_off = (uint32_t)((warp * 16 + (lane & 15)) * kMmaPitch + (lane >> 4) * 16);
    const uint32_t b_off = (uint32_t)((kMmaTile + (lane & 7) + (lane >> 4) * 8) * kMmaPitch + ((lane >> 3) & 1) * 16);
    issue(0);
    for (int st = 0; st < stages; ++st) {
        issue(st + 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const uint32_t base = smem + (uint32_t)((st & 1) * kMmaStageBytes);
#pragma unroll
        for (int ks = 0; ks < kMmaStageK / 16; ++ks) {
            uint32_t a[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                         : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(base + a_off + ks * 32));
#pragma unroll
            for (int t2 = 0; t2 < 4; ++t2) {
                uint32_t b[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(base + b_off + t2 * (16 * kMmaPitch) + ks * 32));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                             : "+f"(acc[2 * t2][0]), "+f"(acc[2 * t2][1]), "+f"(acc[2 * t2][2]), "+f"(acc[2 * t2][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                             : "+f"(acc[2 * t2 + 1][0]), "+f"(acc[2 * t2 + 1][1]), "+f"(acc[2 * t2 + 1][2]), "+f"(acc[2 * t2 + 1][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[2]), "r"(b[3]));
            }
        }
        __syncthreads();  // every warp has read this stage before the copies of stage st + 2 land in it
    }
    // accumulator layout: rows g and g + 8 of the warp's 16, columns 8 t + 2 t4 + {0, 1}
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const int c = col0 + t * 8 + 2 * t4;
        const int ra = r0 + warp * 16 + g, rb = ra + 8;
        if (ra < rows) {
            if (c < n) out[(size_t)ra * n + c] = bf_round(acc[t][0]);
            if (c + 1 < n) out[(size_t)ra * n + c + 1] = bf_round(acc[t][1]);
        }
        if (rb < rows) {
            if (c < n) out[(size_t)rb * n + c] = bf_round(acc[t][2]);
            if (c + 1 < n) out[(size_t)rb * n + c + 1] = bf_round(acc[t][3]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Row RMS normalisation (norm.rs:38-82) with the decoder's follow-ups fused:
//   mode 0: out = bf16(x * inverse * scale)
//   mode 1: out = bf16(residual + mode 0)                         (post-norm + residual add)
//   mode 2: out = bf16(mode 1 * scalar)                           (end of a layer: layer scalar)
// row_index gathers input rows (the rows that want logits).  Dynamic shared memory: width floats.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gm_rms_kernel(const bf16_t* in, const int* row_index, int width, float eps,
                                                     const bf16_t* scale, const bf16_t* residual, const bf16_t* scalar,
                                                     int mode, bf16_t* out) {
    extern __shared__ __align__(16) float squares[];
    __shared__ float slot;
    const int row = blockIdx.x;
    const uint4* x = reinterpret_cast<const uint4*>(in + (size_t)(row_index ? row_index[row] : row) * width);
    const uint4* sc = reinterpret_cast<const uint4*>(scale);
    const uint4* res = reinterpret_cast<const uint4*>(residual + (mode >= 1 ? (size_t)row * width : 0));
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * width);
    const int chunks = width / 8;
    // Eight values per thread per trip; everything a trip needs is requested before the sum starts.
    for (int c0 = 0; c0 < chunks; c0 += blockDim.x) {
        const int c = c0 + threadIdx.x;
        if (c < chunks) {
            const uint4 v = __ldg(x + c);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
                squares[c * 8 + 2 * j] = lo * lo;
                squares[c * 8 + 2 * j + 1] = hi * hi;
            }
        }
    }
    const float energy = ordered_energy(squares, width, &slot);
    const float inverse = inverse_root(energy / (float)width + eps);
    const float factor = mode == 2 ? bf_load(scalar[0]) : 1.0f;
    for (int c0 = 0; c0 < chunks; c0 += blockDim.x) {
        const int c = c0 + threadIdx.x;
        if (c >= chunks) continue;
        const uint4 v = __ldg(x + c);
        const uint4 sv = scale ? __ldg(sc + c) : make_uint4(0, 0, 0, 0);
        const uint4 rv = mode >= 1 ? res[c] : make_uint4(0, 0, 0, 0);
        const uint32_t xw[4] = {v.x, v.y, v.z, v.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w}, rw[4] = {rv.x, rv.y, rv.z, rv.w};
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            bf16_t pair[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bf16_t xb = (bf16_t)(e ? xw[j] >> 16 : xw[j] & 0xffffu);
                float value = bf_load(xb) * inverse;
                if (scale) value *= bf_load((bf16_t)(e ? sw[j] >> 16 : sw[j] & 0xffffu));
                bf16_t r = bf_round(value);
                if (mode >= 1) r = bf_round(bf_load((bf16_t)(e ? rw[j] >> 16 : rw[j] & 0xffffu)) + bf_load(r));
                if (mode == 2) r = bf_round(bf_load(r) * factor);
                pair[e] = r;
            }
            ow[j] = (uint32_t)pair[0] | ((uint32_t)pair[1] << 16);
        }
        dst[c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// ---------------------------------------------------------------------------------------------
// Per-head normalisation, rotary and cache append (decoder.rs:488-530).  One block per (row, head slot):
// slots [0, heads) are queries (scaled norm + rotary -> q buffer), [heads, heads + kv) keys (scaled norm +
// rotary -> key cache at the row's position), the rest values (scale-free norm -> value cache).  Layers
// that do not own their cache launch only the query slots.
// Rotary (rotary.rs:95-140): each product rounds to BF16, the FP32 sum rounds to BF16; cos / sin come
// from the host-built BF16 table of this layer kind, [position][width / 2].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gm_head_kernel(const bf16_t* q_in, const bf16_t* k_in, const bf16_t* v_in,
                                                      const bf16_t* q_scale, const bf16_t* k_scale, const int* slot,
                                                      const int* position, const bf16_t* cosine, const bf16_t* sine,
                                                      int heads, int kv_heads, int width, float eps, int context,
                                                      bf16_t* q_out, bf16_t* key_cache, bf16_t* value_cache) {
    __shared__ __align__(16) float squares[512];
    __shared__ float energy_slot;
    __shared__ bf16_t normed[512];
    const int row = blockIdx.x, h = blockIdx.y, half = width / 2, pos = position[row];
    const bf16_t* x;
    const bf16_t* scale = nullptr;
    bf16_t* out;
    bool rotate = true;
    if (h < heads) {
        x = q_in + ((size_t)row * heads + h) * width;
        scale = q_scale;
        out = q_out + ((size_t)row * heads + h) * width;
    } else {
        const int kh = (h - heads) % kv_heads;
        const size_t at = (((size_t)slot[row] * context + pos) * kv_heads + kh) * width;
        if (h < heads + kv_heads) {
            x = k_in + ((size_t)row * kv_heads + kh) * width;
            scale = k_scale;
            out = key_cache + at;
        } else {
            x = v_in + ((size_t)row * kv_heads + kh) * width;
            out = value_cache + at;
            rotate = false;
        }
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = bf_load(x[i]);
        squares[i] = v * v;
    }
    const float energy = ordered_energy(squares, width, &energy_slot);
    const float inverse = inverse_root(energy / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = bf_load(x[i]) * inverse;
        if (scale) v *= bf_load(scale[i]);
        const bf16_t r = bf_round(v);
        if (rotate) normed[i] = r; else out[i] = r;
    }
    if (!rotate) return;
    __syncthreads();
    const bf16_t* c = cosine + (size_t)pos * half;
    const bf16_t* s = sine + (size_t)pos * half;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float a = bf_load(normed[j]), b = bf_load(normed[j + half]);
        const float cj = bf_load(c[j]), sj = bf_load(s[j]);
        const float first = bf_load(bf_round(a * cj)) + bf_load(bf_round(-b * sj));
        const float second = bf_load(bf_round(b * cj)) + bf_load(bf_round(a * sj));
        out[j] = bf_round(first);
        out[j + half] = bf_round(second);
    }
}

// ---------------------------------------------------------------------------------------------
// Attention (attention.rs:203-277).  One block per (row, query head).  Keys and values pass through shared
// memory in tiles of 64 positions, copied by the whole block with coalesced 128-bit loads (many loads in
// flight per thread: the kernel is bound by load latency, not by arithmetic).  Scores: one thread per key,
// the dot product in channel order, BF16 rounded, scaling 1.0.  Softmax in FP32 with the total added in key
// order; weights rounded to BF16; the output accumulates weight x value in FP32 over the keys in position
// order, one thread per channel.  window 0 = full attention.
// Dynamic shared memory: one float per visible key (rounded up to 16 bytes), then the tile.
// ---------------------------------------------------------------------------------------------
constexpr int kAttnTile = 64;

__host__ __device__ inline size_t attention_smem_bytes(int visible, int width) {
    return (((size_t)visible * sizeof(float) + 15) & ~(size_t)15) + (size_t)kAttnTile * ((size_t)width * 2 + 16);
}

// Copies rows [t0, t0 + count) of a cache (row stride `stride` elements, `chunks` 16-byte chunks used per
// row) into the tile, whose rows are pitched by 16 extra bytes.
__device__ __forceinline__ void attention_load_tile(const bf16_t* base, size_t stride, int t0, int count, int chunks,
                                                    unsigned char* tile, int pitch) {
    const int total = count * chunks;
    for (int first = 0; first < total; first += 8 * 256) {
        // eight requests per thread leave before the first value is stored
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = first + u * 256 + (int)threadIdx.x;
            if (idx < total) {
                const int key = idx / chunks, c = idx - key * chunks;
                v[u] = __ldg(reinterpret_cast<const uint4*>(base + (size_t)(t0 + key) * stride) + c);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = first + u * 256 + (int)threadIdx.x;
            if (idx < total) {
                const int key = idx / chunks, c = idx - key * chunks;
                *reinterpret_cast<uint4*>(tile + (size_t)key * pitch + (size_t)c * 16) = v[u];
            }
        }
    }
}

__global__ void __launch_bounds__(256, 1) gm_attention_kernel(const bf16_t* q, const int* slot, const int* position,
                                                              const bf16_t* key_cache, const bf16_t* value_cache, int heads,
                                                              int kv_heads, int width, int window, int context, bf16_t* out) {
    extern __shared__ __align__(16) unsigned char attention_smem[];
    __shared__ float scratch[8];
    __shared__ float total_slot;
    __shared__ uint4 query[64];  // up to 512 BF16 channels
    const int row = blockIdx.x, h = blockIdx.y, pos = position[row];
    const int kv_head = h / (heads / kv_heads);
    const int last = pos, first = window > 0 ? max(0, pos - (window - 1)) : 0;
    const int visible = last - first + 1;
    float* scores = reinterpret_cast<float*>(attention_smem);
    unsigned char* tile = attention_smem + (((size_t)visible * sizeof(float) + 15) & ~(size_t)15);
    const int pitch = width * 2 + 16;
    const size_t stride = (size_t)kv_heads * width;
    const bf16_t* kbase = key_cache + ((size_t)slot[row] * context + first) * stride + (size_t)kv_head * width;
    const bf16_t* vbase = value_cache + ((size_t)slot[row] * context + first) * stride + (size_t)kv_head * width;
    const int chunks = width / 8;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
        query[i] = reinterpret_cast<const uint4*>(q + ((size_t)row * heads + h) * width)[i];
    }
    float maximum = -INFINITY;
    for (int t0 = 0; t0 < visible; t0 += kAttnTile) {
        const int count = min(kAttnTile, visible - t0);
        __syncthreads();  // the previous tile has been consumed (and the query is in place)
        attention_load_tile(kbase, stride, t0, count, chunks, tile, pitch);
        __syncthreads();
        if ((int)threadIdx.x < count) {
            const uint4* key = reinterpret_cast<const uint4*>(tile + (size_t)threadIdx.x * pitch);
            float sum = 0.0f;
#pragma unroll 4
            for (int i = 0; i < chunks; ++i) {
                const uint4 kv = key[i];
                const uint4 qq = query[i];
                const uint32_t kk[4] = {kv.x, kv.y, kv.z, kv.w}, q4[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    sum = fmaf(__uint_as_float(q4[j] << 16), __uint_as_float(kk[j] << 16), sum);
                    sum = fmaf(__uint_as_float(q4[j] & 0xffff0000u), __uint_as_float(kk[j] & 0xffff0000u), sum);
                }
            }
            const float score = bf_load(bf_round(sum));
            scores[t0 + threadIdx.x] = score;
            maximum = fmaxf(maximum, score);
        }
    }
    maximum = block_max(maximum, scratch);  // its barriers also order the score writes before the reads below
    for (int t = threadIdx.x; t < visible; t += blockDim.x) scores[t] = (float)exp((double)(scores[t] - maximum));
    __syncthreads();
    if (threadIdx.x == 0) {
        const float4* quads = reinterpret_cast<const float4*>(scores);
        float total = 0.0f;
#pragma unroll 8
        for (int t = 0; t < visible / 4; ++t) {
            const float4 v = quads[t];
            total += v.x; total += v.y; total += v.z; total += v.w;
        }
        for (int t = visible & ~3; t < visible; ++t) total += scores[t];
        total_slot = total;
    }
    __syncthreads();
    const float total = total_slot;
    for (int t = threadIdx.x; t < visible; t += blockDim.x) scores[t] = bf_load(bf_round(scores[t] / total));
    // weight x value, two channels per thread at most (width <= 512)
    float acc[2] = {0.0f, 0.0f};
    for (int t0 = 0; t0 < visible; t0 += kAttnTile) {
        const int count = min(kAttnTile, visible - t0);
        __syncthreads();  // weights are final; the previous tile has been consumed
        attention_load_tile(vbase, stride, t0, count, chunks, tile, pitch);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = threadIdx.x + u * 256;
            if (c < width) {
                const bf16_t* column = reinterpret_cast<const bf16_t*>(tile) + c;
#pragma unroll 8
                for (int t = 0; t < count; ++t) acc[u] = fmaf(scores[t0 + t], bf_load(column[(size_t)t * (pitch / 2)]), acc[u]);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int c = threadIdx.x + u * 256;
        if (c < width) out[((size_t)row * heads + h) * width + c] = bf_round(acc[u]);
    }
}

// out = bf16(bf16(gelu(gate)) * other)   (decoder.rs:592-593 and 608-609)
__global__ void gm_gelu_mul_kernel(const bf16_t* gate, const bf16_t* other, size_t n, bf16_t* out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = bf_round(bf_load(gelu_round(gate[i])) * bf_load(other[i]));
}

// Per-layer inputs (decoder.rs:361-385): projection slice * 1/sqrt(H) (rounded), RMS with the shared
// per-layer norm (rounded), + token identity (rounded), * 2^-1/2 (rounded).  One block per (row, layer);
// out is [layer][row][ple].
__global__ void __launch_bounds__(256) gm_ple_kernel(const bf16_t* projection, const bf16_t* identity, const bf16_t* norm,
                                                     int rows, int ple, int packed, float projection_scale, float eps,
                                                     bf16_t* out) {
    __shared__ __align__(16) float squares[1024];
    __shared__ float energy_slot;
    __shared__ bf16_t scaled[1024];
    const int row = blockIdx.x, layer = blockIdx.y;
    const bf16_t* p = projection + (size_t)row * packed + (size_t)layer * ple;
    const bf16_t* id = identity + (size_t)row * packed + (size_t)layer * ple;
    for (int i = threadIdx.x; i < ple; i += blockDim.x) {
        const bf16_t s = bf_round(bf_load(p[i]) * projection_scale);
        scaled[i] = s;
        const float v = bf_load(s);
        squares[i] = v * v;
    }
    const float energy = ordered_energy(squares, ple, &energy_slot);
    const float inverse = inverse_root(energy / (float)ple + eps);
    for (int i = threadIdx.x; i < ple; i += blockDim.x) {
        float v = bf_load(scaled[i]) * inverse;
        v *= bf_load(norm[i]);
        const bf16_t context = bf_round(v);
        const bf16_t sum = bf_round(bf_load(context) + bf_load(id[i]));
        out[((size_t)layer * rows + row) * ple + i] = bf_round(bf_load(sum) * 0.70710678118654752440f);
    }
}

// Soft cap (elementwise.rs:85-107): divide, tanh, multiply, each rounded.
__global__ void gm_softcap_kernel(bf16_t* logits, size_t n, float cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const bf16_t divided = bf_round(__fdiv_rn(bf_load(logits[i]), cap));
    const bf16_t hyperbolic = bf_round((float)tanh((double)bf_load(divided)));
    logits[i] = bf_round(bf_load(hyperbolic) * cap);
}

// Greedy choice (decoder.rs:316-332): the first maximum; a NaN never beats the incumbent, and a NaN in
// element 0 is never replaced.  One block per row.
__global__ void __launch_bounds__(1024) gm_argmax_kernel(const bf16_t* logits, int vocab, uint32_t* out) {
    __shared__ float best_value[32];
    __shared__ int best_index[32];
    const bf16_t* x = logits + (size_t)blockIdx.x * vocab;
    const float head = bf_load(x[0]);
    if (head != head) {  // nothing compares greater than a NaN incumbent
        if (threadIdx.x == 0) out[blockIdx.x] = 0;
        return;
    }
    float value = -INFINITY;
    int index = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = bf_load(x[i]);
        if (v > value || (v == value && i < index)) { value = v; index = i; }
    }
    // -inf everywhere keeps index 0 (the incumbent), as the sequential scan does
    if (index == 0x7fffffff) index = 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, value, o);
        const int oi = __shfl_xor_sync(0xffffffffu, index, o);
        if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (warp == 0) {
        const int warps = blockDim.x >> 5;
        value = lane < warps ? best_value[lane] : -INFINITY;
        index = lane < warps ? best_index[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, value, o);
            const int oi = __shfl_xor_sync(0xffffffffu, index, o);
            if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
        }
        if (lane == 0) out[blockIdx.x] = (uint32_t)index;
    }
}

// Seeded N(0, sigma) values rounded to BF16 (counter-based: SplitMix64 of (seed, index), Box-Muller).
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__global__ void gm_normal_kernel(bf16_t* out, size_t n, uint64_t seed, float sigma) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t r = splitmix64(seed ^ splitmix64(i));
    const float u1 = ((float)(uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = (float)(uint32_t)((r >> 8) & 0xffffffu) * (1.0f / 16777216.0f);
    out[i] = bf_round(sigma * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2));
}
__global__ void gm_fill_kernel(bf16_t* out, size_t n, bf16_t value) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = value;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
enum { G_EMBED, G_PLE_EMBED, G_PLE_PROJ, G_PLE_NORM, G_NORM, G_COUNT };
enum { L_Q, L_K, L_V, L_O, L_QNORM, L_KNORM, L_IN, L_POST_ATTN, L_PRE_FFN, L_POST_FFN, L_GATE, L_UP, L_DOWN, L_PLE_GATE,
       L_PLE_PROJ, L_POST_PLE, L_SCALAR, L_COUNT };
const char* const kGlobalNames[G_COUNT] = {"embed_tokens", "embed_tokens_per_layer", "per_layer_model_projection",
                                           "per_layer_projection_norm", "norm"};
const char* const kLayerNames[L_COUNT] = {"q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "input_layernorm",
                                          "post_attention_layernorm", "pre_feedforward_layernorm",
                                          "post_feedforward_layernorm", "gate_proj", "up_proj", "down_proj",
                                          "per_layer_input_gate", "per_layer_projection", "post_per_layer_input_norm",
                                          "layer_scalar"};

struct Tensor {
    bf16_t* data = nullptr;
    size_t count = 0;
    bool loaded = false;
};

struct Sequence {
    bool open = false;
    uint32_t position = 0;
};

}  // namespace

struct ribn_b200_gemma {
    ribn_b200_gemma_config cfg;
    int owner[RIBN_B200_GEMMA_MAX_LAYERS];
    int cache_of[RIBN_B200_GEMMA_MAX_LAYERS];  // owner layer -> index of its cache pair, -1 for consumers
    Tensor g[G_COUNT];
    Tensor l[RIBN_B200_GEMMA_MAX_LAYERS][L_COUNT];
    std::vector<bf16_t*> key_cache, value_cache;  // per owner: [max_sequences][context][kv_heads][width]
    bf16_t* cosine[2] = {nullptr, nullptr};       // [kind: 0 sliding, 1 full][context][width / 2]
    bf16_t* sine[2] = {nullptr, nullptr};
    std::vector<Sequence> seq;
    bool finalized = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // per-pass device buffers (rows = max_batch_tokens)
    uint32_t* d_tokens = nullptr;
    int *d_slot = nullptr, *d_position = nullptr, *d_out_rows = nullptr;
    bf16_t *hidden = nullptr, *mid = nullptr, *normed = nullptr, *q = nullptr, *q2 = nullptr, *k = nullptr, *v = nullptr,
           *attended = nullptr, *projected = nullptr, *gate = nullptr, *up = nullptr, *identity = nullptr,
           *projection = nullptr, *per_layer = nullptr, *ple_gate = nullptr, *logits = nullptr;
    uint32_t* d_choice = nullptr;
    // pinned staging
    uint32_t* h_tokens = nullptr;
    int *h_slot = nullptr, *h_position = nullptr, *h_out_rows = nullptr;
    uint32_t* h_choice = nullptr;
    int max_outputs = 0;
    std::string error;
    float last_ms = 0.0f;
    uint32_t last_launches = 0;
    // passes of a recurring shape (rows, outputs, context bucket) replay a captured graph
    struct PassGraph { cudaGraphExec_t exec = nullptr; uint32_t launches = 0; };
    std::map<uint64_t, PassGraph> graphs;
    std::map<uint64_t, int> graph_seen;
};

namespace {

int fail(ribn_b200_gemma* m, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (m) m->error = buf;
    return code;
}

int width_of(const ribn_b200_gemma_config& c, int layer) { return c.full[layer] ? c.global_head_dim : c.head_dim; }

size_t global_count(const ribn_b200_gemma_config& c, int id) {
    const size_t packed = (size_t)c.layers * c.ple;
    switch (id) {
        case G_EMBED: return (size_t)c.vocab * c.hidden;
        case G_PLE_EMBED: return (size_t)c.ple_vocab * packed;
        case G_PLE_PROJ: return packed * c.hidden;
        case G_PLE_NORM: return (size_t)c.ple;
        default: return (size_t)c.hidden;
    }
}

size_t layer_count(const ribn_b200_gemma_config& c, int layer, int id) {
    const size_t w = (size_t)width_of(c, layer), h = (size_t)c.hidden;
    switch (id) {
        case L_Q: case L_O: return (size_t)c.heads * w * h;
        case L_K: case L_V: return (size_t)c.kv_heads * w * h;
        case L_QNORM: case L_KNORM: return w;
        case L_GATE: case L_UP: case L_DOWN: return (size_t)c.ffn * h;
        case L_PLE_GATE: case L_PLE_PROJ: return (size_t)c.ple * h;
        case L_SCALAR: return 1;
        default: return h;
    }
}

bool is_matrix(int layer_id) {
    switch (layer_id) {
        case L_Q: case L_K: case L_V: case L_O: case L_GATE: case L_UP: case L_DOWN: case L_PLE_GATE: case L_PLE_PROJ: return true;
        default: return false;
    }
}

// name -> tensor slot and the element count the configuration implies; nullptr for an unknown name
Tensor* find_tensor(ribn_b200_gemma* m, const char* name, size_t* expect) {
    for (int i = 0; i < G_COUNT; ++i) {
        if (strcmp(name, kGlobalNames[i]) == 0) { *expect = global_count(m->cfg, i); return &m->g[i]; }
    }
    if (strncmp(name, "layers.", 7) == 0) {
        char* end = nullptr;
        const long layer = strtol(name + 7, &end, 10);
        if (end && *end == '.' && layer >= 0 && layer < m->cfg.layers) {
            for (int i = 0; i < L_COUNT; ++i) {
                if (strcmp(end + 1, kLayerNames[i]) == 0) {
                    const bool kv_only = i == L_K || i == L_V || i == L_KNORM;
                    if (kv_only && m->owner[layer] != (int)layer) return nullptr;  // consumers hold no key / value weights
                    *expect = layer_count(m->cfg, (int)layer, i);
                    return &m->l[layer][i];
                }
            }
        }
    }
    return nullptr;
}

#define GM_CUDA(m, call)                                                                           \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) return fail((m), RIBN_B200_ERROR, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

template <typename T>
cudaError_t dev_alloc(T** p, size_t count) { return cudaMalloc((void**)p, sizeof(T) * (count ? count : 1)); }

int ensure_tensor(ribn_b200_gemma* m, Tensor* t, size_t count) {
    if (t->data == nullptr) {
        GM_CUDA(m, dev_alloc(&t->data, count));
        t->count = count;
    }
    return RIBN_B200_OK;
}

}  // namespace

extern "C" {

RIBN_B200_API int ribn_b200_gemma_create(const ribn_b200_gemma_config* config, ribn_b200_gemma** out, char* error,
                                         size_t error_capacity) {
    auto refuse = [&](const char* why) {
        if (error && error_capacity) snprintf(error, error_capacity, "%s", why);
        return RIBN_B200_ERROR;
    };
    if (!config || !out) return refuse("null argument");
    const ribn_b200_gemma_config& c = *config;
    if (c.layers <= 0 || c.layers > RIBN_B200_GEMMA_MAX_LAYERS || c.kv_shared < 0 || c.kv_shared >= c.layers) {
        return refuse("layer count or shared-layer count is invalid");
    }
    if (c.hidden <= 0 || c.heads <= 0 || c.kv_heads <= 0 || c.heads % c.kv_heads || c.ffn <= 0 || c.vocab <= 0 ||
        c.ple <= 0 || c.ple_vocab < c.vocab || c.window <= 0 || c.context <= 0 || c.max_sequences <= 0 ||
        c.max_batch_tokens <= 0) {
        return refuse("a model dimension or limit is not positive");
    }
    if (c.hidden % 8 || c.ffn % 8 || c.ple % 8 || c.head_dim % 8 || c.global_head_dim % 8 || c.head_dim > 512 ||
        c.global_head_dim > 512 || c.ple > 1024 || c.hidden > 12288) {
        return refuse("widths must be multiples of 8 (head widths at most 512, per-layer width at most 1024, hidden at most 12288)");
    }
    if (!(c.eps > 0.0f) || !(c.softcap > 0.0f) || !(c.theta_local > 0.0f) || !(c.theta_global > 0.0f)) {
        return refuse("epsilon, soft cap and rotary bases must be positive");
    }
    if (!c.full[c.layers - 1]) return refuse("the last layer must be full attention");
    if (c.context >= (1 << 24)) return refuse("positions must convert to FP32 exactly");
    int devices = 0;
    if (cudaGetDeviceCount(&devices) != cudaSuccess || devices <= 0 || c.device < 0 || c.device >= devices) {
        return refuse("no usable CUDA device (this library has no CPU path)");
    }
    if (cudaSetDevice(c.device) != cudaSuccess) return refuse("cudaSetDevice failed");
    ribn_b200_gemma* m = new ribn_b200_gemma();
    m->cfg = c;
    const int owners = c.layers - c.kv_shared;
    int caches = 0;
    for (int i = 0; i < c.layers; ++i) {
        int owner = i;
        if (i >= owners) {
            owner = -1;
            for (int j = owners - 1; j >= 0; --j) {
                if ((c.full[j] != 0) == (c.full[i] != 0)) { owner = j; break; }
            }
            if (owner < 0) { delete m; return refuse("a shared layer has no owner of its attention kind"); }
        }
        m->owner[i] = owner;
        m->cache_of[i] = owner == i ? caches++ : -1;
    }
    m->seq.resize((size_t)c.max_sequences);
    auto ok = [&](cudaError_t e) { return e == cudaSuccess; };
    const size_t R = (size_t)c.max_batch_tokens, H = (size_t)c.hidden, packed = (size_t)c.layers * c.ple;
    const size_t W = (size_t)(c.head_dim > c.global_head_dim ? c.head_dim : c.global_head_dim);
    m->max_outputs = c.max_sequences < c.max_batch_tokens ? c.max_sequences : c.max_batch_tokens;
    bool good = ok(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking)) && ok(cudaEventCreate(&m->ev0)) &&
                ok(cudaEventCreate(&m->ev1));
    good = good && ok(dev_alloc(&m->d_tokens, R)) && ok(dev_alloc(&m->d_slot, R)) && ok(dev_alloc(&m->d_position, R)) &&
           ok(dev_alloc(&m->d_out_rows, R)) && ok(dev_alloc(&m->hidden, R * H)) && ok(dev_alloc(&m->mid, R * H)) &&
           ok(dev_alloc(&m->normed, R * H)) && ok(dev_alloc(&m->q, R * c.heads * W)) &&
           ok(dev_alloc(&m->q2, R * c.heads * W)) && ok(dev_alloc(&m->k, R * c.kv_heads * W)) &&
           ok(dev_alloc(&m->v, R * c.kv_heads * W)) && ok(dev_alloc(&m->attended, R * c.heads * W)) &&
           ok(dev_alloc(&m->projected, R * H)) && ok(dev_alloc(&m->gate, R * c.ffn)) && ok(dev_alloc(&m->up, R * c.ffn)) &&
           ok(dev_alloc(&m->identity, R * packed)) && ok(dev_alloc(&m->projection, R * packed)) &&
           ok(dev_alloc(&m->per_layer, R * packed)) && ok(dev_alloc(&m->ple_gate, R * c.ple)) &&
           ok(dev_alloc(&m->logits, (size_t)m->max_outputs * c.vocab)) && ok(dev_alloc(&m->d_choice, (size_t)m->max_outputs));
    good = good && ok(cudaMallocHost((void**)&m->h_tokens, sizeof(uint32_t) * R)) &&
           ok(cudaMallocHost((void**)&m->h_slot, sizeof(int) * R)) && ok(cudaMallocHost((void**)&m->h_position, sizeof(int) * R)) &&
           ok(cudaMallocHost((void**)&m->h_out_rows, sizeof(int) * R)) &&
           ok(cudaMallocHost((void**)&m->h_choice, sizeof(uint32_t) * (size_t)m->max_outputs));
    for (int i = 0; i < c.layers && good; ++i) {
        if (m->cache_of[i] < 0) continue;
        const size_t n = (size_t)c.max_sequences * c.context * c.kv_heads * width_of(c, i);
        bf16_t *kc = nullptr, *vc = nullptr;
        good = ok(dev_alloc(&kc, n)) && ok(dev_alloc(&vc, n));
        m->key_cache.push_back(kc);
        m->value_cache.push_back(vc);
    }
    if (!good) {
        const char* why = cudaGetErrorString(cudaGetLastError());
        if (error && error_capacity) snprintf(error, error_capacity, "device allocation failed: %s", why);
        ribn_b200_gemma_destroy(m);
        return RIBN_B200_ERROR;
    }
    *out = m;
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_destroy(ribn_b200_gemma* m) {
    if (!m) return RIBN_B200_OK;
    if (m->stream) cudaStreamSynchronize(m->stream);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second.exec);
    for (auto& t : m->g) cudaFree(t.data);
    for (auto& layer : m->l) for (auto& t : layer) cudaFree(t.data);
    for (bf16_t* p : m->key_cache) cudaFree(p);
    for (bf16_t* p : m->value_cache) cudaFree(p);
    for (int i = 0; i < 2; ++i) { cudaFree(m->cosine[i]); cudaFree(m->sine[i]); }
    void* dev[] = {m->d_tokens, m->d_slot, m->d_position, m->d_out_rows, m->hidden, m->mid, m->normed, m->q, m->q2, m->k,
                   m->v, m->attended, m->projected, m->gate, m->up, m->identity, m->projection, m->per_layer, m->ple_gate,
                   m->logits, m->d_choice};
    for (void* p : dev) cudaFree(p);
    void* host[] = {m->h_tokens, m->h_slot, m->h_position, m->h_out_rows, m->h_choice};
    for (void* p : host) if (p) cudaFreeHost(p);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
    return RIBN_B200_OK;
}

RIBN_B200_API const char* ribn_b200_gemma_last_error(const ribn_b200_gemma* m) { return m ? m->error.c_str() : "null model"; }

RIBN_B200_API int ribn_b200_gemma_load_tensor(ribn_b200_gemma* m, const char* name, const uint16_t* values, size_t count) {
    if (!m || !name || !values) return RIBN_B200_ERROR;
    if (m->finalized) return fail(m, RIBN_B200_ERROR, "tensors cannot change after finalize");
    size_t expect = 0;
    Tensor* t = find_tensor(m, name, &expect);
    if (!t) return fail(m, RIBN_B200_ERROR, "unknown tensor name '%s'", name);
    if (count != expect) return fail(m, RIBN_B200_ERROR, "tensor '%s' has %zu elements, the configuration implies %zu", name, count, expect);
    if (int rc = ensure_tensor(m, t, expect)) return rc;
    GM_CUDA(m, cudaMemcpy(t->data, values, sizeof(bf16_t) * count, cudaMemcpyHostToDevice));
    t->loaded = true;
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_init_synthetic(ribn_b200_gemma* m, uint64_t seed) {
    if (!m) return RIBN_B200_ERROR;
    if (m->finalized) return fail(m, RIBN_B200_ERROR, "tensors cannot change after finalize");
    uint64_t index = 0;
    auto fill = [&](Tensor* t, size_t count, bool matrix) -> int {
        if (int rc = ensure_tensor(m, t, count)) return rc;
        const unsigned blocks = (unsigned)((count + 255) / 256);
        if (matrix) gm_normal_kernel<<<blocks, 256, 0, m->stream>>>(t->data, count, seed * 0x100000001B3ull + (++index) * 0x9E3779B97F4A7C15ull, 0.02f);
        else gm_fill_kernel<<<blocks, 256, 0, m->stream>>>(t->data, count, (bf16_t)0x3f80);
        t->loaded = true;
        return RIBN_B200_OK;
    };
    for (int i = 0; i < G_COUNT; ++i) {
        if (int rc = fill(&m->g[i], global_count(m->cfg, i), i == G_EMBED || i == G_PLE_EMBED || i == G_PLE_PROJ)) return rc;
    }
    for (int l = 0; l < m->cfg.layers; ++l) {
        for (int i = 0; i < L_COUNT; ++i) {
            const bool kv_only = i == L_K || i == L_V || i == L_KNORM;
            if (kv_only && m->owner[l] != l) continue;
            if (int rc = fill(&m->l[l][i], layer_count(m->cfg, l, i), is_matrix(i))) return rc;
        }
    }
    GM_CUDA(m, cudaStreamSynchronize(m->stream));
    GM_CUDA(m, cudaGetLastError());
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_read_tensor(ribn_b200_gemma* m, const char* name, uint16_t* out, size_t capacity,
                                              size_t* count) {
    if (!m || !name) return RIBN_B200_ERROR;
    size_t expect = 0;
    Tensor* t = find_tensor(m, name, &expect);
    if (!t || !t->loaded) return fail(m, RIBN_B200_ERROR, "tensor '%s' is not loaded", name);
    if (count) *count = expect;
    if (!out) return RIBN_B200_OK;
    if (capacity < expect) return fail(m, RIBN_B200_ERROR, "buffer holds %zu elements, '%s' has %zu", capacity, name, expect);
    GM_CUDA(m, cudaMemcpy(out, t->data, sizeof(bf16_t) * expect, cudaMemcpyDeviceToHost));
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_finalize(ribn_b200_gemma* m) {
    if (!m) return RIBN_B200_ERROR;
    if (m->finalized) return RIBN_B200_OK;
    const ribn_b200_gemma_config& c = m->cfg;
    for (int i = 0; i < G_COUNT; ++i) {
        if (!m->g[i].loaded) return fail(m, RIBN_B200_ERROR, "missing tensor '%s'", kGlobalNames[i]);
    }
    for (int l = 0; l < c.layers; ++l) {
        for (int i = 0; i < L_COUNT; ++i) {
            const bool kv_only = i == L_K || i == L_V || i == L_KNORM;
            if (kv_only && m->owner[l] != l) continue;
            if (!m->l[l][i].loaded) return fail(m, RIBN_B200_ERROR, "missing tensor 'layers.%d.%s'", l, kLayerNames[i]);
        }
    }
    // Rotary factor tables (rotary.rs:33-93, config.rs:200-247), with the host libm the reference's CPU path uses.
    for (int kind = 0; kind < 2; ++kind) {
        const int width = kind ? c.global_head_dim : c.head_dim, half = width / 2;
        const float theta = kind ? c.theta_global : c.theta_local;
        const int active = kind ? half / 4 : half;
        std::vector<float> frequency((size_t)half, 0.0f);
        for (int p = 0; p < active; ++p) {
            const float exponent = (float)(p * 2) / (float)width;
            frequency[(size_t)p] = 1.0f / powf(theta, exponent);
        }
        std::vector<bf16_t> cs((size_t)c.context * half), sn((size_t)c.context * half);
        for (int pos = 0; pos < c.context; ++pos) {
            for (int p = 0; p < half; ++p) {
                const float phase = (float)pos * frequency[(size_t)p];
                cs[(size_t)pos * half + p] = bf_round(cosf(phase));
                sn[(size_t)pos * half + p] = bf_round(sinf(phase));
            }
        }
        GM_CUDA(m, dev_alloc(&m->cosine[kind], cs.size()));
        GM_CUDA(m, dev_alloc(&m->sine[kind], sn.size()));
        GM_CUDA(m, cudaMemcpy(m->cosine[kind], cs.data(), sizeof(bf16_t) * cs.size(), cudaMemcpyHostToDevice));
        GM_CUDA(m, cudaMemcpy(m->sine[kind], sn.data(), sizeof(bf16_t) * sn.size(), cudaMemcpyHostToDevice));
    }
    {
        const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
        GM_CUDA(m, cudaFuncSetAttribute(gm_project_kernel<1>, at, project_smem_bytes(1)));
        GM_CUDA(m, cudaFuncSetAttribute(gm_project_kernel<2>, at, project_smem_bytes(2)));
        GM_CUDA(m, cudaFuncSetAttribute(gm_project_kernel<4>, at, project_smem_bytes(4)));
        GM_CUDA(m, cudaFuncSetAttribute(gm_project_kernel<8>, at, project_smem_bytes(8)));
    }
    const size_t attention_bytes = attention_smem_bytes(c.context, c.head_dim > c.global_head_dim ? c.head_dim : c.global_head_dim);
    if (attention_bytes > 48 * 1024) {
        if (attention_bytes > 200 * 1024) return fail(m, RIBN_B200_ERROR, "context %d exceeds the attention kernel's score buffer", c.context);
        GM_CUDA(m, cudaFuncSetAttribute(gm_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attention_bytes));
    }
    m->finalized = true;
    return RIBN_B200_OK;
}

}  // extern "C"

namespace {

struct Pass {
    ribn_b200_gemma* m;
    int rows;
    uint32_t launches = 0;

    void project_many(const bf16_t* in, const int* row_index, int n_rows, int k, int count, const bf16_t* const* w,
                      const int* n, bf16_t* const* out) {
        ProjectTargets t{};
        t.count = count;
        unsigned col_blocks = 0;
        for (int i = 0; i < count; ++i) {
            t.w[i] = w[i]; t.out[i] = out[i]; t.n[i] = n[i];
            t.first_block[i] = (int)col_blocks;
            col_blocks += (unsigned)((n[i] + kProjectCols - 1) / kProjectCols);
        }
        const dim3 block(kProjectCols);
        cudaStream_t s = m->stream;
        if ((m->cfg.flags & RIBN_B200_GEMMA_FLAG_TENSOR_CORE_PREFILL) && n_rows >= 16 && k % kMmaStageK == 0) {
            unsigned tile_blocks = 0;
            for (int i = 0; i < count; ++i) {
                t.first_block[i] = (int)tile_blocks;
                tile_blocks += (unsigned)((n[i] + kMmaTile - 1) / kMmaTile);
            }
            gm_project_mma_kernel<<<dim3(tile_blocks, (unsigned)((n_rows + kMmaTile - 1) / kMmaTile)), 128, 0, s>>>(in, row_index, n_rows, t, k);
            ++launches;
            return;
        }
        if (n_rows <= 1) gm_project_kernel<1><<<dim3(col_blocks, 1), block, project_smem_bytes(1), s>>>(in, row_index, n_rows, t, k);
        else if (n_rows <= 2) gm_project_kernel<2><<<dim3(col_blocks, 1), block, project_smem_bytes(2), s>>>(in, row_index, n_rows, t, k);
        else if (n_rows <= 4) gm_project_kernel<4><<<dim3(col_blocks, 1), block, project_smem_bytes(4), s>>>(in, row_index, n_rows, t, k);
        else gm_project_kernel<8><<<dim3(col_blocks, (unsigned)((n_rows + 7) / 8)), block, project_smem_bytes(8), s>>>(in, row_index, n_rows, t, k);
        ++launches;
    }
    void project(const bf16_t* in, const int* row_index, int n_rows, const bf16_t* w, int n, int k, bf16_t* out) {
        project_many(in, row_index, n_rows, k, 1, &w, &n, &out);
    }
    void rms(const bf16_t* in, const int* row_index, int n_rows, int width, const bf16_t* scale, const bf16_t* residual,
             const bf16_t* scalar, int mode, bf16_t* out) {
        gm_rms_kernel<<<(unsigned)n_rows, 256, sizeof(float) * (size_t)width, m->stream>>>(in, row_index, width, m->cfg.eps, scale, residual, scalar, mode, out);
        ++launches;
    }
    void gelu_mul(const bf16_t* gate, const bf16_t* other, size_t n, bf16_t* out) {
        gm_gelu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, m->stream>>>(gate, other, n, out);
        ++launches;
    }
};

// One pass over `rows` flattened tokens already staged in the model's pinned arrays; n_out of them (their
// indices in h_out_rows) produce logits and a greedy token.
int enqueue_pass(ribn_b200_gemma* m, int rows, int n_out, int max_position, uint32_t* launches) {
    const ribn_b200_gemma_config& c = m->cfg;
    cudaStream_t s = m->stream;
    GM_CUDA(m, cudaMemcpyAsync(m->d_tokens, m->h_tokens, sizeof(uint32_t) * (size_t)rows, cudaMemcpyHostToDevice, s));
    GM_CUDA(m, cudaMemcpyAsync(m->d_slot, m->h_slot, sizeof(int) * (size_t)rows, cudaMemcpyHostToDevice, s));
    GM_CUDA(m, cudaMemcpyAsync(m->d_position, m->h_position, sizeof(int) * (size_t)rows, cudaMemcpyHostToDevice, s));
    if (n_out > 0) GM_CUDA(m, cudaMemcpyAsync(m->d_out_rows, m->h_out_rows, sizeof(int) * (size_t)n_out, cudaMemcpyHostToDevice, s));
    Pass p{m, rows};
    const int H = c.hidden, P = c.ple, packed = c.layers * c.ple;
    // decoder.rs:78-92: the embedding scales are BF16-rounded square roots; the projection scale is plain FP32
    const float embed_scale = bf_load(bf_round(sqrtf((float)H)));
    const float ple_scale = bf_load(bf_round(sqrtf((float)P)));
    const float projection_scale = 1.0f / sqrtf((float)H);
    gm_embed_kernel<<<(unsigned)rows, 256, 0, s>>>(m->d_tokens, m->g[G_EMBED].data, m->g[G_PLE_EMBED].data, H, packed,
                                                    embed_scale, ple_scale, m->hidden, m->identity);
    ++p.launches;
    p.project(m->hidden, nullptr, rows, m->g[G_PLE_PROJ].data, packed, H, m->projection);
    gm_ple_kernel<<<dim3((unsigned)rows, (unsigned)c.layers), 256, 0, s>>>(m->projection, m->identity, m->g[G_PLE_NORM].data, rows,
                                                                           P, packed, projection_scale, c.eps, m->per_layer);
    ++p.launches;
    for (int l = 0; l < c.layers; ++l) {
        Tensor* L = m->l[l];
        const int w = width_of(c, l), kind = c.full[l] ? 1 : 0, owner = m->owner[l], cache = m->cache_of[owner];
        const bool owns = owner == l;
        p.rms(m->hidden, nullptr, rows, H, L[L_IN].data, nullptr, nullptr, 0, m->normed);
        {
            const bf16_t* ws[3] = {L[L_Q].data, L[L_K].data, L[L_V].data};
            const int ns[3] = {c.heads * w, c.kv_heads * w, c.kv_heads * w};
            bf16_t* outs[3] = {m->q, m->k, m->v};
            p.project_many(m->normed, nullptr, rows, H, owns ? 3 : 1, ws, ns, outs);
        }
        gm_head_kernel<<<dim3((unsigned)rows, (unsigned)(c.heads + (owns ? 2 * c.kv_heads : 0))), 128, 0, s>>>(
            m->q, m->k, m->v, L[L_QNORM].data, owns ? L[L_KNORM].data : nullptr, m->d_slot, m->d_position, m->cosine[kind],
            m->sine[kind], c.heads, c.kv_heads, w, c.eps, c.context, m->q2, m->key_cache[(size_t)cache],
            m->value_cache[(size_t)cache]);
        ++p.launches;
        const int window = kind ? 0 : c.window;
        const int visible = window > 0 && window < max_position + 1 ? window : max_position + 1;
        gm_attention_kernel<<<dim3((unsigned)rows, (unsigned)c.heads), 256, attention_smem_bytes(visible, w), s>>>(
            m->q2, m->d_slot, m->d_position, m->key_cache[(size_t)cache], m->value_cache[(size_t)cache], c.heads, c.kv_heads, w,
            window, c.context, m->attended);
        ++p.launches;
        p.project(m->attended, nullptr, rows, L[L_O].data, H, c.heads * w, m->projected);
        p.rms(m->projected, nullptr, rows, H, L[L_POST_ATTN].data, m->hidden, nullptr, 1, m->mid);
        // feed-forward (decoder.rs:570-600)
        p.rms(m->mid, nullptr, rows, H, L[L_PRE_FFN].data, nullptr, nullptr, 0, m->normed);
        {
            const bf16_t* ws[2] = {L[L_GATE].data, L[L_UP].data};
            const int ns[2] = {c.ffn, c.ffn};
            bf16_t* outs[2] = {m->gate, m->up};
            p.project_many(m->normed, nullptr, rows, H, 2, ws, ns, outs);
        }
        p.gelu_mul(m->gate, m->up, (size_t)rows * c.ffn, m->gate);
        p.project(m->gate, nullptr, rows, L[L_DOWN].data, H, c.ffn, m->projected);
        p.rms(m->projected, nullptr, rows, H, L[L_POST_FFN].data, m->mid, nullptr, 1, m->hidden);
        // per-layer embedding gate, layer scalar (decoder.rs:602-626)
        p.project(m->hidden, nullptr, rows, L[L_PLE_GATE].data, P, H, m->ple_gate);
        p.gelu_mul(m->ple_gate, m->per_layer + (size_t)l * rows * P, (size_t)rows * P, m->ple_gate);
        p.project(m->ple_gate, nullptr, rows, L[L_PLE_PROJ].data, H, P, m->projected);
        p.rms(m->projected, nullptr, rows, H, L[L_POST_PLE].data, m->hidden, L[L_SCALAR].data, 2, m->hidden);
    }
    if (n_out > 0) {
        // decoder.rs:410-428: final norm, tied head, soft cap; then the greedy choice
        p.rms(m->hidden, m->d_out_rows, n_out, H, m->g[G_NORM].data, nullptr, nullptr, 0, m->normed);
        p.project(m->normed, nullptr, n_out, m->g[G_EMBED].data, c.vocab, H, m->logits);
        const size_t n = (size_t)n_out * c.vocab;
        gm_softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(m->logits, n, c.softcap);
        gm_argmax_kernel<<<(unsigned)n_out, 1024, 0, s>>>(m->logits, c.vocab, m->d_choice);
        p.launches += 2;
        GM_CUDA(m, cudaMemcpyAsync(m->h_choice, m->d_choice, sizeof(uint32_t) * (size_t)n_out, cudaMemcpyDeviceToHost, s));
    }
    GM_CUDA(m, cudaGetLastError());
    *launches += p.launches;
    return RIBN_B200_OK;
}

// A pass reads its rows (tokens, slots, positions, output rows) from the pinned staging arrays, so passes of one
// shape differ only in data: from the third time a shape (rows, outputs, context bucket of 128) comes up it is
// captured into a CUDA graph, which closes the gaps between its ~100 short launches.
int run_pass(ribn_b200_gemma* m, int rows, int n_out, int max_position, uint32_t* launches) {
    constexpr size_t kMaxPassGraphs = 128;
    const int bucket_end = std::min(((max_position + 1 + 127) / 128) * 128, m->cfg.context);
    const uint64_t key = (uint64_t)rows | ((uint64_t)n_out << 20) | ((uint64_t)bucket_end << 40);
    auto found = m->graphs.find(key);
    if (found == m->graphs.end()) {
        if (++m->graph_seen[key] < 3 || m->graphs.size() >= kMaxPassGraphs) return enqueue_pass(m, rows, n_out, max_position, launches);
        cudaGraph_t graph = nullptr;
        uint32_t captured = 0;
        GM_CUDA(m, cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_pass(m, rows, n_out, bucket_end - 1, &captured);
        const cudaError_t end = cudaStreamEndCapture(m->stream, &graph);
        if (rc != RIBN_B200_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
        GM_CUDA(m, end);
        ribn_b200_gemma::PassGraph entry;
        entry.launches = captured;
        const cudaError_t inst = cudaGraphInstantiate(&entry.exec, graph, 0);
        cudaGraphDestroy(graph);
        GM_CUDA(m, inst);
        found = m->graphs.emplace(key, entry).first;
    }
    GM_CUDA(m, cudaGraphLaunch(found->second.exec, m->stream));
    *launches += found->second.launches;
    return RIBN_B200_OK;
}

Sequence* find_sequence(ribn_b200_gemma* m, uint64_t id) {
    if (id == 0 || id > m->seq.size() || !m->seq[(size_t)id - 1].open) return nullptr;
    return &m->seq[(size_t)id - 1];
}

}  // namespace

extern "C" {

RIBN_B200_API int ribn_b200_gemma_open(ribn_b200_gemma* m, uint64_t* sequence) {
    if (!m || !sequence) return RIBN_B200_ERROR;
    if (!m->finalized) return fail(m, RIBN_B200_ERROR, "finalize the model before opening a sequence");
    for (size_t i = 0; i < m->seq.size(); ++i) {
        if (!m->seq[i].open) {
            m->seq[i].open = true;
            m->seq[i].position = 0;
            *sequence = (uint64_t)i + 1;
            return RIBN_B200_OK;
        }
    }
    return fail(m, RIBN_B200_DEFERRED, "all %zu sequence slots are open", m->seq.size());
}

RIBN_B200_API int ribn_b200_gemma_close(ribn_b200_gemma* m, uint64_t sequence) {
    if (!m) return RIBN_B200_ERROR;
    if (sequence == 0 || sequence > m->seq.size()) return fail(m, RIBN_B200_ERROR, "unknown sequence %llu", (unsigned long long)sequence);
    // every step call completes its device work before it returns, so nothing is in flight here; idempotent
    m->seq[(size_t)sequence - 1].open = false;
    m->seq[(size_t)sequence - 1].position = 0;
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_position(const ribn_b200_gemma* m, uint64_t sequence, uint32_t* position) {
    if (!m || !position || sequence == 0 || sequence > m->seq.size() || !m->seq[(size_t)sequence - 1].open) return RIBN_B200_ERROR;
    *position = m->seq[(size_t)sequence - 1].position;
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_step(ribn_b200_gemma* m, const ribn_b200_gemma_row* rows, uint32_t n_rows,
                                       uint32_t* tokens_out, uint16_t* logits_out) {
    if (!m || !rows || n_rows == 0) return m ? fail(m, RIBN_B200_ERROR, "empty step") : RIBN_B200_ERROR;
    if (!m->finalized) return fail(m, RIBN_B200_ERROR, "finalize the model before stepping");
    const ribn_b200_gemma_config& c = m->cfg;
    // Validate everything before any state changes (decoder.rs:139-160: a failed step leaves the continuation as it was).
    size_t total = 0;
    for (uint32_t i = 0; i < n_rows; ++i) {
        const ribn_b200_gemma_row& r = rows[i];
        Sequence* s = find_sequence(m, r.sequence);
        if (!s) return fail(m, RIBN_B200_REJECTED, "row %u: unknown sequence %llu", i, (unsigned long long)r.sequence);
        for (uint32_t j = 0; j < i; ++j) {
            if (rows[j].sequence == r.sequence) return fail(m, RIBN_B200_REJECTED, "row %u: sequence appears twice in one step", i);
        }
        if (r.n_tokens == 0 || !r.tokens || (uint64_t)s->position + r.n_tokens > (uint64_t)c.context) {
            return fail(m, RIBN_B200_REJECTED, "row %u: empty or overlong token chunk", i);
        }
        for (uint32_t t = 0; t < r.n_tokens; ++t) {
            if (r.tokens[t] >= (uint32_t)c.vocab) return fail(m, RIBN_B200_REJECTED, "row %u: token %u outside the vocabulary", i, r.tokens[t]);
        }
        if (r.want_output && !tokens_out) return fail(m, RIBN_B200_ERROR, "row %u wants output but tokens_out is null", i);
        total += r.n_tokens;
    }
    GM_CUDA(m, cudaSetDevice(c.device));
    GM_CUDA(m, cudaEventRecord(m->ev0, m->stream));
    uint32_t launches = 0;
    // Flatten rows into passes of at most max_batch_tokens tokens, in row order.
    uint32_t row = 0, offset = 0;  // next token to stage
    size_t logits_row = 0;         // next slot of logits_out
    std::vector<uint32_t> out_owner;  // pass-local: which step row each output belongs to
    while (row < n_rows) {
        int staged = 0, n_out = 0, max_position = 0;
        out_owner.clear();
        while (row < n_rows && staged < c.max_batch_tokens && n_out < m->max_outputs) {
            const ribn_b200_gemma_row& r = rows[row];
            Sequence* s = find_sequence(m, r.sequence);
            const uint32_t take = std::min<uint32_t>(r.n_tokens - offset, (uint32_t)(c.max_batch_tokens - staged));
            for (uint32_t t = 0; t < take; ++t) {
                m->h_tokens[staged] = r.tokens[offset + t];
                m->h_slot[staged] = (int)(r.sequence - 1);
                m->h_position[staged] = (int)(s->position + offset + t);
                max_position = std::max(max_position, m->h_position[staged]);
                ++staged;
            }
            offset += take;
            if (offset == r.n_tokens) {
                if (r.want_output) {
                    m->h_out_rows[n_out++] = staged - 1;
                    out_owner.push_back(row);
                }
                ++row;
                offset = 0;
            }
        }
        if (int rc = run_pass(m, staged, n_out, max_position, &launches)) return rc;
        GM_CUDA(m, cudaStreamSynchronize(m->stream));
        for (int o = 0; o < n_out; ++o) {
            tokens_out[out_owner[(size_t)o]] = m->h_choice[o];
            if (logits_out) {
                GM_CUDA(m, cudaMemcpy(logits_out + logits_row * (size_t)c.vocab, m->logits + (size_t)o * c.vocab,
                                      sizeof(bf16_t) * (size_t)c.vocab, cudaMemcpyDeviceToHost));
                ++logits_row;
            }
        }
    }
    GM_CUDA(m, cudaEventRecord(m->ev1, m->stream));
    GM_CUDA(m, cudaEventSynchronize(m->ev1));
    cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1);
    m->last_launches = launches;
    for (uint32_t i = 0; i < n_rows; ++i) find_sequence(m, rows[i].sequence)->position += rows[i].n_tokens;
    (void)total;
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_advance_prefill(ribn_b200_gemma* m, uint64_t sequence, const uint32_t* tokens, uint32_t n_tokens) {
    const ribn_b200_gemma_row row = {sequence, tokens, n_tokens, 0};
    return ribn_b200_gemma_step(m, &row, 1, nullptr, nullptr);
}

RIBN_B200_API int ribn_b200_gemma_prefill(ribn_b200_gemma* m, uint64_t sequence, const uint32_t* tokens, uint32_t n_tokens,
                                          uint16_t* logits, uint32_t* token) {
    const ribn_b200_gemma_row row = {sequence, tokens, n_tokens, 1};
    uint32_t choice = 0;
    const int rc = ribn_b200_gemma_step(m, &row, 1, &choice, logits);
    if (rc == RIBN_B200_OK && token) *token = choice;
    return rc;
}

RIBN_B200_API int ribn_b200_gemma_decode(ribn_b200_gemma* m, uint64_t sequence, uint32_t input, uint16_t* logits, uint32_t* token) {
    return ribn_b200_gemma_prefill(m, sequence, &input, 1, logits, token);
}

RIBN_B200_API int ribn_b200_gemma_synchronize(ribn_b200_gemma* m) {
    if (!m) return RIBN_B200_ERROR;
    GM_CUDA(m, cudaStreamSynchronize(m->stream));
    return RIBN_B200_OK;
}

RIBN_B200_API int ribn_b200_gemma_last_step_stats(const ribn_b200_gemma* m, float* milliseconds, uint32_t* launches) {
    if (!m) return RIBN_B200_ERROR;
    if (milliseconds) *milliseconds = m->last_ms;
    if (launches) *launches = m->last_launches;
    return RIBN_B200_OK;
}

}  // extern "C"
