// Tile-major weight repack and the tensor-core GEMV built on it.
//
// A packed matrix is a sequence of tiles of 16 output rows x 256 inputs,
// ordered k-tile-major inside each row tile, so that a CTA streams one
// contiguous, 16-byte-aligned byte range with bulk (TMA) copies.  The byte
// order inside a tile is chosen so that each lane's 128-bit shared-memory
// reads are exactly the operands of its `mma.sync.m16n8k16` A fragment (rows
// g and g + 8, g = lane / 4; for each 16-wide k step the four inputs
// 4t .. 4t + 3, t = lane % 4).  Per type (a tile is exactly 16 raw GGUF
// super-blocks' worth of bytes, no padding):
//   Q4_K 2304 B: 4 x 512 B nibble chunks (group pairs) + 16 x 16 B headers
//   Q6_K 3360 B: 4 x 512 B low nibbles + 2 x 512 B high bits + 16 x 16 B scales + 16 x 2 B d
//   Q8_0 4352 B: 8 x 512 B offset-binary bytes (q + 128) + 16 x 16 B of f16 d
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ribn {

constexpr int kTileRows = 16;
constexpr int kTileCols = 256;
constexpr int kMaxDevices = 64;  // per-device launcher state (function attributes, SM counts) is kept per ordinal

struct PackedMatrix {
    unsigned char* data = nullptr;  // device
    size_t bytes = 0;
    int type = -1;
    long long n = 0, k = 0;
    int row_tiles = 0, k_tiles = 0;
    bool ready() const { return data != nullptr; }
};

__host__ __device__ inline int packed_tile_bytes(int type) {
    switch (type) {
        case 12: return 2304;
        case 14: return 3360;
        case 8: return 4352;
        default: return 0;
    }
}

// True when the fast kernels can take a matrix of this type and shape.
inline bool packable(int type, long long n, long long k) {
    return packed_tile_bytes(type) != 0 && k % kTileCols == 0 && n > 0;
}

inline size_t packed_bytes(int type, long long n, long long k) {
    const long long row_tiles = (n + kTileRows - 1) / kTileRows;
    return (size_t)row_tiles * (size_t)(k / kTileCols) * (size_t)packed_tile_bytes(type);
}

// Host repack of raw GGUF rows [n][k / block] into the tile-major layout.
// Rows beyond n (padding of the last row tile) decode to zero.
void repack_host(int type, const unsigned char* raw, long long n, long long k, unsigned char* out,
                 int threads);

// Activations in tensor-core operand form: signed 8-bit digits for the
// integer MMA.  Every 32 consecutive inputs share a scale sx = max|x| / 127 and
// each input is carried as three digits d1, d2, d3 in [-127, 127] with
//     x ~= sx * (d1 + d2 / 128 + d3 / 16384)           (|error| <= max|x| * 2.4e-7)
// so the integer dot products are exact and the only rounding is this one.
// Inside a 32-span the bytes are permuted so that lane t's MMA fragment
// (inputs 4t..4t+3 and 16+4t..16+4t+3) is one 8-byte word:
//     position(k) = ((k & 15) >> 2) * 8 + ((k >> 4) & 1) * 4 + (k & 3).
// Alongside: `sxs16` = sx * (sum of the digit values over each 16-span), used
// to remove the formats' offsets (Q4_K minimum, Q6_K -32, Q8_0 -128), and,
// when an RMSNorm precedes the projection, `ss32` = sums of squares of the
// *unscaled* input per 32-span.  The norm weight is already folded into x; the
// consumer multiplies its result by 1 / sqrt(mean square + eps).  The kernel
// that produces x writes this form in its epilogue, so the consuming GEMV
// loads its B operand with plain bulk copies.
struct ActOperand {
    signed char* dig = nullptr;  // [members][3][k]
    float* sx = nullptr;         // [members][k / 32]
    float* sxs16 = nullptr;      // [members][k / 16]
    float* ss32 = nullptr;       // [members][k / 32]
};

__host__ __device__ inline int operand_position(int k) {
    return (k & ~31) + (((k & 15) >> 2) * 8) + (((k >> 4) & 1) * 4) + (k & 3);
}

// f32 activations -> operand form (standalone; producers fuse the same math).
// norm_weight == nullptr: x is used as is and ss32 is not written.
// `index` (optional) gathers rows of x.
cudaError_t launch_to_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                              int members, int k, ActOperand out);

// One fused GEMV launch covers up to three matrices that share the input
// vector (q|k|v, gate|up) as consecutive row-tile segments.
struct GemvSegment {
    const unsigned char* data;
    int type;
    int n;          // valid output rows
    int row_tiles;
    float* y;       // [members][n] F32 output (the residual stream for kResidual)
    // K-quant matrices only, optional: the matrix once more as tensor-core operands (launch_tc_cache); the
    // tensor-memory GEMM then copies operand stages instead of converting packed tiles
    const unsigned char* op_a = nullptr;
    const unsigned char* op_meta = nullptr;
};

enum GemvEpilogue : int {
    kStore = 0,     // y = W x
    kResidual = 1,  // y += W x           (y is the residual stream)
    kSwiGLU = 2     // two segments (gate, up): silu(gate x) * (up x)
};

struct GemvArgs {
    GemvSegment seg[3];
    int n_segments;
    int k;
    int members;          // 1..kGemvMaxMembers input vectors
    ActOperand in;        // B operand
    int in_has_norm;      // multiply the result by rsqrt(mean(ss32) + eps)
    float eps;
    int epilogue;
    // Optional operand-form copy of the result (kResidual: of the updated
    // residual stream times `out_norm_weight`; kSwiGLU: of the gated product).
    ActOperand out;
    const float* out_norm_weight;
    float* swiglu_f32;    // optional F32 copy of the gated product [members][n]
    int* error_flag;      // set non-zero when a bounded wait gives up
    uint32_t spin_limit;  // polls before a wait gives up (0: the default, 1 << 22)
};

constexpr int kGemvMaxMembers = 2;

// Enqueue the GEMV.  `programmatic` launches it as a programmatic dependent of
// the previous kernel in the stream, so its weight prefetch overlaps that
// kernel's tail.
cudaError_t launch_gemv_mma(cudaStream_t stream, const GemvArgs& args, bool programmatic);
// One-time function attributes (call outside stream capture, with the device current).
cudaError_t gemv_prepare();
// Failure-detection aid: a one-thread kernel that waits, through the kernels' bounded wait, on a barrier
// nothing completes; after `spin_limit` polls (at most 1 << 20) it writes `code` to *error_flag and returns.
cudaError_t launch_wait_probe(cudaStream_t stream, int* error_flag, uint32_t spin_limit, int code);

// ---- batched form (3..64 members) ---------------------------------------------------------------
// Activations for the batched kernel: one scale per member for its whole vector
// (x ~= scale * (d1 + d2/128 + d3/16384), |error| <= max|x| * 2.4e-7), stored as one chunk per
// k tile so that a single bulk copy brings everything the kernel needs for that k tile:
//   [member][digit][kBatchPlaneBytes]   256 digits in `operand_position` order + padding that spreads
//                                       the digit planes over the shared-memory banks
//   [sub / 4][member][sub % 4] F32      digit-value sums per 16 inputs `sub` (offset removal)
// and, outside the chunks, member_scale[member]: the digit scale, times the RMSNorm factor when a
// norm precedes.  Members are padded to a multiple of 8 with zero digits.
constexpr int kBatchPlaneBytes = 288;
constexpr int kGemmMaxMembers = 64;

struct BatchOperand {
    signed char* chunks = nullptr;
    float* member_scale = nullptr;  // [members]
    float* digit_inv = nullptr;     // [members] scratch: 127 / max|x|
};

size_t batch_operand_bytes(int members, int k);

// f32 activations [members][k] (rows gathered through `index` when given), optionally times
// `norm_weight` with the RMSNorm factor folded into member_scale -> batch operand form.
cudaError_t launch_to_batch_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                                    int members, int k, float eps, BatchOperand out);

struct GemmArgs {
    GemvSegment seg[3];   // y is [members][n] F32
    int n_segments;
    int k;
    int members;          // 1..kGemmMaxMembers
    const signed char* chunks;
    const float* member_scale;
    int epilogue;         // GemvEpilogue; kSwiGLU writes seg[0].y = silu(gate) * up
    int* error_flag;
    int kquant;           // tensor-memory kernels: the activations are in the K-quant form (see TcOperand)
    float* partial;       // optional scratch for split-K sums [slices][members][rows of all segments]
    size_t partial_floats;
    // K-quant tensor-memory form only: `groups` > 1 runs that many consecutive groups of `members` rows in one
    // launch (their operands `group_chunk_bytes` apart, scales and outputs consecutive), so every weight tile
    // meets all the row groups of a prefill step while it is in L2.
    int groups;
    size_t group_chunk_bytes;
    uint32_t spin_limit;  // polls before a bounded wait gives up (0: the default, 1 << 22)
};

cudaError_t launch_gemm_imma(cudaStream_t stream, const GemmArgs& args);

// ---- tensor-memory form (tcgen05, 3..128 members) ---------------------------------------------------
// Activations as binary16 pairs hi + lo of x * scale_in[member] (scale_in a power of two that brings
// the member's largest |x| into [1, 2)), in the K-major core-matrix order the tensor core reads:
// per 64 inputs one chunk [8-input block][column][8 halves] with the hi parts in columns
// [0, padded members) and the lo parts behind them; members are padded to a multiple of 16.
// member_scale[member] = RMSNorm factor / scale_in, applied by the kernel's epilogue.
constexpr int kGemmTcMaxMembers = 128;

struct TcOperand {
    __half* chunks = nullptr;
    float* scale_in = nullptr;      // [members]
    float* member_scale = nullptr;  // [members]
};

size_t tc_operand_bytes(int members, int k);
// True when the launch can take the K-quant form: only Q4_K / Q6_K matrices and at most 64 members.
// There the tensor core multiplies the blocks' exact integers (scale x quant) and the F32 super-block
// scales are applied per 256 inputs; the activations then carry, per k tile, the sums of their eight
// 32-input groups behind the four chunks (`kquant` below).  Otherwise every weight is decoded to F32
// and split into a binary16 pair.
bool gemm_tc_kquant(const GemvSegment* segments, int n_segments, int members);
cudaError_t launch_to_tc_operand(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                                 int members, int k, float eps, bool kquant, TcOperand out);
// The K-quant form for `members` input rows at once, as consecutive operands of `group` members each
// (tc_operand_bytes(group, k) apart; scales indexed by member): one conversion for all the groups of a
// prefill chunk.  `out` must hold ceil(members / group) operands and `members` scales.
cudaError_t launch_to_tc_operand_groups(cudaStream_t stream, const float* x, const int32_t* index, const float* norm_weight,
                                        int members, int group, int k, float eps, TcOperand out);
// GemmArgs::chunks points at TcOperand::chunks, GemmArgs::kquant says which form; epilogue kStore or kResidual.
cudaError_t launch_gemm_tc(cudaStream_t stream, const GemmArgs& args);
// Parity aid: decodes a tile-major packed matrix back to F32 [rows][cols] with the weight decoder of the
// decode-and-split tensor-memory kernel (the reference's arithmetic), reading the packed bytes only.
// A Q4_K / Q6_K packed matrix as tensor-core operands: per 128-row unit and 256-input k tile the four 64-input
// operand pieces (one binary16 plane of 16 KB for Q4_K, two for Q6_K) into `cache_a`, and the rows' scales with the
// minima operand (5 KB) into `cache_meta`.  The bytes are the ones the converting kernels build in shared memory.
size_t tc_cache_a_bytes(int type, long long rows, long long cols);
size_t tc_cache_meta_bytes(long long rows, long long cols);
cudaError_t launch_tc_cache(cudaStream_t stream, int type, const unsigned char* packed, long long rows, long long cols,
                            unsigned char* cache_a, unsigned char* cache_meta);

cudaError_t launch_unpack_packed(cudaStream_t stream, int type, const unsigned char* packed, long long rows, long long cols,
                                 float* out);
// Kernels the calling thread's last launch_gemm_tc enqueued (2 when a split-K launch adds its ordered reduction).
int gemm_tc_last_launches();

// Scratch shared by the step kernels: per-span attention accumulators.
struct StepScratch {
    float* attn_partial = nullptr;
    size_t attn_partial_bytes = 0;
};

}  // namespace ribn
