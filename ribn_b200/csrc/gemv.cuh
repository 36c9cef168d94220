// Tile-major weight repack and the tensor-core GEMV built on it.
//
// A packed matrix is a sequence of tiles of 16 output rows x 256 inputs,
// ordered k-tile-major inside each row tile, so that one warp streams
// contiguous 16-byte-aligned memory with 128-bit loads.  The byte order
// inside a tile is chosen so that each lane's loads are exactly the operands
// of its `mma.sync.m16n8k16` A fragment (rows g and g + 8, g = lane / 4;
// for each 16-wide k step the four inputs 4t .. 4t + 3, t = lane % 4).
// Per type (sizes per tile equal 16 raw GGUF blocks, no padding bytes):
//   Q4_K 2304 B: 4 x 512 B nibble chunks (group pairs) + 16 x 16 B headers
//   Q6_K 3360 B: 4 x 512 B low nibbles + 2 x 512 B high bits + 16 x 16 B scales + 16 x 2 B d
//   Q8_0 4352 B: 8 x 512 B offset-binary bytes (q + 128) + 16 x 16 B of f16 d
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ribn {

constexpr int kTileRows = 16;
constexpr int kTileCols = 256;

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

// One fused GEMV launch covers up to three matrices that share the input
// vector (q|k|v, gate|up) as consecutive row-tile segments.
struct GemvSegment {
    const unsigned char* data;
    int type;
    int n;          // valid output rows
    int row_tiles;
    float* y;       // [members][n] output (or residual stream for kResidual)
};

enum GemvEpilogue : int {
    kStore = 0,     // y = W x
    kResidual = 1,  // y += W x           (y is the residual stream)
    kSwiGLU = 2     // two segments (gate, up): out = silu(gate x) * (up x), written to segment 0's y
};

struct GemvArgs {
    GemvSegment seg[3];
    int n_segments;
    int k;
    int members;             // 1..4 input vectors
    const float* x;          // [members][k] F32 activations
    const float* norm_weight;  // optional RMSNorm weight applied to x first (nullptr: none)
    float eps;
    int epilogue;
};

cudaError_t launch_gemv_mma(cudaStream_t stream, const GemvArgs& args, bool dependent_launch);

constexpr int kGemvMaxMembers = 4;

// Scratch shared by the step kernels: per-span attention accumulators.
struct StepScratch {
    float* attn_partial = nullptr;
    size_t attn_partial_bytes = 0;
};

}  // namespace ribn
