// Paged split-KV attention for callers that cannot allocate device memory.
//
// Some hosts run this library where cudaMalloc is off limits: inside a region that is being
// captured into a CUDA graph, inside a latency-critical serving loop whose memory was carved up
// at start-up, or under an allocator policy that forbids driver allocations after initialisation.
// The ordinary attention entry point needs scratch for the per-span accumulators that the merge
// pass folds together; this variant keeps that scratch in a fixed array that is part of the
// library image, so it allocates nothing: no cudaMalloc, no cudaFree, no allocating library call.
//
// Cost and limits.  Every GPU that loads the library holds the array (8 MiB) until the process
// exits.  A call whose span accumulators would not fit is refused with a message.  All calls
// share the one array: calls that may overlap on the GPU (different streams, or different host
// threads) race on it and must be serialised by the caller.  Nothing in the array needs to
// start at zero -- every slot that the merge pass reads is written by the span pass of the same
// call first -- so stale contents from the previous call are harmless.
//
// The device address of the array is looked up on the first call made for a device (one
// cudaGetSymbolAddress per device, with that device current); make that first call before
// any stream capture begins.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include "../../include/ribn_b200.h"
#include "kernels.cuh"

namespace {

constexpr size_t kScratchFloats = 2u * 1024u * 1024u;  // 8 MiB of span accumulators
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) float g_span_scratch[kScratchFloats];

float* g_scratch_address[kMaxDevices] = {nullptr};

int refuse(char* error, size_t capacity, const char* message) {
    if (error != nullptr && capacity > 0) snprintf(error, capacity, "%s", message);
    return RIBN_B200_ERROR;
}

}  // namespace

extern "C" int ribn_b200_attention_noalloc(int32_t device, void* stream, const float* q, const uint16_t* keys,
                                           const uint16_t* values, const int32_t* page_table,
                                           const int32_t* token_pos, int32_t rows, int32_t max_tokens,
                                           int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t window,
                                           float* out, char* error, size_t error_capacity) {
    if (q == nullptr || keys == nullptr || values == nullptr || page_table == nullptr || token_pos == nullptr ||
        out == nullptr) {
        return refuse(error, error_capacity, "null device pointer");
    }
    if (rows <= 0 || max_tokens <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 ||
        q_heads / kv_heads > 16 || (head_dim != 64 && head_dim != 128 && head_dim != 256)) {
        return refuse(error, error_capacity, "unsupported attention geometry (head_dim must be 64, 128 or 256; at most 16 query heads per kv head)");
    }
    if (device < 0 || device >= kMaxDevices) return refuse(error, error_capacity, "device ordinal out of range");
    // The launch needs `device` current; the caller's own current device is put back before returning.
    struct DeviceScope {
        int previous = -1;
        bool ok = false;
        explicit DeviceScope(int device) {
            if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
            ok = previous == device || cudaSetDevice(device) == cudaSuccess;
        }
        ~DeviceScope() {
            int now = -1;
            if (previous >= 0 && cudaGetDevice(&now) == cudaSuccess && now != previous) cudaSetDevice(previous);
        }
    } scope(device);
    if (!scope.ok) return refuse(error, error_capacity, "cannot select the CUDA device");
    const int keys_per_row = window > 0 && window < max_tokens ? window : max_tokens;
    const size_t spans = ((size_t)keys_per_row + ribn::kAttnSpanKeys - 1) / ribn::kAttnSpanKeys;
    const size_t need = (size_t)rows * q_heads * spans * (size_t)(head_dim + 2);
    if (spans > (size_t)ribn::kAttnMaxSpans || need > kScratchFloats) {
        char message[256];
        snprintf(message, sizeof(message),
                 "rows x q_heads x spans x (head_dim + 2) = %zu floats exceeds the built-in scratch of %zu floats "
                 "(8 MiB): use fewer rows per call or the allocating entry point",
                 need, (size_t)kScratchFloats);
        return refuse(error, error_capacity, message);
    }
    if (g_scratch_address[device] == nullptr) {
        // Set-up, once per device: resolve the array's device address.
        void* address = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&address, g_span_scratch);
        if (e != cudaSuccess || address == nullptr) {
            return refuse(error, error_capacity, "cudaGetSymbolAddress failed for the built-in scratch");
        }
        g_scratch_address[device] = static_cast<float*>(address);
    }
    const int pages = (max_tokens + ribn::kPageTokens - 1) / ribn::kPageTokens;
    cudaError_t e = ribn::launch_attention(static_cast<cudaStream_t>(stream), q, reinterpret_cast<const __half*>(keys),
                                           reinterpret_cast<const __half*>(values), page_table, pages, nullptr,
                                           token_pos, rows, q_heads, kv_heads, head_dim, window, max_tokens,
                                           g_scratch_address[device], kScratchFloats * sizeof(float), out, nullptr);
    if (e != cudaSuccess) return refuse(error, error_capacity, cudaGetErrorString(e));
    return RIBN_B200_OK;
}
