// Paged-KV ragged attention for decode rows and prefill chunks: split-KV
// ("flash-decoding") over fixed 64-key spans with an online softmax, then a
// deterministic merge of the spans.
//
// One CTA serves one (token, kv head, span); its warps are the q heads of the
// GQA group, so the group's K/V rows are fetched once per CTA and shared
// through L1.  Inside a warp the 32 lanes first take 32 different keys (a full
// head_dim dot product each, no cross-lane reduction), then switch to owning
// head_dim / 32 output dims for the P.V accumulation.  Spans depend only on
// the token's own key range, never on what else is in the batch, so a token's
// result is bit-identical whatever it is batched with and wherever its pages
// live.  The reference's two-pass form with a global scores buffer
// (crates/nvidia/src/model_ops.rs:441-545) is replaced, not translated.
#include <cuda_fp16.h>
#include <math.h>

#include <algorithm>

#include "kernels.cuh"

namespace ribn {

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int HD>
__global__ void attention_span_kernel(const float* __restrict__ q, const __half* __restrict__ cache_k,
                                      const __half* __restrict__ cache_v, const int32_t* __restrict__ page_tables,
                                      int pages_per_sequence, const int32_t* __restrict__ token_seq,
                                      const int32_t* __restrict__ token_pos, int token_base, int q_heads,
                                      int kv_heads, int window, int max_spans, float* __restrict__ partial,
                                      float* __restrict__ out) {
    constexpr int DPL = HD / 32;  // output dims per lane
    extern __shared__ float q_smem[];  // [warps][HD]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q_per_kv = q_heads / kv_heads;
    const int t = token_base + blockIdx.x / kv_heads, kvh = blockIdx.x % kv_heads;
    const int span = blockIdx.y;
    const int qh = kvh * q_per_kv + warp;
    const int pos = token_pos[t];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_keys = pos + 1 - first;
    const int spans = (n_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
    if (span >= spans) return;
    const int begin = first + span * kAttnSpanKeys;
    const int end = min(pos + 1, begin + kAttnSpanKeys);
    const int32_t* table = page_tables + (long long)token_seq[t] * pages_per_sequence;
    const float scale = 1.0f / sqrtf((float)HD);

    float* qs = q_smem + warp * HD;
    const float* qp = q + ((long long)t * q_heads + qh) * HD;
    for (int d = lane; d < HD; d += 32) qs[d] = qp[d];
    __syncwarp();

    float acc[DPL];
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[d] = 0.0f;
    float run_max = -INFINITY, total = 0.0f;
    const long long row_stride = (long long)kv_heads * HD;
    for (int base = begin; base < end; base += 32) {
        const int key = base + lane;
        const bool live = key < end;
        long long phys = 0;
        float s = -INFINITY;
        if (live) {
            phys = (long long)table[key / kPageTokens] * kPageTokens + key % kPageTokens;
            const uint4* kp = reinterpret_cast<const uint4*>(cache_k + phys * row_stride + (long long)kvh * HD);
            float dot = 0.0f;
#pragma unroll 4
            for (int i = 0; i < HD / 8; ++i) {
                const uint4 kk = __ldg(kp + i);
                const float4 qa = *reinterpret_cast<const float4*>(qs + i * 8);
                const float4 qb = *reinterpret_cast<const float4*>(qs + i * 8 + 4);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kk.x));
                const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kk.y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kk.z));
                const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kk.w));
                dot = fmaf(qa.x, k0.x, dot); dot = fmaf(qa.y, k0.y, dot);
                dot = fmaf(qa.z, k1.x, dot); dot = fmaf(qa.w, k1.y, dot);
                dot = fmaf(qb.x, k2.x, dot); dot = fmaf(qb.y, k2.y, dot);
                dot = fmaf(qb.z, k3.x, dot); dot = fmaf(qb.w, k3.y, dot);
            }
            s = dot * scale;
        }
        const float new_max = fmaxf(run_max, warp_max(s));
        const float factor = expf(run_max - new_max);  // 0 on the first tile (run_max = -inf)
        const float p = live ? expf(s - new_max) : 0.0f;
        total = total * factor + warp_sum(p);
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[d] *= factor;
        run_max = new_max;
        const int count = min(32, end - base);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long pj_phys = __shfl_sync(0xffffffffu, phys, j);
            const __half* vp = cache_v + pj_phys * row_stride + (long long)kvh * HD + lane * DPL;
            if (DPL == 4) {
                const uint2 vv = __ldg(reinterpret_cast<const uint2*>(vp));
                const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&vv.x));
                const float2 v1 = __half22float2(*reinterpret_cast<const __half2*>(&vv.y));
                acc[0] = fmaf(pj, v0.x, acc[0]); acc[1] = fmaf(pj, v0.y, acc[1]);
                acc[2 % DPL] = fmaf(pj, v1.x, acc[2 % DPL]); acc[3 % DPL] = fmaf(pj, v1.y, acc[3 % DPL]);
            } else {
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[d] = fmaf(pj, __half2float(vp[d]), acc[d]);
            }
        }
    }
    if (spans == 1) {
        float* op = out + ((long long)t * q_heads + qh) * HD + lane * DPL;
        const float inv = 1.0f / total;
#pragma unroll
        for (int d = 0; d < DPL; ++d) op[d] = acc[d] * inv;
    } else {
        float* pp = partial + (((long long)(t - token_base) * q_heads + qh) * max_spans + span) * (HD + 2);
#pragma unroll
        for (int d = 0; d < DPL; ++d) pp[lane * DPL + d] = acc[d];
        if (lane == 0) { pp[HD] = run_max; pp[HD + 1] = total; }
    }
}

// Merge a token's spans in span order: out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M).
template <int HD>
__global__ void attention_merge_kernel(const float* __restrict__ partial, const int32_t* __restrict__ token_pos,
                                       int token_base, int q_heads, int window, int max_spans,
                                       float* __restrict__ out) {
    const int t = token_base + blockIdx.x / q_heads, qh = blockIdx.x % q_heads;
    const int pos = token_pos[t];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int spans = (pos + 1 - first + kAttnSpanKeys - 1) / kAttnSpanKeys;
    if (spans <= 1) return;  // written directly by the span kernel
    const float* pp = partial + ((long long)(t - token_base) * q_heads + qh) * max_spans * (HD + 2);
    float top = -INFINITY;
    for (int s = 0; s < spans; ++s) top = fmaxf(top, pp[s * (HD + 2) + HD]);
    float denom = 0.0f;
    for (int s = 0; s < spans; ++s) denom += pp[s * (HD + 2) + HD + 1] * expf(pp[s * (HD + 2) + HD] - top);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float sum = 0.0f;
        for (int s = 0; s < spans; ++s) sum = fmaf(pp[s * (HD + 2) + d], expf(pp[s * (HD + 2) + HD] - top), sum);
        out[((long long)t * q_heads + qh) * HD + d] = sum / denom;
    }
}

template <int HD>
cudaError_t launch_hd(cudaStream_t stream, const float* q, const __half* cache_k, const __half* cache_v,
                      const int32_t* page_tables, int pages_per_sequence, const int32_t* token_seq,
                      const int32_t* token_pos, int n_tokens, int q_heads, int kv_heads, int window, int max_keys,
                      float* partial, size_t partial_bytes, float* out, int* launches) {
    const int q_per_kv = q_heads / kv_heads;
    const int max_spans = (max_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
    const size_t per_token = (size_t)q_heads * max_spans * (HD + 2) * sizeof(float);
    int chunk = n_tokens;
    if (max_spans > 1) {
        if (partial == nullptr || partial_bytes < per_token) return cudaErrorInvalidValue;
        chunk = (int)std::min<size_t>((size_t)n_tokens, partial_bytes / per_token);
    }
    for (int base = 0; base < n_tokens; base += chunk) {
        const int n = std::min(chunk, n_tokens - base);
        dim3 grid(n * kv_heads, max_spans);
        attention_span_kernel<HD><<<grid, q_per_kv * 32, q_per_kv * HD * sizeof(float), stream>>>(
            q, cache_k, cache_v, page_tables, pages_per_sequence, token_seq, token_pos, base, q_heads, kv_heads,
            window, max_spans, partial, out);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        if (launches) ++*launches;
        if (max_spans > 1) {
            attention_merge_kernel<HD><<<n * q_heads, HD < 128 ? 64 : 128, 0, stream>>>(partial, token_pos, base, q_heads,
                                                                                     window, max_spans, out);
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
            if (launches) ++*launches;
        }
    }
    return cudaSuccess;
}

}  // namespace

cudaError_t launch_attention(cudaStream_t stream, const float* q, const __half* cache_k, const __half* cache_v,
                             const int32_t* page_tables, int pages_per_sequence, const int32_t* token_seq,
                             const int32_t* token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                             int window, int max_keys, float* partial, size_t partial_bytes, float* out,
                             int* launches) {
    if (n_tokens <= 0) return cudaSuccess;
    if (q_heads % kv_heads != 0 || q_heads / kv_heads > 32 || max_keys <= 0) return cudaErrorInvalidValue;
    if (window > 0) max_keys = std::min(max_keys, window);
#define RIBN_ATTN(D)                                                                                          \
    return launch_hd<D>(stream, q, cache_k, cache_v, page_tables, pages_per_sequence, token_seq, token_pos, \
                        n_tokens, q_heads, kv_heads, window, max_keys, partial, partial_bytes, out, launches)
    switch (head_dim) {
        case 32: RIBN_ATTN(32);
        case 64: RIBN_ATTN(64);
        case 128: RIBN_ATTN(128);
        case 256: RIBN_ATTN(256);
        default: return cudaErrorInvalidValue;
    }
#undef RIBN_ATTN
}

}  // namespace ribn
