// Paged-KV ragged attention for decode rows and prefill chunks: split-KV
// ("flash-decoding") over fixed 64-key spans with an online softmax, then a
// deterministic merge of the spans.
//
// One CTA serves one (token, kv head, span); its warps are the q heads of the
// GQA group, so the group's K/V rows are fetched once per CTA and shared
// through L1.  Inside a warp the 32 lanes first take 32 different keys (a full
// head_dim dot product each, no cross-lane reduction, all loads in flight at
// once), then regroup as 4 key groups x 8 dim chunks for P.V, so every lane
// again issues independent 128-bit loads; the key groups are folded together
// once at the end of the span.  Spans depend only on the token's own key
// range, never on what else is in the batch, so a token's result is
// bit-identical whatever it is batched with and wherever its pages live.
//
// The decode form (FUSED) also applies the per-head Q/K RMSNorm and the NeoX
// rotary and appends the new K/V row to the paged cache: the CTA that owns
// the span holding the token's own position computes that row, stores it, and
// serves it to its warps from shared memory.  Results leave in F32 and,
// optionally, in the tensor-core operand form the output projection consumes.
//
// The reference's two-pass form with a global scores buffer
// (crates/nvidia/src/model_ops.rs:441-545) is replaced, not translated.
#include <cuda_fp16.h>
#include <math.h>

#include <algorithm>

#include "gemv.cuh"
#include "kernels.cuh"
#include "operand.cuh"

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

struct AttnArgs {
    const float* q;            // [T][q_heads][HD]; raw projections when fused
    const float* k_new;        // [T][kv_heads][HD] raw (fused only)
    const float* v_new;        // [T][kv_heads][HD] (fused only)
    const float* q_norm;       // [HD] (fused only)
    const float* k_norm;       // [HD] (fused only)
    const float* inv_freq;     // [HD / 2] (fused only)
    float eps;
    __half* cache_k;
    __half* cache_v;
    const int32_t* page_tables;
    int pages_per_sequence;
    const int32_t* token_seq;
    const int32_t* token_pos;
    const int32_t* token_slot; // physical slot of the token's own position (fused only)
    int token_base;
    int q_heads, kv_heads, window, max_spans;
    float* partial;
    float* out;                // [T][q_heads][HD]
    ActOperand operand;        // optional operand form of `out`, K = q_heads * HD
};

// RMSNorm + NeoX rotary of one head vector held lane-strided: element i of a
// lane is dimension lane + 32 i, so dimension d and its partner d + HD/2 sit
// in the same lane (i and i + DPL/2).
template <int HD>
__device__ __forceinline__ void norm_rope(float (&x)[HD / 32], const float* weight, const float* inv_freq, float eps,
                                          float pos, int lane) {
    constexpr int DPL = HD / 32;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int i = 0; i < DPL; ++i) x[i] = x[i] * inv * weight[lane + 32 * i];
#pragma unroll
    for (int i = 0; i < DPL / 2; ++i) {
        const float theta = pos * inv_freq[lane + 32 * i];
        const float s = sinf(theta), c = cosf(theta);
        const float x0 = x[i], x1 = x[i + DPL / 2];
        x[i] = x0 * c - x1 * s;
        x[i + DPL / 2] = x0 * s + x1 * c;
    }
}

// One warp's share of a span: query head `qh` of token `t` against keys [begin, end), whose K / V rows sit in
// shared memory from position `tile_begin` on.  Writes the final output when the token has a single span,
// else this span's partial sums.  Every span kernel runs exactly this arithmetic in this order.
template <int HD>
__device__ __forceinline__ void span_compute(const AttnArgs& a, float* qs, const __half* k_tile, const __half* v_tile,
                                             int tile_begin, int begin, int end, int t, int qh, int span, int spans,
                                             float scale, int lane) {
    constexpr int DPL = HD / 32;
    constexpr int CH = HD / 8;
    constexpr int kRowHalfs = HD + 8;
    const int kg = lane >> 3, dc = lane & 7;
    float acc[CH];
#pragma unroll
    for (int d = 0; d < CH; ++d) acc[d] = 0.0f;
    float run_max = -INFINITY, total = 0.0f;
    for (int base = begin; base < end; base += 32) {
        const int key = base + lane;
        const bool live = key < end;
        float s = -INFINITY;
        if (live) {
            const uint4* kp = reinterpret_cast<const uint4*>(k_tile + (key - tile_begin) * kRowHalfs);
            uint4 kk[HD / 8];
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) kk[i] = kp[i];
            // packed FP32 pairs (sm_100): even and odd dimensions accumulate side by side
            float2 dot2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                const float4 qa = *reinterpret_cast<const float4*>(qs + i * 8);
                const float4 qb = *reinterpret_cast<const float4*>(qs + i * 8 + 4);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].x));
                const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].z));
                const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].w));
                dot2 = __ffma2_rn(make_float2(qa.x, qa.y), k0, dot2);
                dot2 = __ffma2_rn(make_float2(qa.z, qa.w), k1, dot2);
                dot2 = __ffma2_rn(make_float2(qb.x, qb.y), k2, dot2);
                dot2 = __ffma2_rn(make_float2(qb.z, qb.w), k3, dot2);
            }
            s = (dot2.x + dot2.y) * scale;
        }
        const float new_max = fmaxf(run_max, warp_max(s));
        const float factor = expf(run_max - new_max);  // 0 on the first tile (run_max = -inf)
        const float p = live ? expf(s - new_max) : 0.0f;
        total = total * factor + warp_sum(p);
#pragma unroll
        for (int d = 0; d < CH; ++d) acc[d] *= factor;
        run_max = new_max;
        const int count = min(32, end - base);
        // P.V: lane (kg, dc) takes keys j = 4 jj + kg and dims [dc * CH, dc * CH + CH)
        uint4 vv[8][CH / 8];
        float pj[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
            const int j = jj * 4 + kg;
            pj[jj] = __shfl_sync(0xffffffffu, p, j);
            const __half* vp = v_tile + (base - tile_begin + j) * kRowHalfs;
            if (j < count) {
#pragma unroll
                for (int c = 0; c < CH / 8; ++c) vv[jj][c] = *reinterpret_cast<const uint4*>(vp + dc * CH + c * 8);
            } else {
#pragma unroll
                for (int c = 0; c < CH / 8; ++c) vv[jj][c] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
#pragma unroll
            for (int c = 0; c < CH / 8; ++c) {
                const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].x));
                const float2 v1 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].y));
                const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].z));
                const float2 v3 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].w));
                float* o = acc + c * 8;
                const float2 pp = make_float2(pj[jj], pj[jj]);
                const float2 o0 = __ffma2_rn(pp, v0, make_float2(o[0], o[1]));
                const float2 o1 = __ffma2_rn(pp, v1, make_float2(o[2], o[3]));
                const float2 o2 = __ffma2_rn(pp, v2, make_float2(o[4], o[5]));
                const float2 o3 = __ffma2_rn(pp, v3, make_float2(o[6], o[7]));
                o[0] = o0.x; o[1] = o0.y; o[2] = o1.x; o[3] = o1.y; o[4] = o2.x; o[5] = o2.y; o[6] = o3.x; o[7] = o3.y;
            }
        }
    }
    // Fold the four key groups (fixed order: xor 8, then xor 16).
#pragma unroll
    for (int d = 0; d < CH; ++d) {
        acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 8);
        acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 16);
    }
    if (spans == 1) {
        if (kg == 0) {
            const float inv = 1.0f / total;
            float* op = a.out + ((long long)t * a.q_heads + qh) * HD + dc * CH;
#pragma unroll
            for (int d = 0; d < CH; ++d) { acc[d] *= inv; op[d] = acc[d]; qs[dc * CH + d] = acc[d]; }
        }
        if (a.operand.dig != nullptr) {
            // back to one input per lane: lane takes dims lane + 32 i of this head
            __syncwarp();
            ActOperand op = a.operand;
            op.ss32 = nullptr;
            const int K = a.q_heads * HD, m = t - a.token_base;
#pragma unroll
            for (int i = 0; i < DPL; ++i) operand_store_span(op, m, K, (qh * HD) / 32 + i, lane, qs[lane + 32 * i], 0.0f);
        }
    } else if (kg == 0) {
        float* pp = a.partial + (((long long)(t - a.token_base) * a.q_heads + qh) * a.max_spans + span) * (HD + 2);
#pragma unroll
        for (int d = 0; d < CH; ++d) pp[dc * CH + d] = acc[d];
        if (dc == 0) { pp[HD] = run_max; pp[HD + 1] = total; }
    }
}

template <int HD, bool FUSED>
__global__ void attention_span_kernel(const AttnArgs a) {
    constexpr int DPL = HD / 32;  // dims per lane in the lane-strided layout
    constexpr int CH = HD / 8;    // dims per lane in the P.V phase (8 chunks x 4 key groups)
    // Programmatic dependent launch: wait for the projections that produced q/k/v, then let the next
    // kernel (which first only prefetches weights) start.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char attn_smem[];
    constexpr int kRowHalfs = HD + 8;  // staged K / V rows, padded by 16 bytes so that a lane per key reads conflict-free
    float* q_smem = reinterpret_cast<float*>(attn_smem);                                 // [warps][HD]
    __half* k_tile = reinterpret_cast<__half*>(attn_smem + (size_t)(blockDim.x >> 5) * HD * sizeof(float));  // [64][kRowHalfs]
    __half* v_tile = k_tile + kAttnSpanKeys * kRowHalfs;                                 // [64][kRowHalfs]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q_per_kv = a.q_heads / a.kv_heads;
    const int t = a.token_base + blockIdx.x / a.kv_heads, kvh = blockIdx.x % a.kv_heads;
    const int span = blockIdx.y;
    const int qh = kvh * q_per_kv + warp;
    const int pos = a.token_pos[t];
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int n_keys = pos + 1 - first;
    const int spans = (n_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
    if (span >= spans) return;
    const int begin = first + span * kAttnSpanKeys;
    const int end = min(pos + 1, begin + kAttnSpanKeys);
    const int32_t* table = a.page_tables + (long long)(a.token_seq != nullptr ? a.token_seq[t] : 0) * a.pages_per_sequence;
    const float scale = 1.0f / sqrtf((float)HD);
    const long long row_stride = (long long)a.kv_heads * HD;
    const bool owns_self = FUSED && span == spans - 1;  // this CTA's span holds the token's own position

    // The span's K and V rows come to shared memory once for all the query heads of the group, as
    // asynchronous 16-byte copies that bypass the registers: every piece of the span is in flight at once.
    // The span's page-table entries (at most five 16-token pages) are fetched first, so that no copy waits
    // on a table lookup of its own.
    __shared__ long long page_base[8];
    {
        const int page0 = begin / kPageTokens, pages = (end - 1) / kPageTokens - page0 + 1;
        if ((int)threadIdx.x < pages) page_base[threadIdx.x] = (long long)table[page0 + threadIdx.x] * kPageTokens;
        __syncthreads();
        constexpr int kChunks = HD / 8;  // 16-byte pieces per row (a power of two: index arithmetic is shifts)
        const int pieces = (end - begin) * kChunks;
        for (int idx = threadIdx.x; idx < pieces; idx += blockDim.x) {
            const int r = idx / kChunks, c = idx % kChunks;
            const int key = begin + r;
            if (owns_self && key == pos) continue;  // the token's own row is produced below
            const long long phys = page_base[key / kPageTokens - page0] + key % kPageTokens;
            const long long at = phys * row_stride + (long long)kvh * HD + c * 8;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(k_tile + r * kRowHalfs + c * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(a.cache_k + at) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(kAttnSpanKeys * kRowHalfs * sizeof(__half))),
                         "l"(a.cache_v + at)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    float* qs = q_smem + warp * HD;
    {
        const float* qp = a.q + ((long long)t * a.q_heads + qh) * HD;
        float x[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) x[i] = qp[lane + 32 * i];
        if (FUSED) norm_rope<HD>(x, a.q_norm, a.inv_freq, a.eps, (float)pos, lane);
#pragma unroll
        for (int i = 0; i < DPL; ++i) qs[lane + 32 * i] = x[i];
    }
    if (owns_self && warp == 0) {
        // The token's own K (normalised, rotated) and V, rounded to F16 exactly as the cache holds them.
        const float* kp = a.k_new + ((long long)t * a.kv_heads + kvh) * HD;
        const float* vp = a.v_new + ((long long)t * a.kv_heads + kvh) * HD;
        float x[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) x[i] = kp[lane + 32 * i];
        norm_rope<HD>(x, a.k_norm, a.inv_freq, a.eps, (float)pos, lane);
        __half* ck = a.cache_k + (long long)a.token_slot[t] * row_stride + (long long)kvh * HD;
        __half* cv = a.cache_v + (long long)a.token_slot[t] * row_stride + (long long)kvh * HD;
        __half* k_self = k_tile + (pos - begin) * kRowHalfs;
        __half* v_self = v_tile + (pos - begin) * kRowHalfs;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            const __half kh = __float2half_rn(x[i]), vh = __float2half_rn(vp[d]);
            k_self[d] = kh; v_self[d] = vh;
            ck[d] = kh; cv[d] = vh;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    span_compute<HD>(a, qs, k_tile, v_tile, begin, begin, end, t, qh, span, spans, scale, lane);
}

// Prefill steps: consecutive tokens of one sequence see the same keys of a span (up to the diagonal), so a
// CTA walks kAttnRowsPerCta consecutive tokens and stages the span's K / V rows once for all of them (the
// copies from L2 into shared memory are what bounds a per-token launch at these sizes).  A token of another
// sequence, or one whose span differs, restages.  The cache already holds every K / V row of the step.
constexpr int kAttnRowsPerCta = 4;

template <int HD>
__global__ void attention_span_rows_kernel(const AttnArgs a, const int n_tokens) {
    constexpr int DPL = HD / 32;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char attn_smem[];
    constexpr int kRowHalfs = HD + 8;
    float* q_smem = reinterpret_cast<float*>(attn_smem);                                 // [warps][HD]
    __half* k_tile = reinterpret_cast<__half*>(attn_smem + (size_t)(blockDim.x >> 5) * HD * sizeof(float));  // [64][kRowHalfs]
    __half* v_tile = k_tile + kAttnSpanKeys * kRowHalfs;
    __shared__ long long page_base[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q_per_kv = a.q_heads / a.kv_heads;
    const int group = blockIdx.x / a.kv_heads, kvh = blockIdx.x % a.kv_heads;
    const int span = blockIdx.y;
    const int qh = kvh * q_per_kv + warp;
    const float scale = 1.0f / sqrtf((float)HD);
    const long long row_stride = (long long)a.kv_heads * HD;
    float* qs = q_smem + warp * HD;
    int staged_seq = -1, staged_begin = -1, staged_end = 0;
    for (int r = 0; r < kAttnRowsPerCta; ++r) {
        const int local = group * kAttnRowsPerCta + r;
        if (local >= n_tokens) break;
        const int t = a.token_base + local;
        const int pos = a.token_pos[t];
        const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
        const int n_keys = pos + 1 - first;
        const int spans = (n_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
        if (span >= spans) continue;
        const int begin = first + span * kAttnSpanKeys;
        const int end = min(pos + 1, begin + kAttnSpanKeys);
        const int seq = a.token_seq != nullptr ? a.token_seq[t] : 0;
        if (seq != staged_seq || begin != staged_begin || end > staged_end) {
            // Stage [begin, stage_end): far enough for the following tokens of this sequence in the CTA.
            int stage_end = end;
            for (int r2 = r + 1; r2 < kAttnRowsPerCta && group * kAttnRowsPerCta + r2 < n_tokens; ++r2) {
                const int t2 = t + (r2 - r);
                if ((a.token_seq != nullptr ? a.token_seq[t2] : 0) != seq) break;
                const int pos2 = a.token_pos[t2];
                if (pos2 < pos || (a.window > 0 ? max(0, pos2 - a.window + 1) : 0) != first) break;
                stage_end = max(stage_end, min(pos2 + 1, begin + kAttnSpanKeys));
            }
            __syncthreads();  // every warp has finished with the previous tile
            const int32_t* table = a.page_tables + (long long)seq * a.pages_per_sequence;
            const int page0 = begin / kPageTokens, pages = (stage_end - 1) / kPageTokens - page0 + 1;
            if ((int)threadIdx.x < pages) page_base[threadIdx.x] = (long long)table[page0 + threadIdx.x] * kPageTokens;
            __syncthreads();
            constexpr int kChunks = HD / 8;
            const int pieces = (stage_end - begin) * kChunks;
            for (int idx = threadIdx.x; idx < pieces; idx += blockDim.x) {
                const int row = idx / kChunks, c = idx % kChunks;
                const int key = begin + row;
                const long long phys = page_base[key / kPageTokens - page0] + key % kPageTokens;
                const long long at = phys * row_stride + (long long)kvh * HD + c * 8;
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(k_tile + row * kRowHalfs + c * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(a.cache_k + at) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(kAttnSpanKeys * kRowHalfs * sizeof(__half))),
                             "l"(a.cache_v + at)
                             : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            staged_seq = seq; staged_begin = begin; staged_end = stage_end;
        }
        {
            const float* qp = a.q + ((long long)t * a.q_heads + qh) * HD;
            __syncwarp();  // the previous token's reads of qs are done
#pragma unroll
            for (int i = 0; i < DPL; ++i) qs[lane + 32 * i] = qp[lane + 32 * i];
            __syncwarp();
        }
        span_compute<HD>(a, qs, k_tile, v_tile, begin, begin, end, t, qh, span, spans, scale, lane);
    }
}

// The same span computation with every warp reading its keys straight from the cache: fewer steps in
// series, which wins when the launch has too few CTAs to fill the GPU (decode at batch 1 or 2).  Both
// kernels perform identical arithmetic in identical order.
template <int HD, bool FUSED, bool EARLY>
__global__ void __launch_bounds__(EARLY ? 256 : 512) attention_span_direct_kernel(const AttnArgs a) {
    constexpr int DPL = HD / 32;  // dims per lane in the lane-strided layout
    constexpr int CH = HD / 8;    // dims per lane in the P.V phase (8 chunks x 4 key groups)
    // Before the programmatic dependency resolves: the span's K / V rows of earlier positions were written by
    // earlier steps, and the step's positions and page tables by kernels that completed before the projection
    // ahead of this one began, so warp 0 asks L2 for those rows while that projection drains.
    if (threadIdx.x < 32) {
        const int pt = a.token_base + blockIdx.x / a.kv_heads, pkvh = blockIdx.x % a.kv_heads;
        const int ppos = a.token_pos[pt];
        const int pfirst = a.window > 0 ? max(0, ppos - a.window + 1) : 0;
        const int pbegin = pfirst + (int)blockIdx.y * kAttnSpanKeys, pend = min(ppos + 1, pbegin + kAttnSpanKeys);
        const int32_t* ptable = a.page_tables + (long long)(a.token_seq != nullptr ? a.token_seq[pt] : 0) * a.pages_per_sequence;
        for (int key = pbegin + (int)threadIdx.x; key < pend; key += 32) {
            if (FUSED && key == ppos) continue;  // the token's own row does not exist yet
            const long long phys = (long long)ptable[key / kPageTokens] * kPageTokens + key % kPageTokens;
            const long long at = phys * (long long)a.kv_heads * HD + (long long)pkvh * HD;
#pragma unroll
            for (int line = 0; line < HD * 2 / 128; ++line) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a.cache_k + at + line * 64));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a.cache_v + at + line * 64));
            }
        }
    }
    // Programmatic dependent launch: wait for the projections that produced q/k/v, then let the next
    // kernel (which first only prefetches weights) start.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char attn_smem[];
    float* q_smem = reinterpret_cast<float*>(attn_smem);                                 // [warps][HD]
    __half* k_self = reinterpret_cast<__half*>(attn_smem + (size_t)(blockDim.x >> 5) * HD * sizeof(float));  // [HD]
    __half* v_self = k_self + HD;                                                         // [HD]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q_per_kv = a.q_heads / a.kv_heads;
    const int t = a.token_base + blockIdx.x / a.kv_heads, kvh = blockIdx.x % a.kv_heads;
    const int span = blockIdx.y;
    const int qh = kvh * q_per_kv + warp;
    const int pos = a.token_pos[t];
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int n_keys = pos + 1 - first;
    const int spans = (n_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
    if (span >= spans) return;
    const int begin = first + span * kAttnSpanKeys;
    const int end = min(pos + 1, begin + kAttnSpanKeys);
    const int32_t* table = a.page_tables + (long long)(a.token_seq != nullptr ? a.token_seq[t] : 0) * a.pages_per_sequence;
    const float scale = 1.0f / sqrtf((float)HD);
    const long long row_stride = (long long)a.kv_heads * HD;
    const bool owns_self = FUSED && span == spans - 1;  // this CTA's span holds the token's own position

    float* qs = q_smem + warp * HD;
    {
        const float* qp = a.q + ((long long)t * a.q_heads + qh) * HD;
        float x[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) x[i] = qp[lane + 32 * i];
        if (FUSED) norm_rope<HD>(x, a.q_norm, a.inv_freq, a.eps, (float)pos, lane);
#pragma unroll
        for (int i = 0; i < DPL; ++i) qs[lane + 32 * i] = x[i];
    }
    if (owns_self && warp == 0) {
        // The token's own K (normalised, rotated) and V, rounded to F16 exactly as the cache holds them.
        const float* kp = a.k_new + ((long long)t * a.kv_heads + kvh) * HD;
        const float* vp = a.v_new + ((long long)t * a.kv_heads + kvh) * HD;
        float x[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) x[i] = kp[lane + 32 * i];
        norm_rope<HD>(x, a.k_norm, a.inv_freq, a.eps, (float)pos, lane);
        __half* ck = a.cache_k + (long long)a.token_slot[t] * row_stride + (long long)kvh * HD;
        __half* cv = a.cache_v + (long long)a.token_slot[t] * row_stride + (long long)kvh * HD;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            const __half kh = __float2half_rn(x[i]), vh = __float2half_rn(vp[d]);
            k_self[d] = kh; v_self[d] = vh;
            ck[d] = kh; cv[d] = vh;
        }
    }
    if (FUSED) __syncthreads(); else __syncwarp();

    const int kg = lane >> 3, dc = lane & 7;
    float acc[CH];
#pragma unroll
    for (int d = 0; d < CH; ++d) acc[d] = 0.0f;
    float run_max = -INFINITY, total = 0.0f;
    for (int base = begin; base < end; base += 32) {
        const int key = base + lane;
        const bool live = key < end;
        long long phys = 0;
        float s = -INFINITY;
        uint4 kk[HD / 8];
        if (live) {
            phys = (long long)table[key / kPageTokens] * kPageTokens + key % kPageTokens;
            const uint4* kp = (owns_self && key == pos)
                                  ? reinterpret_cast<const uint4*>(k_self)
                                  : reinterpret_cast<const uint4*>(a.cache_k + phys * row_stride + (long long)kvh * HD);
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) kk[i] = kp[i];
        }
        // The V rows are requested right behind the K rows (their addresses need only the page lookup), so the two
        // round trips to memory overlap; lane (kg, dc) takes keys j = 4 jj + kg and dims [dc * CH, dc * CH + CH).
        const int count = min(32, end - base);
        uint4 vv[8][CH / 8];
        auto load_values = [&]() {
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const int j = jj * 4 + kg;
                const long long pphys = __shfl_sync(0xffffffffu, phys, j);
                const bool self = owns_self && base + j == pos;
                const __half* vp = self ? v_self : a.cache_v + pphys * row_stride + (long long)kvh * HD;
                if (j < count) {
#pragma unroll
                    for (int c = 0; c < CH / 8; ++c) vv[jj][c] = *reinterpret_cast<const uint4*>(vp + dc * CH + c * 8);
                } else {
#pragma unroll
                    for (int c = 0; c < CH / 8; ++c) vv[jj][c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        };
        // EARLY: groups of at most 8 query heads (256 threads) and head dims up to 128 keep both row sets in registers
        constexpr bool kEarlyValues = EARLY;
        if (kEarlyValues) load_values();
        if (live) {
            // packed FP32 pairs (sm_100): even and odd dimensions accumulate side by side
            float2 dot2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                const float4 qa = *reinterpret_cast<const float4*>(qs + i * 8);
                const float4 qb = *reinterpret_cast<const float4*>(qs + i * 8 + 4);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].x));
                const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].z));
                const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kk[i].w));
                dot2 = __ffma2_rn(make_float2(qa.x, qa.y), k0, dot2);
                dot2 = __ffma2_rn(make_float2(qa.z, qa.w), k1, dot2);
                dot2 = __ffma2_rn(make_float2(qb.x, qb.y), k2, dot2);
                dot2 = __ffma2_rn(make_float2(qb.z, qb.w), k3, dot2);
            }
            s = (dot2.x + dot2.y) * scale;
        }
        const float new_max = fmaxf(run_max, warp_max(s));
        const float factor = expf(run_max - new_max);  // 0 on the first tile (run_max = -inf)
        const float p = live ? expf(s - new_max) : 0.0f;
        total = total * factor + warp_sum(p);
#pragma unroll
        for (int d = 0; d < CH; ++d) acc[d] *= factor;
        run_max = new_max;
        if (!kEarlyValues) load_values();
        float pj[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) pj[jj] = __shfl_sync(0xffffffffu, p, jj * 4 + kg);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
#pragma unroll
            for (int c = 0; c < CH / 8; ++c) {
                const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].x));
                const float2 v1 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].y));
                const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].z));
                const float2 v3 = __half22float2(*reinterpret_cast<const __half2*>(&vv[jj][c].w));
                float* o = acc + c * 8;
                const float2 pp = make_float2(pj[jj], pj[jj]);
                const float2 o0 = __ffma2_rn(pp, v0, make_float2(o[0], o[1]));
                const float2 o1 = __ffma2_rn(pp, v1, make_float2(o[2], o[3]));
                const float2 o2 = __ffma2_rn(pp, v2, make_float2(o[4], o[5]));
                const float2 o3 = __ffma2_rn(pp, v3, make_float2(o[6], o[7]));
                o[0] = o0.x; o[1] = o0.y; o[2] = o1.x; o[3] = o1.y; o[4] = o2.x; o[5] = o2.y; o[6] = o3.x; o[7] = o3.y;
            }
        }
    }
    // Fold the four key groups (fixed order: xor 8, then xor 16).
#pragma unroll
    for (int d = 0; d < CH; ++d) {
        acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 8);
        acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 16);
    }
    if (spans == 1) {
        if (kg == 0) {
            const float inv = 1.0f / total;
            float* op = a.out + ((long long)t * a.q_heads + qh) * HD + dc * CH;
#pragma unroll
            for (int d = 0; d < CH; ++d) { acc[d] *= inv; op[d] = acc[d]; qs[dc * CH + d] = acc[d]; }
        }
        if (a.operand.dig != nullptr) {
            // back to one input per lane: lane takes dims lane + 32 i of this head
            __syncwarp();
            ActOperand op = a.operand;
            op.ss32 = nullptr;
            const int K = a.q_heads * HD, m = t - a.token_base;
#pragma unroll
            for (int i = 0; i < DPL; ++i) operand_store_span(op, m, K, (qh * HD) / 32 + i, lane, qs[lane + 32 * i], 0.0f);
        }
    } else if (kg == 0) {
        float* pp = a.partial + (((long long)(t - a.token_base) * a.q_heads + qh) * a.max_spans + span) * (HD + 2);
#pragma unroll
        for (int d = 0; d < CH; ++d) pp[dc * CH + d] = acc[d];
        if (dc == 0) { pp[HD] = run_max; pp[HD + 1] = total; }
    }
}

// Merge a token's spans in span order: out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M).
// One block of HD threads per (token, q head).
template <int HD>
__global__ void attention_merge_kernel(const AttnArgs a) {
    __shared__ float weight[kAttnMaxSpans];
    __shared__ float denom_s;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int t = a.token_base + blockIdx.x / a.q_heads, qh = blockIdx.x % a.q_heads;
    const int pos = a.token_pos[t];
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int spans = (pos + 1 - first + kAttnSpanKeys - 1) / kAttnSpanKeys;
    if (spans <= 1) return;  // written directly by the span kernel
    const float* pp = a.partial + ((long long)(t - a.token_base) * a.q_heads + qh) * a.max_spans * (HD + 2);
    if (threadIdx.x < 32) {
        float top = -INFINITY;
        for (int s = threadIdx.x; s < spans; s += 32) top = fmaxf(top, pp[s * (HD + 2) + HD]);
        top = warp_max(top);
        float denom = 0.0f;  // per-lane partial sums in span order, folded in a fixed shuffle order
        for (int s = threadIdx.x; s < spans; s += 32) {
            const float w = expf(pp[s * (HD + 2) + HD] - top);
            weight[s] = w;
            denom += pp[s * (HD + 2) + HD + 1] * w;
        }
        denom = warp_sum(denom);
        if (threadIdx.x == 0) denom_s = denom;
    }
    __syncthreads();
    const int d = threadIdx.x;
    float sum = 0.0f;
    // eight spans' values are requested before the first is used (the additions keep span order)
    for (int s0 = 0; s0 < spans; s0 += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = s0 + u < spans ? pp[(s0 + u) * (HD + 2) + d] : 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (s0 + u < spans) sum = fmaf(v[u], weight[s0 + u], sum);
        }
    }
    const float value = sum / denom_s;
    a.out[((long long)t * a.q_heads + qh) * HD + d] = value;
    if (a.operand.dig != nullptr) {
        ActOperand op = a.operand;
        op.ss32 = nullptr;
        operand_store_span(op, t - a.token_base, a.q_heads * HD, (qh * HD + d) / 32, d & 31, value, 0.0f);
    }
}

template <typename Kernel>
cudaError_t launch_pdl(cudaStream_t stream, Kernel kernel, dim3 grid, int threads, size_t smem, const AttnArgs& a,
                       bool programmatic) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned int)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <typename Kernel>
cudaError_t launch_pdl(cudaStream_t stream, Kernel kernel, dim3 grid, int threads, size_t smem, const AttnArgs& a,
                       bool programmatic, int extra) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned int)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a, extra);
}

template <int HD>
cudaError_t launch_hd(cudaStream_t stream, AttnArgs a, bool fused, int n_tokens, int max_keys, size_t partial_bytes,
                      int* launches, bool programmatic = false) {
    const int q_per_kv = a.q_heads / a.kv_heads;
    a.max_spans = (max_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
    if (a.max_spans > kAttnMaxSpans) return cudaErrorInvalidValue;
    const size_t per_token = (size_t)a.q_heads * a.max_spans * (HD + 2) * sizeof(float);
    int chunk = n_tokens;
    if (a.max_spans > 1) {
        if (a.partial == nullptr || partial_bytes < per_token) return cudaErrorInvalidValue;
        chunk = (int)std::min<size_t>((size_t)n_tokens, partial_bytes / per_token);
    }
    if (a.operand.dig != nullptr && chunk < n_tokens) return cudaErrorInvalidValue;  // operand rows are launch-relative
    // Few CTAs: the direct kernel (shorter dependency chain); many: K / V rows staged once per query-head group.
    const bool staged = (long long)n_tokens * a.kv_heads * a.max_spans >= 1024;
    const size_t smem = staged ? (size_t)q_per_kv * HD * sizeof(float) + (size_t)2 * kAttnSpanKeys * (HD + 8) * sizeof(__half)
                               : (size_t)q_per_kv * HD * sizeof(float) + 2 * HD * sizeof(__half);
    if (smem > 48 * 1024) {
        // above the default limit (head_dim 256): opt in once per instantiation
        static bool configured_on[kMaxDevices] = {false};  // function attributes are per device
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
        bool& configured = configured_on[dev];
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(attention_span_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_span_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_span_rows_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            if (e != cudaSuccess) return e;
            configured = true;
        }
    }
    for (int base = 0; base < n_tokens; base += chunk) {
        const int n = std::min(chunk, n_tokens - base);
        a.token_base = base;
        dim3 grid(n * a.kv_heads, a.max_spans);
        cudaError_t e;
        if (staged && !fused && a.operand.dig == nullptr && n >= 4 * kAttnRowsPerCta) {
            // prefill-sized launches of tokens whose K / V rows are all in the cache: several tokens per staged span
            const dim3 row_grid((unsigned)((n + kAttnRowsPerCta - 1) / kAttnRowsPerCta) * a.kv_heads, a.max_spans);
            e = launch_pdl(stream, attention_span_rows_kernel<HD>, row_grid, q_per_kv * 32, smem, a, programmatic, n);
        } else if (staged) {
            e = fused ? launch_pdl(stream, attention_span_kernel<HD, true>, grid, q_per_kv * 32, smem, a, programmatic)
                      : launch_pdl(stream, attention_span_kernel<HD, false>, grid, q_per_kv * 32, smem, a, programmatic);
        } else {
            if (HD <= 128 && q_per_kv <= 8) {
                e = fused ? launch_pdl(stream, attention_span_direct_kernel<HD, true, (HD <= 128)>, grid, q_per_kv * 32, smem, a, programmatic)
                          : launch_pdl(stream, attention_span_direct_kernel<HD, false, (HD <= 128)>, grid, q_per_kv * 32, smem, a, programmatic);
            } else {
                e = fused ? launch_pdl(stream, attention_span_direct_kernel<HD, true, false>, grid, q_per_kv * 32, smem, a, programmatic)
                          : launch_pdl(stream, attention_span_direct_kernel<HD, false, false>, grid, q_per_kv * 32, smem, a, programmatic);
            }
        }
        if (e != cudaSuccess) return e;
        if (launches) ++*launches;
        if (a.max_spans > 1) {
            e = launch_pdl(stream, attention_merge_kernel<HD>, dim3(n * a.q_heads), HD, 0, a, programmatic);
            if (e != cudaSuccess) return e;
            if (launches) ++*launches;
        }
    }
    return cudaSuccess;
}

cudaError_t dispatch(cudaStream_t stream, const AttnArgs& a, bool fused, int head_dim, int n_tokens, int max_keys,
                     size_t partial_bytes, int* launches, bool programmatic = false) {
    switch (head_dim) {
        case 64: return launch_hd<64>(stream, a, fused, n_tokens, max_keys, partial_bytes, launches, programmatic);
        case 128: return launch_hd<128>(stream, a, fused, n_tokens, max_keys, partial_bytes, launches, programmatic);
        case 256: return launch_hd<256>(stream, a, fused, n_tokens, max_keys, partial_bytes, launches, programmatic);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_attention(cudaStream_t stream, const float* q, const __half* cache_k, const __half* cache_v,
                             const int32_t* page_tables, int pages_per_sequence, const int32_t* token_seq,
                             const int32_t* token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                             int window, int max_keys, float* partial, size_t partial_bytes, float* out,
                             int* launches) {
    if (n_tokens <= 0) return cudaSuccess;
    if (q_heads % kv_heads != 0 || q_heads / kv_heads > 32 || max_keys <= 0) return cudaErrorInvalidValue;
    if (head_dim == 32) {
        // Below 64 dims the span kernel's lane layout does not apply: the plain kernel serves.
        cudaError_t e = launch_attention_ref(stream, q, cache_k, cache_v, page_tables, pages_per_sequence, token_seq,
                                             token_pos, n_tokens, q_heads, kv_heads, head_dim, window, out);
        if (e == cudaSuccess && launches) ++*launches;
        return e;
    }
    if (window > 0) max_keys = std::min(max_keys, window);
    AttnArgs a{};
    a.q = q;
    a.cache_k = const_cast<__half*>(cache_k);
    a.cache_v = const_cast<__half*>(cache_v);
    a.page_tables = page_tables;
    a.pages_per_sequence = pages_per_sequence;
    a.token_seq = token_seq;
    a.token_pos = token_pos;
    a.q_heads = q_heads;
    a.kv_heads = kv_heads;
    a.window = window;
    a.partial = partial;
    a.out = out;
    return dispatch(stream, a, false, head_dim, n_tokens, max_keys, partial_bytes, launches);
}

cudaError_t launch_attention_decode(cudaStream_t stream, const DecodeAttention& d, int* launches) {
    if (d.n_tokens <= 0) return cudaSuccess;
    if (d.q_heads % d.kv_heads != 0 || d.q_heads / d.kv_heads > 32 || d.max_keys <= 0) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.q = d.q; a.k_new = d.k; a.v_new = d.v;
    a.q_norm = d.q_norm; a.k_norm = d.k_norm; a.inv_freq = d.inv_freq; a.eps = d.eps;
    a.cache_k = d.cache_k; a.cache_v = d.cache_v;
    a.page_tables = d.page_tables; a.pages_per_sequence = d.pages_per_sequence;
    a.token_seq = d.token_seq; a.token_pos = d.token_pos; a.token_slot = d.token_slot;
    a.q_heads = d.q_heads; a.kv_heads = d.kv_heads; a.window = d.window;
    a.partial = d.partial; a.out = d.out; a.operand = d.operand;
    const int max_keys = d.window > 0 ? std::min(d.max_keys, d.window) : d.max_keys;
    return dispatch(stream, a, true, d.head_dim, d.n_tokens, max_keys, d.partial_bytes, launches, d.programmatic);
}

}  // namespace ribn
