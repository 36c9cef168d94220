// Model-op kernels of the decode / chunked-prefill step: batch metadata,
// embedding, RMSNorm, per-head QK-norm + rotary + paged KV append, the plain
// one-warp-per-row GEMV and attention kernels used as on-device references,
// SwiGLU gating, residual add, greedy selection, and the seeded synthetic
// checkpoint generator.
#include <cooperative_groups.h>

#include "blocks.cuh"
#include "kernels.cuh"

namespace ribn {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float block_sum(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < warps; ++w) total += smem[w];
    return total;
}

// ---------------------------------------------------------------------------
// Ragged batch metadata.  One block; rows <= 1024.
// ---------------------------------------------------------------------------
__device__ void scan_rows(const int32_t* tokens, int n_rows, int32_t* cu /* smem [n_rows + 1] */) {
    // Serial by construction sizes (<= 1024 rows): a single warp-level pass.
    if (threadIdx.x < 32) {
        int carry = 0;
        for (int base = 0; base < n_rows; base += 32) {
            const int i = base + (int)threadIdx.x;
            int v = i < n_rows ? tokens[i] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, v, o);
                if ((int)threadIdx.x >= o) v += up;
            }
            if (i < n_rows) cu[i + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (threadIdx.x == 0) cu[0] = 0;
    }
    __syncthreads();
}

__device__ __forceinline__ int find_row(const int32_t* cu, int n_rows, int t) {
    int lo = 0, hi = n_rows - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__global__ void step_metadata_kernel(const RowDesc* rows, int n_rows, int n_tokens,
                                     const uint32_t* prompt_tokens, const uint32_t* next_token,
                                     const int32_t* page_tables, int pages_per_sequence, StepMeta meta) {
    extern __shared__ int32_t cu[];
    __shared__ int32_t row_tokens[1024];
    for (int i = threadIdx.x; i < n_rows; i += blockDim.x) row_tokens[i] = rows[i].tokens;
    __syncthreads();
    scan_rows(row_tokens, n_rows, cu);
    for (int i = threadIdx.x; i <= n_rows; i += blockDim.x) meta.cu_seqlens[i] = cu[i];
    for (int i = threadIdx.x; i < n_rows; i += blockDim.x) {
        if (rows[i].sample_row >= 0) {
            meta.sample_token[rows[i].sample_row] = cu[i + 1] - 1;
            meta.sample_slot[rows[i].sample_row] = rows[i].slot;
        }
    }
    for (int t = threadIdx.x; t < n_tokens; t += blockDim.x) {
        const int r = find_row(cu, n_rows, t);
        const RowDesc row = rows[r];
        const int local = t - cu[r];
        const int pos = row.prefix + local;
        const int page = page_tables[(long long)row.slot * pages_per_sequence + pos / kPageTokens];
        meta.token_row[t] = r;
        meta.token_seq[t] = row.slot;
        meta.token_pos[t] = pos;
        meta.token_slot[t] = page * kPageTokens + pos % kPageTokens;
        meta.token_id[t] = row.token_offset >= 0 ? prompt_tokens[row.token_offset + local]
                                                 : next_token[row.slot];
    }
}

__global__ void batch_metadata_kernel(const int32_t* row_slot, const int32_t* row_prefix,
                                      const int32_t* row_tokens, int n_rows, int n_tokens,
                                      const int32_t* page_tables, int pages_per_sequence, int page_tokens,
                                      int32_t* cu_out, int32_t* token_row, int32_t* token_pos,
                                      int32_t* token_slot) {
    extern __shared__ int32_t cu[];
    scan_rows(row_tokens, n_rows, cu);
    for (int i = threadIdx.x; i <= n_rows; i += blockDim.x) cu_out[i] = cu[i];
    for (int t = threadIdx.x; t < n_tokens; t += blockDim.x) {
        const int r = find_row(cu, n_rows, t);
        const int pos = row_prefix[r] + (t - cu[r]);
        const int page = page_tables[(long long)row_slot[r] * pages_per_sequence + pos / page_tokens];
        token_row[t] = r;
        token_pos[t] = pos;
        token_slot[t] = page * page_tokens + pos % page_tokens;
    }
}

__global__ void synth_kv_kernel(__half* cache_k, __half* cache_v, long long layer_stride, int layers,
                                const int32_t* page_table, int tokens, int row_elems, uint64_t seed);
__global__ void gather_kv_kernel(const __half* cache, const int32_t* page_table, int tokens, int row_elems,
                                 __half* out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * row_elems) return;
    const int t = (int)(i / row_elems), e = (int)(i - (long long)t * row_elems);
    const long long phys = (long long)page_table[t / kPageTokens] * kPageTokens + t % kPageTokens;
    out[i] = cache[phys * row_elems + e];
}

// ---------------------------------------------------------------------------
// Embedding / dequantise
// ---------------------------------------------------------------------------
__global__ void embedding_kernel(int type, const unsigned char* table, int hidden, int vocab,
                                 const uint32_t* token_id, int n_tokens, float* out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * hidden) return;
    const int t = (int)(i / hidden), h = (int)(i - (long long)t * hidden);
    const uint32_t token = token_id[t];
    if (token >= (uint32_t)vocab) { out[i] = 0.0f; return; }
    const long long row_bytes = (long long)(hidden / block_elems(type)) * block_bytes(type);
    out[i] = row_element(type, table + (long long)token * row_bytes, h);
}

__global__ void dequantize_kernel(int type, const unsigned char* bytes, long long rows, long long cols,
                                  float* out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * cols) return;
    const long long r = i / cols, c = i - r * cols;
    const long long row_bytes = (cols / block_elems(type)) * block_bytes(type);
    out[i] = row_element(type, bytes + r * row_bytes, c);
}

// ---------------------------------------------------------------------------
// RMSNorm: one block per member vector (crates/nvidia/src/model_ops.rs:108-201)
// ---------------------------------------------------------------------------
__global__ void rms_norm_kernel(const float* x, const int32_t* index, const float* weight, int length,
                                float eps, float* out) {
    __shared__ float partial[32];
    const int m = blockIdx.x;
    const float* in = x + (long long)(index ? index[m] : m) * length;
    float* o = out + (long long)m * length;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < length; i += blockDim.x) sum = fmaf(in[i], in[i], sum);
    const float total = block_sum(sum, partial);
    const float inv = 1.0f / sqrtf(total / (float)length + eps);
    for (int i = threadIdx.x; i < length; i += blockDim.x) o[i] = in[i] * inv * weight[i];
}

// ---------------------------------------------------------------------------
// Reference GEMV: one warp per output row, lanes stride over k, up to 8
// members per pass (crates/nvidia/src/kernels/quantized/q4_k.cu:103-159 is the
// shape this mirrors; decode math is blocks.cuh's bit-exact element decoder).
// ---------------------------------------------------------------------------
constexpr int kRefMembers = 8;

__global__ void gemv_ref_kernel(int type, const unsigned char* w, long long n, long long k, const float* x,
                                int members, float* y, int accumulate) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const int m0 = blockIdx.y * kRefMembers;
    const long long row_bytes = (k / block_elems(type)) * block_bytes(type);
    const unsigned char* wr = w + row * row_bytes;
    float acc[kRefMembers];
#pragma unroll
    for (int m = 0; m < kRefMembers; ++m) acc[m] = 0.0f;
    for (long long kk = lane; kk < k; kk += 32) {
        const float wv = row_element(type, wr, kk);
#pragma unroll
        for (int m = 0; m < kRefMembers; ++m) {
            if (m0 + m < members) acc[m] = fmaf(wv, x[(long long)(m0 + m) * k + kk], acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < kRefMembers; ++m) {
        const float total = warp_sum(acc[m]);
        if (lane == 0 && m0 + m < members) {
            float* dst = y + (long long)(m0 + m) * n + row;
            *dst = accumulate ? *dst + total : total;
        }
    }
}

// ---------------------------------------------------------------------------
// elementwise
// ---------------------------------------------------------------------------
__global__ void silu_mul_kernel(const float* gate, const float* up, long long n, float* out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float g = gate[i];
        out[i] = g / (1.0f + expf(-g)) * up[i];
    }
}

__global__ void residual_add_kernel(float* acc, const float* inc, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) acc[i] += inc[i];
}

__global__ void f32_to_f16_kernel(const float* in, long long n, uint16_t* out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __half_as_ushort(__float2half_rn(in[i]));
}

__global__ void fill_f32_kernel(float* out, long long n, float value) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = value;
}

// Monotone unsigned key of a float; NaN never selected; ties -> lowest index
// (crates/nvidia/src/model_ops.rs:148-153, 203-260).
__device__ __forceinline__ unsigned int logit_key(float v) {
    const unsigned int bits = __float_as_uint(v);
    return (bits >> 31) ? ~bits : (bits ^ 0x80000000u);
}

// One cluster of PARTS CTAs per row: a vocabulary-sized row is a latency problem for one CTA (ten trips of loads),
// so every CTA scans its share of the row and leaves its best in the first CTA's shared memory.  Eight parts for
// the few rows of a decode step, fewer when the rows alone fill the GPU.
template <int PARTS>
__global__ void __cluster_dims__(PARTS, 1, 1) argmax_kernel(const float* logits, long long length, uint32_t* out,
                                                            const int32_t* slot, uint32_t* next_token) {
    constexpr int kArgmaxParts = PARTS;
    __shared__ unsigned long long best[32];
    __shared__ unsigned long long part_best[kArgmaxParts];
    cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
    const int part = (int)cluster.block_rank();
    const long long r = blockIdx.x / kArgmaxParts;
    const float* row = logits + r * length;
    // Packed (key << 32) | ~index: the maximum picks the largest key and, among
    // equal keys, the smallest index.
    unsigned long long mine = 0ull;
    auto consider = [&](float v, long long i) {
        if (v == v) {
            const unsigned long long cand =
                ((unsigned long long)logit_key(v) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
            // A key of 0 cannot occur for a non-NaN value, so `mine == 0` means "none yet".
            if (cand > mine) mine = cand;
        }
    };
    if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
        // Four independent 128-bit loads per thread and trip; the maximum does not depend on the visiting order.
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const long long quads = length / 4, q_begin = quads * part / kArgmaxParts, q_end = quads * (part + 1) / kArgmaxParts;
        const long long stride = (long long)blockDim.x * 4;
        for (long long q0 = q_begin; q0 < q_end; q0 += stride) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long q = q0 + (long long)u * blockDim.x + threadIdx.x;
                v[u] = q < q_end ? row4[q] : make_float4(NAN, NAN, NAN, NAN);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long i = (q0 + (long long)u * blockDim.x + threadIdx.x) * 4;
                consider(v[u].x, i); consider(v[u].y, i + 1); consider(v[u].z, i + 2); consider(v[u].w, i + 3);
            }
        }
        // the last part also takes what is left behind the last whole quad
        if (part == kArgmaxParts - 1) {
            for (long long i = quads * 4 + threadIdx.x; i < length; i += blockDim.x) consider(row[i], i);
        }
    } else {
        const long long begin = length * part / kArgmaxParts, end = length * (part + 1) / kArgmaxParts;
        for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) consider(row[i], i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
        if (other > mine) mine = other;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) best[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long top = 0ull;
        for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) top = best[w] > top ? best[w] : top;
        cluster.map_shared_rank(part_best, 0)[part] = top;
    }
    cluster.sync();   // every part's best is in the first CTA's shared memory
    if (part == 0 && threadIdx.x == 0) {
        unsigned long long top = 0ull;
        for (int q = 0; q < kArgmaxParts; ++q) top = part_best[q] > top ? part_best[q] : top;
        const uint32_t pick = top == 0ull ? 0u : 0xffffffffu - (uint32_t)(top & 0xffffffffull);
        out[r] = pick;
        if (slot != nullptr) next_token[slot[r]] = pick;
    }
}

// NeoX half-split rotary, theta = (float)pos * inv_freq[pair] with
// inv_freq[pair] = powf(base, -(2 pair) / rot) tabulated by the host
// (crates/nvidia/src/qwen_reference.rs:410-425).
__global__ void rope_neox_kernel(float* values, const long long* positions, int members, int heads,
                                 int head_dim, int half, const float* inv_freq) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int per_member = heads * half;
    if (i >= members * per_member) return;
    const int m = i / per_member, r = i - m * per_member;
    const int head = r / half, pair = r - head * half;
    const float theta = (float)positions[m] * inv_freq[pair];
    const float s = sinf(theta), c = cosf(theta);
    float* p = values + ((long long)m * heads + head) * head_dim;
    const float x0 = p[pair], x1 = p[half + pair];
    p[pair] = x0 * c - x1 * s;
    p[half + pair] = x0 * s + x1 * c;
}

// One warp per (token, head): heads [0, q_heads) are query heads, the rest are
// K heads, which also carry the V copy into the cache.
__global__ void qk_norm_rope_append_kernel(float* q, float* k, const float* v, const float* q_norm,
                                           const float* k_norm, const float* inv_freq,
                                           const int32_t* token_pos, const int32_t* token_slot,
                                           int n_tokens, int q_heads, int kv_heads, int head_dim, float eps,
                                           __half* cache_k, __half* cache_v) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int heads = q_heads + kv_heads;
    if (warp >= (long long)n_tokens * heads) return;
    const int t = (int)(warp / heads), h = (int)(warp - (long long)t * heads);
    const bool is_q = h < q_heads;
    float* vec = is_q ? q + ((long long)t * q_heads + h) * head_dim
                      : k + ((long long)t * kv_heads + (h - q_heads)) * head_dim;
    const float* weight = is_q ? q_norm : k_norm;
    float sum = 0.0f;
    for (int d = lane; d < head_dim; d += 32) sum = fmaf(vec[d], vec[d], sum);
    sum = warp_sum(sum);
    const float inv = 1.0f / sqrtf(sum / (float)head_dim + eps);
    const int half = head_dim >> 1;
    const float pos = (float)token_pos[t];
    for (int p = lane; p < half; p += 32) {
        const float x0 = vec[p] * inv * weight[p];
        const float x1 = vec[half + p] * inv * weight[half + p];
        const float theta = pos * inv_freq[p];
        const float s = sinf(theta), c = cosf(theta);
        const float r0 = x0 * c - x1 * s, r1 = x0 * s + x1 * c;
        vec[p] = r0;
        vec[half + p] = r1;
        if (!is_q) {
            __half* dst = cache_k + ((long long)token_slot[t] * kv_heads + (h - q_heads)) * head_dim;
            dst[p] = __float2half_rn(r0);
            dst[half + p] = __float2half_rn(r1);
        }
    }
    if (!is_q) {
        const float* src = v + ((long long)t * kv_heads + (h - q_heads)) * head_dim;
        __half* dst = cache_v + ((long long)token_slot[t] * kv_heads + (h - q_heads)) * head_dim;
        for (int d = lane; d < head_dim; d += 32) dst[d] = __float2half_rn(src[d]);
    }
}

// Reference attention: one warp per (token, q head); softmax computed online
// (running max and total rescaled when the max moves), lanes own contiguous
// dims (crates/nvidia/src/model_ops.rs:441-545 is the two-pass form).
template <int DIMS_PER_LANE>
__global__ void attention_ref_kernel(const float* q, const __half* cache_k, const __half* cache_v,
                                     const int32_t* page_tables, int pages_per_sequence,
                                     const int32_t* token_seq, const int32_t* token_pos, int n_tokens,
                                     int q_heads, int kv_heads, int window, float* out) {
    constexpr int HD = DIMS_PER_LANE * 32;
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (warp >= (long long)n_tokens * q_heads) return;
    const int t = (int)(warp / q_heads), qh = (int)(warp - (long long)t * q_heads);
    const int kvh = qh / (q_heads / kv_heads);
    const int pos = token_pos[t];
    const int32_t* table = page_tables + (long long)token_seq[t] * pages_per_sequence;
    const float scale = 1.0f / sqrtf((float)HD);
    float qv[DIMS_PER_LANE], acc[DIMS_PER_LANE];
    const float* qp = q + ((long long)t * q_heads + qh) * HD + lane * DIMS_PER_LANE;
#pragma unroll
    for (int d = 0; d < DIMS_PER_LANE; ++d) { qv[d] = qp[d]; acc[d] = 0.0f; }
    float run_max = -INFINITY, total = 0.0f;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    for (int key = first; key <= pos; ++key) {
        const long long phys = (long long)table[key / kPageTokens] * kPageTokens + key % kPageTokens;
        const __half* kp = cache_k + (phys * kv_heads + kvh) * HD + lane * DIMS_PER_LANE;
        float dot = 0.0f;
#pragma unroll
        for (int d = 0; d < DIMS_PER_LANE; ++d) dot = fmaf(qv[d], __half2float(kp[d]), dot);
        const float s = warp_sum(dot) * scale;
        const float new_max = fmaxf(run_max, s);
        const float factor = expf(run_max - new_max);
        const float p = expf(s - new_max);
        total = total * factor + p;
        const __half* vp = cache_v + (phys * kv_heads + kvh) * HD + lane * DIMS_PER_LANE;
#pragma unroll
        for (int d = 0; d < DIMS_PER_LANE; ++d) acc[d] = fmaf(p, __half2float(vp[d]), acc[d] * factor);
        run_max = new_max;
    }
    float* op = out + ((long long)t * q_heads + qh) * HD + lane * DIMS_PER_LANE;
    const float inv_total = 1.0f / total;
#pragma unroll
    for (int d = 0; d < DIMS_PER_LANE; ++d) op[d] = acc[d] * inv_total;
}

// ---------------------------------------------------------------------------
// Seeded synthetic checkpoint: N(0, stddev) values from a counter hash,
// quantised per block with a plain min/max (K-quants) or abs-max (Q8_0) rule.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t index, float stddev) {
    const uint64_t h = splitmix64(seed ^ splitmix64(index));
    const float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = (float)(uint32_t)((h >> 8) & 0xffffffu) * (1.0f / 16777216.0f);
    return stddev * sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
}

__device__ __forceinline__ void store_f16(unsigned char* p, float v, float* rounded) {
    // Every f16 field of the three block formats sits at an even offset of an even-sized block.
    const __half h = __float2half_rn(v);
    *reinterpret_cast<unsigned short*>(p) = __half_as_ushort(h);
    *rounded = __half2float(h);
}

__global__ void synth_quantized_kernel(int type, unsigned char* out, long long blocks, uint64_t seed,
                                       float stddev) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const int elems = block_elems(type);
    float v[256];
    for (int i = 0; i < elems; ++i) v[i] = normal_at(seed, (uint64_t)b * 256u + (uint64_t)i, stddev);
    unsigned char* blk = out + b * block_bytes(type);
    if (type == kQ8_0) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        float d;
        store_f16(blk, amax / 127.0f, &d);
        const float inv = d > 0.0f ? 1.0f / d : 0.0f;
        for (int i = 0; i < 32; ++i) {
            const int q = max(-127, min(127, __float2int_rn(v[i] * inv)));
            blk[2 + i] = (unsigned char)(signed char)q;
        }
    } else if (type == kQ4_K) {
        float scale[8], minimum[8], max_scale = 0.0f, max_min = 0.0f;
        for (int g = 0; g < 8; ++g) {
            float lo = 0.0f, hi = 0.0f;
            for (int i = 0; i < 32; ++i) { lo = fminf(lo, v[g * 32 + i]); hi = fmaxf(hi, v[g * 32 + i]); }
            scale[g] = (hi - lo) / 15.0f;
            minimum[g] = -lo;
            max_scale = fmaxf(max_scale, scale[g]);
            max_min = fmaxf(max_min, minimum[g]);
        }
        float d, dmin;
        store_f16(blk, max_scale / 63.0f, &d);
        store_f16(blk + 2, max_min / 63.0f, &dmin);
        int sc[8], mn[8];
        for (int g = 0; g < 8; ++g) {
            sc[g] = d > 0.0f ? max(0, min(63, __float2int_rn(scale[g] / d))) : 0;
            mn[g] = dmin > 0.0f ? max(0, min(63, __float2int_rn(minimum[g] / dmin))) : 0;
        }
        for (int i = 0; i < 4; ++i) {
            blk[4 + i] = (unsigned char)(sc[i] | ((sc[i + 4] >> 4) << 6));
            blk[8 + i] = (unsigned char)(mn[i] | ((mn[i + 4] >> 4) << 6));
            blk[12 + i] = (unsigned char)((sc[i + 4] & 0x0f) | ((mn[i + 4] & 0x0f) << 4));
        }
        for (int i = 0; i < 128; ++i) blk[16 + i] = 0;
        for (int g = 0; g < 8; ++g) {
            const float gs = d * (float)sc[g], gm = dmin * (float)mn[g];
            const float inv = gs > 0.0f ? 1.0f / gs : 0.0f;
            for (int i = 0; i < 32; ++i) {
                const int q = max(0, min(15, __float2int_rn((v[g * 32 + i] + gm) * inv)));
                blk[16 + (g >> 1) * 32 + i] |= (unsigned char)(q << ((g & 1) * 4));
            }
        }
    } else if (type == kQ6_K) {
        float scale[16], max_scale = 0.0f;
        for (int s = 0; s < 16; ++s) {
            float amax = 0.0f;
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[s * 16 + i]));
            scale[s] = amax / 31.0f;
            max_scale = fmaxf(max_scale, scale[s]);
        }
        float d;
        store_f16(blk + 208, max_scale / 127.0f, &d);
        for (int i = 0; i < 192; ++i) blk[i] = 0;
        for (int s = 0; s < 16; ++s) {
            const int sc = d > 0.0f ? max(1, min(127, __float2int_rn(scale[s] / d))) : 0;
            blk[192 + s] = (unsigned char)(signed char)sc;
            const float gs = d * (float)sc;
            const float inv = gs > 0.0f ? 1.0f / gs : 0.0f;
            for (int i = 0; i < 16; ++i) {
                const int e = s * 16 + i;
                const int q = max(-32, min(31, __float2int_rn(v[e] * inv))) + 32;
                const int g = e >> 5, l = e & 31, chunk = g >> 2, variant = g & 3;
                blk[chunk * 64 + (variant & 1) * 32 + l] |= (unsigned char)((q & 0x0f) << (variant < 2 ? 0 : 4));
                blk[128 + chunk * 32 + l] |= (unsigned char)((q >> 4) << (variant * 2));
            }
        }
    }
}

__global__ void synth_kv_kernel(__half* cache_k, __half* cache_v, long long layer_stride, int layers,
                                const int32_t* page_table, int tokens, int row_elems, uint64_t seed) {
    const long long per_layer = (long long)tokens * row_elems;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per_layer * layers) return;
    const int layer = (int)(i / per_layer);
    const long long r = i - (long long)layer * per_layer;
    const int t = (int)(r / row_elems), e = (int)(r - (long long)t * row_elems);
    const long long phys = (long long)page_table[t / kPageTokens] * kPageTokens + t % kPageTokens;
    const long long dst = (long long)layer * layer_stride + phys * row_elems + e;
    cache_k[dst] = __float2half_rn(normal_at(seed, (uint64_t)i * 2u, 1.0f));
    cache_v[dst] = __float2half_rn(normal_at(seed, (uint64_t)i * 2u + 1u, 1.0f));
}

__global__ void synth_f16_kernel(__half* out, long long n, uint64_t seed, float stddev) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(normal_at(seed, (uint64_t)i, stddev));
}

inline unsigned int grid_for(long long n, int block) { return (unsigned int)((n + block - 1) / block); }

}  // namespace

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
cudaError_t launch_step_metadata(cudaStream_t stream, const RowDesc* rows, int n_rows, int n_tokens,
                                 const uint32_t* prompt_tokens, const uint32_t* next_token,
                                 const int32_t* page_tables, int pages_per_sequence, StepMeta meta) {
    if (n_rows > 1024) return cudaErrorInvalidValue;
    step_metadata_kernel<<<1, 1024, (n_rows + 1) * sizeof(int32_t), stream>>>(
        rows, n_rows, n_tokens, prompt_tokens, next_token, page_tables, pages_per_sequence, meta);
    return cudaGetLastError();
}

cudaError_t launch_batch_metadata(cudaStream_t stream, const int32_t* row_slot, const int32_t* row_prefix,
                                  const int32_t* row_tokens, int n_rows, int n_tokens,
                                  const int32_t* page_tables, int pages_per_sequence, int page_tokens,
                                  int32_t* cu_seqlens, int32_t* token_row, int32_t* token_pos,
                                  int32_t* token_slot) {
    if (n_rows > 8192) return cudaErrorInvalidValue;
    batch_metadata_kernel<<<1, 1024, (n_rows + 1) * sizeof(int32_t), stream>>>(
        row_slot, row_prefix, row_tokens, n_rows, n_tokens, page_tables, pages_per_sequence, page_tokens,
        cu_seqlens, token_row, token_pos, token_slot);
    return cudaGetLastError();
}

cudaError_t launch_synth_kv(cudaStream_t stream, __half* cache_k, __half* cache_v, long long layer_stride,
                            int layers, const int32_t* page_table, int tokens, int row_elems, uint64_t seed) {
    const long long n = (long long)tokens * row_elems * layers;
    if (n <= 0) return cudaSuccess;
    synth_kv_kernel<<<grid_for(n, 256), 256, 0, stream>>>(cache_k, cache_v, layer_stride, layers, page_table,
                                                         tokens, row_elems, seed);
    return cudaGetLastError();
}

cudaError_t launch_gather_kv(cudaStream_t stream, const __half* cache, const int32_t* page_table, int tokens,
                             int row_elems, __half* out) {
    const long long n = (long long)tokens * row_elems;
    if (n <= 0) return cudaSuccess;
    gather_kv_kernel<<<grid_for(n, 256), 256, 0, stream>>>(cache, page_table, tokens, row_elems, out);
    return cudaGetLastError();
}

cudaError_t launch_embedding(cudaStream_t stream, int type, const unsigned char* table, int hidden,
                             int vocab, const uint32_t* token_id, int n_tokens, float* out) {
    const long long n = (long long)n_tokens * hidden;
    if (n <= 0) return cudaSuccess;
    embedding_kernel<<<grid_for(n, 256), 256, 0, stream>>>(type, table, hidden, vocab, token_id, n_tokens, out);
    return cudaGetLastError();
}

cudaError_t launch_dequantize(cudaStream_t stream, int type, const unsigned char* bytes, long long rows,
                              long long cols, float* out) {
    if (rows * cols <= 0) return cudaSuccess;
    dequantize_kernel<<<grid_for(rows * cols, 256), 256, 0, stream>>>(type, bytes, rows, cols, out);
    return cudaGetLastError();
}

cudaError_t launch_rms_norm(cudaStream_t stream, const float* x, const float* weight, int members,
                            int length, float eps, float* out) {
    return launch_rms_norm_gather(stream, x, nullptr, weight, members, length, eps, out);
}

cudaError_t launch_rms_norm_gather(cudaStream_t stream, const float* x, const int32_t* index,
                                   const float* weight, int members, int length, float eps, float* out) {
    if (members <= 0) return cudaSuccess;
    rms_norm_kernel<<<members, 256, 0, stream>>>(x, index, weight, length, eps, out);
    return cudaGetLastError();
}

cudaError_t launch_gemv_ref(cudaStream_t stream, int type, const unsigned char* w, long long n, long long k,
                            const float* x, int members, float* y, bool accumulate) {
    if (members <= 0 || n <= 0) return cudaSuccess;
    dim3 grid(grid_for(n, 4), (members + kRefMembers - 1) / kRefMembers);
    gemv_ref_kernel<<<grid, 128, 0, stream>>>(type, w, n, k, x, members, y, accumulate ? 1 : 0);
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(cudaStream_t stream, const float* gate, const float* up, long long length,
                            float* out) {
    if (length <= 0) return cudaSuccess;
    silu_mul_kernel<<<grid_for(length, 256), 256, 0, stream>>>(gate, up, length, out);
    return cudaGetLastError();
}

cudaError_t launch_residual_add(cudaStream_t stream, float* acc, const float* inc, long long length) {
    if (length <= 0) return cudaSuccess;
    residual_add_kernel<<<grid_for(length, 256), 256, 0, stream>>>(acc, inc, length);
    return cudaGetLastError();
}

cudaError_t launch_argmax(cudaStream_t stream, const float* logits, int members, long long length,
                          uint32_t* out, const int32_t* slot, uint32_t* next_token) {
    if (members <= 0) return cudaSuccess;
    if (members <= 32) argmax_kernel<8><<<members * 8, 1024, 0, stream>>>(logits, length, out, slot, next_token);
    else if (members <= 128) argmax_kernel<2><<<members * 2, 1024, 0, stream>>>(logits, length, out, slot, next_token);
    else argmax_kernel<1><<<members, 1024, 0, stream>>>(logits, length, out, slot, next_token);
    return cudaGetLastError();
}

cudaError_t launch_f32_to_f16(cudaStream_t stream, const float* in, long long length, uint16_t* out) {
    if (length <= 0) return cudaSuccess;
    f32_to_f16_kernel<<<grid_for(length, 256), 256, 0, stream>>>(in, length, out);
    return cudaGetLastError();
}

cudaError_t launch_rope_neox(cudaStream_t stream, float* values, const long long* positions, int members,
                             int heads, int head_dim, int rot_dims, const float* inv_freq) {
    const long long n = (long long)members * heads * (rot_dims / 2);
    if (n <= 0) return cudaSuccess;
    rope_neox_kernel<<<grid_for(n, 64), 64, 0, stream>>>(values, positions, members, heads, head_dim,
                                                        rot_dims / 2, inv_freq);
    return cudaGetLastError();
}

cudaError_t launch_qk_norm_rope_append(cudaStream_t stream, float* q, float* k, const float* v,
                                       const float* q_norm, const float* k_norm, const float* inv_freq,
                                       const int32_t* token_pos, const int32_t* token_slot, int n_tokens,
                                       int q_heads, int kv_heads, int head_dim, float eps,
                                       __half* cache_k, __half* cache_v) {
    const long long warps = (long long)n_tokens * (q_heads + kv_heads);
    if (warps <= 0) return cudaSuccess;
    qk_norm_rope_append_kernel<<<grid_for(warps, 4), 128, 0, stream>>>(
        q, k, v, q_norm, k_norm, inv_freq, token_pos, token_slot, n_tokens, q_heads, kv_heads, head_dim,
        eps, cache_k, cache_v);
    return cudaGetLastError();
}

cudaError_t launch_attention_ref(cudaStream_t stream, const float* q, const __half* cache_k,
                                 const __half* cache_v, const int32_t* page_tables, int pages_per_sequence,
                                 const int32_t* token_seq, const int32_t* token_pos, int n_tokens,
                                 int q_heads, int kv_heads, int head_dim, int window, float* out) {
    const long long warps = (long long)n_tokens * q_heads;
    if (warps <= 0) return cudaSuccess;
    const unsigned int grid = grid_for(warps, 4);
#define RIBN_ATTN_REF(D)                                                                           \
    attention_ref_kernel<D><<<grid, 128, 0, stream>>>(q, cache_k, cache_v, page_tables,            \
                                                      pages_per_sequence, token_seq, token_pos, \
                                                      n_tokens, q_heads, kv_heads, window, out)
    switch (head_dim) {
        case 32: RIBN_ATTN_REF(1); break;
        case 64: RIBN_ATTN_REF(2); break;
        case 128: RIBN_ATTN_REF(4); break;
        case 256: RIBN_ATTN_REF(8); break;
        default: return cudaErrorInvalidValue;
    }
#undef RIBN_ATTN_REF
    return cudaGetLastError();
}

cudaError_t launch_fill_f32(cudaStream_t stream, float* out, long long n, float value) {
    if (n <= 0) return cudaSuccess;
    fill_f32_kernel<<<grid_for(n, 256), 256, 0, stream>>>(out, n, value);
    return cudaGetLastError();
}

cudaError_t launch_synth_quantized(cudaStream_t stream, int type, unsigned char* out, long long rows,
                                   long long cols, uint64_t seed, float stddev) {
    const long long blocks = rows * (cols / block_elems(type));
    if (blocks <= 0) return cudaSuccess;
    synth_quantized_kernel<<<grid_for(blocks, 128), 128, 0, stream>>>(type, out, blocks, seed, stddev);
    return cudaGetLastError();
}

cudaError_t launch_synth_f16(cudaStream_t stream, __half* out, long long n, uint64_t seed, float stddev) {
    if (n <= 0) return cudaSuccess;
    synth_f16_kernel<<<grid_for(n, 256), 256, 0, stream>>>(out, n, seed, stddev);
    return cudaGetLastError();
}

}  // namespace ribn
