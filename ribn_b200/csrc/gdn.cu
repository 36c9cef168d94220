// Decode step of a Gated-DeltaNet recurrent layer (the Qwen3.5 hybrid model's linear-attention layers)
// behind the projections, and the sigmoid output gate of its gated full-attention layers.
//
// What the reference computes per token (crates/nvidia/src/qwen_reference.rs:202-278, its device kernels
// crates/nvidia/src/model_ops.rs:372-394, 614-820, 983-1040): beta = sigmoid(W_beta x), decay =
// exp(softplus(W_alpha x + dt_bias) * a); a causal depth-4 convolution + SiLU over the q | k | v
// channels with a three-deep history per channel; q and k heads l2-normalised and tiled across the
// value heads (value head h uses key head h % k_heads); per value head the state update
//   S *= decay,  sk = S^T k,  d = (v - sk) beta,  S += k (x) d,  o = S^T q / sqrt(head_dim)
// and the gated norm  rms(o) * norm_weight * silu(z).
//
// Here that is two launches per layer and step:
//   gdn_prepare_kernel   gates of every value head and convolution + SiLU + history shift of every channel;
//   gdn_state_kernel     one CTA per (member, value head): the head's 64 KB state passes through registers
//                        once (read, decay, both matrix-vector products, rank-one update, write), with the
//                        l2 norms in front and the gated norm behind it in the same CTA.
// The state's columns are independent, so a warp owns 16 rows x all columns and lanes walk columns:
// every global access is a full 128-byte row segment.  Sums over rows are per-warp partial sums folded in
// warp order (fixed order: results do not depend on the batch).
#include <math.h>

#include "kernels.cuh"

namespace ribn {

namespace {

constexpr int kGdnConvTaps = 4;

__device__ __forceinline__ float gdn_softplus(float v) { return v > 20.0f ? v : logf(1.0f + expf(v)); }
__device__ __forceinline__ float gdn_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gdn_silu(float v) { return v / (1.0f + expf(-v)); }

__global__ void gdn_prepare_kernel(const GdnStep g) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y;
    if (id < g.v_heads) {
        for (int t = 0; t < g.tokens; ++t) {
            const long long at = ((long long)m * g.tokens + t) * g.v_heads + id;
            g.beta[at] = gdn_sigmoid(g.beta_raw[at]);
            g.decay[at] = expf(gdn_softplus(g.alpha_raw[at] + g.dt_bias[id]) * g.a[id]);
        }
    }
    if (id < g.channels) {
        // history is oldest first; the tap weights of channel c sit at c * 4 + tap; the member's tokens in order
        float* h = g.conv_state[m] + id * (kGdnConvTaps - 1);
        const float* w = g.conv_weight + id * kGdnConvTaps;
        const float w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3];
        float h0 = h[0], h1 = h[1], h2 = h[2];
        for (int t = 0; t < g.tokens; ++t) {
            const long long row = (long long)m * g.tokens + t;
            const float x = g.qkv[row * g.channels + id];
            float sum = h0 * w0;
            sum += h1 * w1;
            sum += h2 * w2;
            sum += x * w3;
            h0 = h1; h1 = h2; h2 = x;
            g.conv_act[row * g.channels + id] = gdn_silu(sum);
        }
        h[0] = h0; h[1] = h1; h[2] = h2;
    }
}

// 256 threads: warp w owns rows [HD / 8 * w, HD / 8 * (w + 1)), lane l owns columns l, l + 32, ...
template <int HD>
__global__ void __launch_bounds__(256) gdn_state_kernel(const GdnStep g) {
    constexpr int kWarps = 8, kRows = HD / kWarps, kCols = HD / 32;
    __shared__ float q_s[HD], k_s[HD], fold[kWarps][HD], vec[HD];
    __shared__ float red[kWarps];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = blockIdx.y, vh = blockIdx.x, kh = vh % g.k_heads;
    float* state = g.state[m] + (long long)vh * HD * HD;
    // The head's state stays in registers for all the member's tokens: read once, written once.
    float s[kRows][kCols];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
#pragma unroll
        for (int c = 0; c < kCols; ++c) s[r][c] = state[(warp * kRows + r) * HD + lane + 32 * c];
    }
    for (int t = 0; t < g.tokens; ++t) {
        const long long token = (long long)m * g.tokens + t;
        const float* act = g.conv_act + token * g.channels;
        // l2-normalised q and k of the key head this value head is tiled from: 1 / max(|x|, eps)
        if (warp < 2) {
            const float* src = act + (warp == 0 ? 0 : g.k_offset) + kh * HD;
            float x[kCols], ss = 0.0f;
#pragma unroll
            for (int i = 0; i < kCols; ++i) { x[i] = src[lane + 32 * i]; ss = fmaf(x[i], x[i], ss); }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float scale = 1.0f / fmaxf(sqrtf(ss), g.l2_eps);
            float* dst = warp == 0 ? q_s : k_s;
#pragma unroll
            for (int i = 0; i < kCols; ++i) dst[lane + 32 * i] = x[i] * scale;
        }
        __syncthreads();
        const float decay = g.decay[token * g.v_heads + vh], beta = g.beta[token * g.v_heads + vh];
        float part[kCols];
#pragma unroll
        for (int c = 0; c < kCols; ++c) part[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const float kr = k_s[warp * kRows + r];
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                s[r][c] *= decay;
                part[c] = fmaf(s[r][c], kr, part[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < kCols; ++c) fold[warp][lane + 32 * c] = part[c];
        __syncthreads();
        if (threadIdx.x < HD) {
            float sk = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sk += fold[w][threadIdx.x];
            vec[threadIdx.x] = (act[g.v_offset + vh * HD + threadIdx.x] - sk) * beta;   // d
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < kCols; ++c) part[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const float kr = k_s[warp * kRows + r], qr = q_s[warp * kRows + r];
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                s[r][c] = fmaf(kr, vec[lane + 32 * c], s[r][c]);
                part[c] = fmaf(s[r][c], qr, part[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < kCols; ++c) fold[warp][lane + 32 * c] = part[c];
        __syncthreads();
        // o, its mean square, then rms(o) * norm_weight * silu(z)
        float o = 0.0f;
        if (threadIdx.x < HD) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) o += fold[w][threadIdx.x];
            o *= 1.0f / sqrtf((float)HD);
            if (g.attn_out != nullptr) g.attn_out[(token * g.v_heads + vh) * HD + threadIdx.x] = o;
        }
        float ss = threadIdx.x < HD ? o * o : 0.0f;
#pragma unroll
        for (int x = 16; x > 0; x >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, x);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (threadIdx.x < HD) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) total += red[w];
            const float inv = 1.0f / sqrtf(total / (float)HD + g.norm_eps);
            const long long at = (token * g.v_heads + vh) * HD + threadIdx.x;
            g.out[at] = o * inv * g.norm_weight[threadIdx.x] * gdn_silu(g.z[at]);
        }
        // the next token's first barrier orders these reads of q_s, k_s, fold and red before they are rewritten
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
#pragma unroll
        for (int c = 0; c < kCols; ++c) state[(warp * kRows + r) * HD + lane + 32 * c] = s[r][c];
    }
}

// Gated full attention: the q projection carries [q | gate] per head; out = attention * sigmoid(gate).
__global__ void attention_gate_kernel(const float* attn, const float* q_gate, long long rows, int heads, int head_dim, float* out) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long width = (long long)heads * head_dim;
    if (id >= rows * width) return;
    const long long row = id / width;
    const int head = (int)((id % width) / head_dim), d = (int)(id % head_dim);
    const float gate = q_gate[(row * heads + head) * 2 * head_dim + head_dim + d];
    out[id] = attn[id] * gdn_sigmoid(gate);
}

}  // namespace

cudaError_t launch_gdn_step(cudaStream_t stream, const GdnStep& g) {
    if (g.members <= 0 || g.tokens <= 0 || g.v_heads <= 0 || g.k_heads <= 0 || g.v_heads % g.k_heads != 0) return cudaErrorInvalidValue;
    if (g.head_dim != 64 && g.head_dim != 128) return cudaErrorInvalidValue;
    if (g.channels < g.v_offset + g.v_heads * g.head_dim || g.k_offset + g.k_heads * g.head_dim > g.channels) return cudaErrorInvalidValue;
    const int widest = g.channels > g.v_heads ? g.channels : g.v_heads;
    gdn_prepare_kernel<<<dim3((unsigned)((widest + 255) / 256), (unsigned)g.members), 256, 0, stream>>>(g);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const dim3 grid((unsigned)g.v_heads, (unsigned)g.members);
    if (g.head_dim == 128) gdn_state_kernel<128><<<grid, 256, 0, stream>>>(g);
    else gdn_state_kernel<64><<<grid, 256, 0, stream>>>(g);
    return cudaGetLastError();
}

cudaError_t launch_attention_gate(cudaStream_t stream, const float* attn, const float* q_gate, long long rows, int heads,
                                  int head_dim, float* out) {
    if (rows <= 0 || heads <= 0 || head_dim <= 0) return cudaErrorInvalidValue;
    const long long n = rows * heads * head_dim;
    attention_gate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(attn, q_gate, rows, heads, head_dim, out);
    return cudaGetLastError();
}

}  // namespace ribn
