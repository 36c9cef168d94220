/*
 * CPU oracle for one decode step of a Gated-DeltaNet recurrent layer behind its projections, and for the
 * sigmoid output gate of the gated full-attention layers.  TEST INFRASTRUCTURE ONLY: nothing in the shipped
 * library links, imports or executes it.
 *
 * A plain-C restatement of the reference's host equations, same operations in the same order:
 *   softplus, sigmoid gates           crates/nvidia/src/qwen_reference.rs:51-58, 213-223
 *   convolution + SiLU, history shift crates/nvidia/src/qwen_reference.rs:112-141
 *   l2 normalisation of q / k heads   crates/nvidia/src/qwen_reference.rs:42-48, 227-246
 *   state step of one value head      crates/nvidia/src/qwen_reference.rs:70-105
 *   gated norm                        crates/nvidia/src/qwen_reference.rs:259-271
 *   attention output gate             crates/nvidia/src/qwen_reference.rs:386-392, 462-472
 * The reference's device tests hold its kernels to these equations (crates/nvidia/tests/cuda_reference.rs:
 * 1002-1056 scalar gates 1e-5, 2144-2201 convolution 1e-4, 2203-2270 head norms 1e-4, 2282-2395 state update
 * 1e-2); tests/test_gdn_oracle.py replays those fixtures here against an independent float64 evaluation.
 * The reference's end-to-end check of this layer needs its 27B checkpoint (llama.cpp captures of real
 * weights), which is not available: whole-layer parity is unpinned beyond these equations.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#define ORC_API __attribute__((visibility("default")))

static float softplus_f(float v) { return v > 20.0f ? v : logf(1.0f + expf(v)); }

/* decay[h] = exp(softplus(alpha[h] + dt_bias[h]) * a[h]);  beta[h] = sigmoid(beta_raw[h]) */
ORC_API void orc_gdn_scalar_gate(const float* alpha, const float* beta_raw, const float* dt_bias, const float* a, int heads,
                                 float* decay, float* beta) {
    for (int h = 0; h < heads; ++h) {
        decay[h] = expf(softplus_f(alpha[h] + dt_bias[h]) * a[h]);
        beta[h] = 1.0f / (1.0f + expf(-beta_raw[h]));
    }
}

/* Depth-4 causal convolution over [history | new] per channel, then SiLU; history advances in place. */
ORC_API void orc_gdn_conv_silu(const float* input, const float* weight, float* history, int channels, float* raw, float* act) {
    for (int c = 0; c < channels; ++c) {
        float sum = 0.0f;
        for (int tap = 0; tap < 4; ++tap) {
            const float x = tap < 3 ? history[c * 3 + tap] : input[c];
            sum += x * weight[tap + c * 4];
        }
        history[c * 3] = history[c * 3 + 1];
        history[c * 3 + 1] = history[c * 3 + 2];
        history[c * 3 + 2] = input[c];
        if (raw) raw[c] = sum;
        act[c] = sum / (1.0f + expf(-sum));
    }
}

/* values[h][:] *= 1 / max(sqrt(sum of squares), eps) */
ORC_API void orc_l2_norm_heads(float* values, int heads, int head_dim, float eps) {
    for (int h = 0; h < heads; ++h) {
        float* x = values + (size_t)h * head_dim;
        float sum = 0.0f;
        for (int i = 0; i < head_dim; ++i) sum += x[i] * x[i];
        const float scale = 1.0f / fmaxf(sqrtf(sum), eps);
        for (int i = 0; i < head_dim; ++i) x[i] *= scale;
    }
}

/* Every value head: S *= decay; sk = S^T k; d = (v - sk) beta; S += k (x) d; o = S^T q / sqrt(head_dim).
 * q and k are [k_heads][head_dim] (value head h reads key head h % k_heads); v = conv[v_offset + h * head_dim ...]. */
ORC_API void orc_gdn_state_update(float* matrix, const float* q, const float* k, const float* conv, const float* decay,
                                  const float* beta, int v_heads, int k_heads, int head_dim, int v_offset, float* out) {
    float* sk = (float*)malloc(sizeof(float) * (size_t)head_dim * 2);
    float* d = sk + head_dim;
    const float scale = 1.0f / sqrtf((float)head_dim);
    for (int h = 0; h < v_heads; ++h) {
        float* s = matrix + (size_t)h * head_dim * head_dim;
        const float* qh = q + (size_t)(h % k_heads) * head_dim;
        const float* kh = k + (size_t)(h % k_heads) * head_dim;
        const float* v = conv + v_offset + (size_t)h * head_dim;
        for (int i = 0; i < head_dim * head_dim; ++i) s[i] *= decay[h];
        for (int col = 0; col < head_dim; ++col) sk[col] = 0.0f;
        for (int row = 0; row < head_dim; ++row) {
            for (int col = 0; col < head_dim; ++col) sk[col] += s[row * head_dim + col] * kh[row];
        }
        for (int col = 0; col < head_dim; ++col) d[col] = (v[col] - sk[col]) * beta[h];
        for (int row = 0; row < head_dim; ++row) {
            for (int col = 0; col < head_dim; ++col) s[row * head_dim + col] += kh[row] * d[col];
        }
        for (int col = 0; col < head_dim; ++col) {
            float sum = 0.0f;
            for (int row = 0; row < head_dim; ++row) sum += s[row * head_dim + col] * qh[row];
            out[(size_t)h * head_dim + col] = sum * scale;
        }
    }
    free(sk);
}

/* out[h][i] = o[h][i] * (mean square of o[h] + eps)^-1/2 * norm[i] * silu(z[h][i]) */
ORC_API void orc_gdn_gated_norm(const float* o, const float* z, const float* norm, int heads, int head_dim, float eps, float* out) {
    for (int h = 0; h < heads; ++h) {
        const float* x = o + (size_t)h * head_dim;
        float sum = 0.0f;
        for (int i = 0; i < head_dim; ++i) sum += x[i] * x[i];
        const float inv = 1.0f / sqrtf(sum / (float)head_dim + eps);
        for (int i = 0; i < head_dim; ++i) {
            const float zv = z[(size_t)h * head_dim + i];
            const float silu = zv / (1.0f + expf(-zv));
            out[(size_t)h * head_dim + i] = x[i] * inv * norm[i] * silu;
        }
    }
}

/* The whole step behind the projections for one sequence; conv_act, attn_out may be NULL. */
ORC_API void orc_gdn_step(int k_heads, int v_heads, int head_dim, const float* qkv, const float* z, const float* beta_raw,
                          const float* alpha_raw, const float* dt_bias, const float* a, const float* conv_weight,
                          const float* norm_weight, float* conv_state, float* matrix, float l2_eps, float norm_eps,
                          float* decay, float* beta, float* conv_act, float* attn_out, float* out) {
    const int channels = (2 * k_heads + v_heads) * head_dim, k_offset = k_heads * head_dim, v_offset = 2 * k_heads * head_dim;
    float* act = conv_act ? conv_act : (float*)malloc(sizeof(float) * (size_t)channels);
    float* o = attn_out ? attn_out : (float*)malloc(sizeof(float) * (size_t)v_heads * head_dim);
    float* qk = (float*)malloc(sizeof(float) * (size_t)2 * k_heads * head_dim);
    orc_gdn_scalar_gate(alpha_raw, beta_raw, dt_bias, a, v_heads, decay, beta);
    orc_gdn_conv_silu(qkv, conv_weight, conv_state, channels, NULL, act);
    for (int i = 0; i < k_heads * head_dim; ++i) { qk[i] = act[i]; qk[k_heads * head_dim + i] = act[k_offset + i]; }
    orc_l2_norm_heads(qk, 2 * k_heads, head_dim, l2_eps);
    orc_gdn_state_update(matrix, qk, qk + (size_t)k_heads * head_dim, act, decay, beta, v_heads, k_heads, head_dim, v_offset, o);
    orc_gdn_gated_norm(o, z, norm_weight, v_heads, head_dim, norm_eps, out);
    free(qk);
    if (!conv_act) free(act);
    if (!attn_out) free(o);
}

/* out[r][h][i] = attn[r][h][i] * sigmoid(q_gate[r][h][head_dim + i]) */
ORC_API void orc_attention_gate(const float* attn, const float* q_gate, int rows, int heads, int head_dim, float* out) {
    for (int r = 0; r < rows; ++r) {
        for (int h = 0; h < heads; ++h) {
            for (int i = 0; i < head_dim; ++i) {
                const float g = q_gate[((size_t)r * heads + h) * 2 * head_dim + head_dim + i];
                const size_t at = ((size_t)r * heads + h) * head_dim + i;
                out[at] = attn[at] * (1.0f / (1.0f + expf(-g)));
            }
        }
    }
}
