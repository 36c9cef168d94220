/*
 * CPU oracle for the dense-Qwen3 GGUF decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference's own host equations.
 * It is the checker for the CUDA kernels and the timed CPU baseline; nothing
 * in the shipped library links, imports or executes it.  The reference is a
 * Rust workspace that cannot be compiled where this repository is built (no
 * cargo/rustc), so every function below cites the reference file:line whose
 * arithmetic it follows, and the oracle is pinned against the reference's own
 * known-answer values (crates/gguf/src/lib.rs:1479-1565 and the fixture
 * generators of crates/nvidia/tests/cuda_reference.rs) by tests/test_oracle_*.py.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 * (no FMA contraction: the Q4_K dequant expression is three separately
 * rounded f32 operations in the reference host code).
 *
 * End-to-end token parity for dense Qwen3 shapes is "parity unpinned" by the
 * reference itself (its full-model gates need a 27B hybrid checkpoint that is
 * not available); the composed model below is pinned primitive by primitive.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

enum { GGML_F32 = 0, GGML_F16 = 1, GGML_Q8_0 = 8, GGML_Q4_K = 12, GGML_Q6_K = 14 };

/* ------------------------------------------------------------------------- */
/* scalar conversions                                                          */
/* ------------------------------------------------------------------------- */

/* binary16 -> binary32, exact for every finite value and infinities
 * (crates/gguf/src/lib.rs:539-551 computes the same value arithmetically;
 * NaN maps to a quiet NaN there and here). */
ORC_API float orc_f16_to_f32(uint16_t bits) {
    uint32_t sign = (uint32_t)(bits & 0x8000u) << 16;
    uint32_t exponent = (bits >> 10) & 0x1fu;
    uint32_t fraction = bits & 0x03ffu;
    uint32_t out;
    if (exponent == 0) {
        if (fraction == 0) {
            out = sign;
        } else {
            /* subnormal: fraction * 2^-24, normalise */
            int shift = 0;
            while ((fraction & 0x400u) == 0) { fraction <<= 1; ++shift; }
            fraction &= 0x3ffu;
            out = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (fraction << 13);
        }
    } else if (exponent == 0x1f) {
        out = sign | 0x7f800000u | (fraction ? 0x00400000u : 0u);
    } else {
        out = sign | ((exponent - 15 + 127) << 23) | (fraction << 13);
    }
    float value;
    memcpy(&value, &out, 4);
    return value;
}

/* binary32 -> binary16 round-to-nearest-even
 * (crates/nvidia/src/model_ops.rs:1213-1256, f32_to_f16_bits). */
ORC_API uint16_t orc_f32_to_f16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int exponent = (int)((bits >> 23) & 0xffu) - 127 + 15;
    uint32_t mantissa = bits & 0x7fffffu;
    if (((bits >> 23) & 0xffu) == 0xffu) {
        return (uint16_t)(sign | 0x7c00u | (mantissa ? 0x0200u : 0u));
    }
    if (exponent >= 31) {
        return (uint16_t)(sign | 0x7c00u);
    }
    if (exponent <= 0) {
        if (exponent < -10) {
            return (uint16_t)sign;
        }
        mantissa |= 0x800000u;
        int shift = 14 - exponent;
        uint32_t result = mantissa >> shift;
        uint32_t remainder = mantissa & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (remainder > halfway || (remainder == halfway && (result & 1u))) {
            result += 1u;
        }
        return (uint16_t)(sign | result);
    }
    uint32_t result = mantissa >> 13;
    uint32_t remainder = mantissa & 0x1fffu;
    if (remainder > 0x1000u || (remainder == 0x1000u && (result & 1u))) {
        result += 1u;
        if (result == 0x400u) {
            if (exponent + 1 >= 31) {
                return (uint16_t)(sign | 0x7c00u);
            }
            return (uint16_t)(sign | ((uint32_t)(exponent + 1) << 10));
        }
    }
    return (uint16_t)(sign | ((uint32_t)exponent << 10) | result);
}

/* ------------------------------------------------------------------------- */
/* GGUF block decoders                                                         */
/* ------------------------------------------------------------------------- */

/* (elements, bytes) per block: crates/gguf/src/lib.rs tensor_layout. */
ORC_API int orc_block_elems(int type) {
    switch (type) {
        case GGML_F32: case GGML_F16: return 1;
        case GGML_Q8_0: return 32;
        case GGML_Q4_K: case GGML_Q6_K: return 256;
        default: return 0;
    }
}

ORC_API int orc_block_bytes(int type) {
    switch (type) {
        case GGML_F32: return 4;
        case GGML_F16: return 2;
        case GGML_Q8_0: return 34;
        case GGML_Q4_K: return 144;
        case GGML_Q6_K: return 210;
        default: return 0;
    }
}

static float read_f16(const uint8_t* p) {
    return orc_f16_to_f32((uint16_t)(p[0] | ((uint16_t)p[1] << 8)));
}

/* crates/gguf/src/lib.rs:577-582 */
static void dequant_q8_0(const uint8_t* e, float* out) {
    float scale = read_f16(e);
    for (int i = 0; i < 32; ++i) {
        out[i] = scale * (float)(int8_t)e[2 + i];
    }
}

/* crates/gguf/src/lib.rs:561-575: 12 packed bytes -> 8 six-bit scales and
 * 8 six-bit minima. `p` points at byte 4 of the block. */
static void q4_k_scales(const uint8_t* p, uint8_t scales[8], uint8_t minima[8]) {
    for (int i = 0; i < 4; ++i) {
        scales[i] = p[i] & 0x3f;
        scales[i + 4] = (uint8_t)((p[8 + i] & 0x0f) | ((p[i] >> 2) & 0x30));
        minima[i] = p[4 + i] & 0x3f;
        minima[i + 4] = (uint8_t)((p[8 + i] >> 4) | ((p[4 + i] >> 2) & 0x30));
    }
}

/* crates/gguf/src/lib.rs:584-600.  group_scale and group_minimum are rounded
 * to f32 before the per-element multiply and subtract (three roundings). */
static void dequant_q4_k(const uint8_t* e, float* out) {
    float scale = read_f16(e);
    float minimum_scale = read_f16(e + 2);
    uint8_t scales[8], minima[8];
    q4_k_scales(e + 4, scales, minima);
    for (int group = 0; group < 8; ++group) {
        int data_offset = 16 + (group / 2) * 32;
        int shift = (group % 2) * 4;
        float group_scale = scale * (float)scales[group];
        float group_minimum = minimum_scale * (float)minima[group];
        for (int i = 0; i < 32; ++i) {
            int q = (e[data_offset + i] >> shift) & 0x0f;
            float product = group_scale * (float)q;
            out[group * 32 + i] = product - group_minimum;
        }
    }
}

/* crates/gguf/src/lib.rs:623-649 */
static void dequant_q6_k(const uint8_t* e, float* out) {
    const uint8_t* low_bits = e;
    const uint8_t* high_bits = e + 128;
    const uint8_t* scales = e + 192;
    float scale = read_f16(e + 208);
    int o = 0;
    for (int group = 0; group < 8; ++group) {
        int chunk = group / 4;
        int variant = group % 4;
        int low_offset = chunk * 64 + (variant % 2) * 32;
        int low_shift = variant < 2 ? 0 : 4;
        int high_offset = chunk * 32;
        int high_shift = variant * 2;
        for (int half = 0; half < 2; ++half) {
            float group_scale = scale * (float)(int8_t)scales[group * 2 + half];
            for (int i = 0; i < 16; ++i) {
                int position = half * 16 + i;
                int low = (low_bits[low_offset + position] >> low_shift) & 0x0f;
                int high = (high_bits[high_offset + position] >> high_shift) & 0x03;
                int q = (low | (high << 4)) - 32;
                out[o++] = group_scale * (float)q;
            }
        }
    }
}

/* crates/gguf/src/lib.rs:508-535 dequantize_block.
 * Returns 0, -1 for an unsupported type, -2 for a wrong encoded length. */
ORC_API int orc_dequantize_block(int type, const uint8_t* encoded, int64_t length, float* out) {
    int bytes = orc_block_bytes(type);
    if (bytes == 0) return -1;
    if (length != bytes) return -2;
    switch (type) {
        case GGML_F32: memcpy(out, encoded, 4); return 0;
        case GGML_F16: out[0] = read_f16(encoded); return 0;
        case GGML_Q8_0: dequant_q8_0(encoded, out); return 0;
        case GGML_Q4_K: dequant_q4_k(encoded, out); return 0;
        case GGML_Q6_K: dequant_q6_k(encoded, out); return 0;
    }
    return -1;
}

/* A row of `k` elements = k / block_elems consecutive encoded blocks
 * (crates/nvidia/src/quantized.rs:139-143). */
ORC_API int orc_dequantize_row(int type, const uint8_t* encoded, int64_t k, float* out) {
    int elems = orc_block_elems(type), bytes = orc_block_bytes(type);
    if (elems == 0 || k % elems != 0) return -1;
    for (int64_t b = 0; b < k / elems; ++b) {
        orc_dequantize_block(type, encoded + b * bytes, bytes, out + b * elems);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* primitives                                                                  */
/* ------------------------------------------------------------------------- */

static int g_threads = 1;

ORC_API void orc_set_threads(int threads) {
    g_threads = threads < 1 ? 1 : threads;
#ifdef _OPENMP
    omp_set_num_threads(g_threads);
#endif
}

ORC_API int orc_get_threads(void) { return g_threads; }

/* y[n] = sum_k deq(W[n,k]) * x[k], f32, summed sequentially over k
 * (crates/nvidia/src/qwen_reference.rs:31-40 gguf_gemv over
 * engine_gguf::dequantize_block output; the same expectation the reference's
 * device tests build at crates/nvidia/tests/cuda_reference.rs:725-738).
 * Rows are independent, so the OpenMP split over n does not change any bit. */
ORC_API int orc_gemv(int type, const uint8_t* w, int64_t k, int64_t n, const float* x, float* y) {
    int elems = orc_block_elems(type), bytes = orc_block_bytes(type);
    if (elems == 0 || k % elems != 0) return -1;
    int64_t blocks = k / elems;
    #pragma omp parallel for schedule(static) if (g_threads > 1)
    for (int64_t row = 0; row < n; ++row) {
        float tmp[256];
        float sum = 0.0f;
        const uint8_t* base = w + row * blocks * bytes;
        for (int64_t b = 0; b < blocks; ++b) {
            orc_dequantize_block(type, base + b * bytes, bytes, tmp);
            const float* xs = x + b * elems;
            for (int i = 0; i < elems; ++i) {
                sum += xs[i] * tmp[i];
            }
        }
        y[row] = sum;
    }
    return 0;
}

/* crates/nvidia/src/qwen_reference.rs:550-556 rms_norm_raw */
ORC_API void orc_rms_norm(const float* x, const float* w, int n, float eps, float* out) {
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += x[i] * x[i];
    float inv = 1.0f / sqrtf(sum / (float)n + eps);
    for (int i = 0; i < n; ++i) out[i] = x[i] * inv * w[i];
}

/* NeoX half-split rotary over the first `rot` dims of every head
 * (crates/nvidia/src/qwen_reference.rs:410-425; device twin
 * crates/nvidia/src/model_ops.rs:395-425). */
ORC_API void orc_rope_neox(float* v, int heads, int head_dim, int rot, float base, int64_t pos) {
    int half = rot / 2;
    for (int h = 0; h < heads; ++h) {
        float* p = v + (int64_t)h * head_dim;
        for (int pair = 0; pair < half; ++pair) {
            float theta = (float)pos * powf(base, -(2.0f * (float)pair) / (float)rot);
            float s = sinf(theta), c = cosf(theta);
            float x0 = p[pair], x1 = p[half + pair];
            p[pair] = x0 * c - x1 * s;
            p[half + pair] = x0 * s + x1 * c;
        }
    }
}

/* crates/nvidia/src/qwen_reference.rs:533-537 (host_ffn_step gating) */
ORC_API void orc_silu_mul(const float* g, const float* u, int n, float* out) {
    for (int i = 0; i < n; ++i) out[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
}

/* Greedy selection: strict '>' scan, NaN never wins, ties keep the lowest
 * index, all-NaN gives 0 (crates/nvidia/src/model_ops.rs:203-260). */
ORC_API uint32_t orc_argmax(const float* logits, int64_t n) {
    uint32_t best = 0;
    int have = 0;
    float best_value = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        float v = logits[i];
        if (v != v) continue;
        if (!have || v > best_value) {
            /* -inf maps to key 0x007fffff > 0 in the device kernel, so it can
             * win over "nothing"; an explicit flag gives the same answer. */
            have = 1;
            best_value = v;
            best = (uint32_t)i;
        }
    }
    return best;
}

/* GQA softmax attention for one query row over `tokens` cached keys.
 * keys/values: F16 bits, contiguous [token][kv_head][head_dim]
 * (crates/nvidia/src/qwen_reference.rs:431-461 without the sigmoid gate;
 * device twin crates/nvidia/src/model_ops.rs:441-545). */
ORC_API void orc_attention(const float* q, const uint16_t* keys, const uint16_t* values,
                           int tokens, int q_heads, int kv_heads, int head_dim, float* out) {
    int q_per_kv = q_heads / kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    #pragma omp parallel for schedule(static) if (g_threads > 1)
    for (int qh = 0; qh < q_heads; ++qh) {
        int kvh = qh / q_per_kv;
        const float* qv = q + (int64_t)qh * head_dim;
        float* scores = (float*)malloc(sizeof(float) * (size_t)tokens);
        for (int t = 0; t < tokens; ++t) {
            const uint16_t* key = keys + ((int64_t)t * kv_heads + kvh) * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += qv[d] * orc_f16_to_f32(key[d]);
            scores[t] = dot * scale;
        }
        float max = -INFINITY;
        for (int t = 0; t < tokens; ++t) max = fmaxf(max, scores[t]);
        float total = 0.0f;
        for (int t = 0; t < tokens; ++t) { scores[t] = expf(scores[t] - max); total += scores[t]; }
        float* o = out + (int64_t)qh * head_dim;
        for (int d = 0; d < head_dim; ++d) o[d] = 0.0f;
        for (int t = 0; t < tokens; ++t) {
            const uint16_t* value = values + ((int64_t)t * kv_heads + kvh) * head_dim;
            float weight = scores[t] / total;
            for (int d = 0; d < head_dim; ++d) o[d] += weight * orc_f16_to_f32(value[d]);
        }
        free(scores);
    }
}

/* ------------------------------------------------------------------------- */
/* dense Qwen3 decoder, one token at a time                                    */
/* ------------------------------------------------------------------------- */

typedef struct {
    int32_t layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab, context;
    float rope_base, eps;
} orc_qwen3_config;

typedef struct {
    int type;
    int64_t n, k;
    uint8_t* bytes;
    int owned;
} orc_tensor;

enum { T_ATTN_NORM, T_Q, T_K, T_V, T_Q_NORM, T_K_NORM, T_O, T_FFN_NORM, T_GATE, T_UP, T_DOWN, T_PER_LAYER };

typedef struct {
    orc_qwen3_config cfg;
    orc_tensor* layer; /* [layers][T_PER_LAYER] */
    orc_tensor token_embd, output_norm, output;
} orc_qwen3;

typedef struct {
    const orc_qwen3* model;
    int32_t position;
    uint16_t* keys;   /* [layer][token][kv_head][head_dim] */
    uint16_t* values;
} orc_qwen3_seq;

ORC_API orc_qwen3* orc_qwen3_create(const orc_qwen3_config* cfg) {
    orc_qwen3* m = (orc_qwen3*)calloc(1, sizeof(orc_qwen3));
    m->cfg = *cfg;
    m->layer = (orc_tensor*)calloc((size_t)cfg->layers * T_PER_LAYER, sizeof(orc_tensor));
    return m;
}

static void free_tensor(orc_tensor* t) {
    if (t->owned) free(t->bytes);
    memset(t, 0, sizeof(*t));
}

ORC_API void orc_qwen3_destroy(orc_qwen3* m) {
    if (!m) return;
    for (int i = 0; i < m->cfg.layers * T_PER_LAYER; ++i) free_tensor(&m->layer[i]);
    free_tensor(&m->token_embd); free_tensor(&m->output_norm); free_tensor(&m->output);
    free(m->layer);
    free(m);
}

static orc_tensor* find_tensor(orc_qwen3* m, const char* name) {
    if (!strcmp(name, "token_embd.weight")) return &m->token_embd;
    if (!strcmp(name, "output_norm.weight")) return &m->output_norm;
    if (!strcmp(name, "output.weight")) return &m->output;
    int layer = -1;
    char rest[64];
    if (sscanf(name, "blk.%d.%63s", &layer, rest) != 2 || layer < 0 || layer >= m->cfg.layers) return NULL;
    static const char* names[T_PER_LAYER] = {
        "attn_norm.weight", "attn_q.weight", "attn_k.weight", "attn_v.weight",
        "attn_q_norm.weight", "attn_k_norm.weight", "attn_output.weight",
        "ffn_norm.weight", "ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"};
    for (int i = 0; i < T_PER_LAYER; ++i) {
        if (!strcmp(rest, names[i])) return &m->layer[layer * T_PER_LAYER + i];
    }
    return NULL;
}

/* Tensor names follow GGUF (`blk.N.attn_q.weight`, ...).  A matrix is
 * [n = out rows][k = in, contiguous] encoded blocks; norms are F32 vectors
 * (n = 1).  `copy` = 0 borrows the caller's buffer. */
ORC_API int orc_qwen3_set_tensor(orc_qwen3* m, const char* name, int type, int64_t n, int64_t k,
                                 const uint8_t* bytes, int copy) {
    orc_tensor* t = find_tensor(m, name);
    int elems = orc_block_elems(type);
    if (!t || elems == 0 || k % elems != 0) return -1;
    free_tensor(t);
    size_t size = (size_t)n * (size_t)(k / elems) * (size_t)orc_block_bytes(type);
    t->type = type; t->n = n; t->k = k;
    if (copy) {
        t->bytes = (uint8_t*)malloc(size);
        memcpy(t->bytes, bytes, size);
        t->owned = 1;
    } else {
        t->bytes = (uint8_t*)bytes;
    }
    return 0;
}

ORC_API orc_qwen3_seq* orc_qwen3_seq_create(const orc_qwen3* m) {
    orc_qwen3_seq* s = (orc_qwen3_seq*)calloc(1, sizeof(orc_qwen3_seq));
    s->model = m;
    size_t per_layer = (size_t)m->cfg.context * m->cfg.kv_heads * m->cfg.head_dim;
    s->keys = (uint16_t*)calloc(per_layer * m->cfg.layers, 2);
    s->values = (uint16_t*)calloc(per_layer * m->cfg.layers, 2);
    return s;
}

ORC_API void orc_qwen3_seq_destroy(orc_qwen3_seq* s) {
    if (!s) return;
    free(s->keys); free(s->values); free(s);
}

ORC_API int orc_qwen3_seq_position(const orc_qwen3_seq* s) { return s->position; }

/* Preload a sequence's cache with synthetic F16 K/V for `tokens` positions so
 * a decode step at a long context can be timed without running the prefill.
 * keys/values: [layer][token][kv_head][head_dim]. */
ORC_API int orc_qwen3_seq_fill(orc_qwen3_seq* s, int tokens, const uint16_t* keys, const uint16_t* values) {
    const orc_qwen3_config* c = &s->model->cfg;
    if (tokens > c->context) return -1;
    size_t row = (size_t)c->kv_heads * c->head_dim;
    for (int l = 0; l < c->layers; ++l) {
        memcpy(s->keys + (size_t)l * c->context * row, keys + (size_t)l * tokens * row, tokens * row * 2);
        memcpy(s->values + (size_t)l * c->context * row, values + (size_t)l * tokens * row, tokens * row * 2);
    }
    s->position = tokens;
    return 0;
}

static const float* as_f32(const orc_tensor* t) { return (const float*)t->bytes; }

/* One token through the dense decoder at the sequence's current position.
 * Layer order: crates/nvidia/src/decode.rs:589-637 and 976-1106 with the
 * dense-Qwen3 substitutions (plain per-head Q/K RMSNorm instead of
 * q_gate_norm, rotary over the whole head, no sigmoid output gate, no
 * recurrent layers); head: decode.rs:686-704.  `logits` may be NULL for an
 * intermediate prefill token (no head pass).  `hidden_out` (optional) gets
 * the final residual stream before the output norm.  Returns 0, or -1 when
 * the context is full or a tensor is missing. */
ORC_API int orc_qwen3_step(orc_qwen3_seq* s, uint32_t token, float* logits, float* hidden_out) {
    const orc_qwen3* m = s->model;
    const orc_qwen3_config* c = &m->cfg;
    if (s->position >= c->context || token >= (uint32_t)c->vocab) return -1;
    int H = c->hidden, QD = c->q_heads * c->head_dim, KD = c->kv_heads * c->head_dim, F = c->ffn;
    float* hidden = (float*)malloc(sizeof(float) * H);
    float* normed = (float*)malloc(sizeof(float) * H);
    float* q = (float*)malloc(sizeof(float) * QD);
    float* k = (float*)malloc(sizeof(float) * KD);
    float* v = (float*)malloc(sizeof(float) * KD);
    float* attn = (float*)malloc(sizeof(float) * QD);
    float* proj = (float*)malloc(sizeof(float) * H);
    float* gate = (float*)malloc(sizeof(float) * F);
    float* up = (float*)malloc(sizeof(float) * F);
    float* tmp = (float*)malloc(sizeof(float) * (c->head_dim > 256 ? c->head_dim : 256));
    int rc = 0;

    /* embedding: dequantise row `token` of token_embd [vocab][hidden]
     * (crates/nvidia/src/kernels/quantized/q4_k.cu:1-28). */
    {
        const orc_tensor* e = &m->token_embd;
        if (!e->bytes) { rc = -1; goto done; }
        int64_t row_bytes = (e->k / orc_block_elems(e->type)) * orc_block_bytes(e->type);
        orc_dequantize_row(e->type, e->bytes + (int64_t)token * row_bytes, e->k, hidden);
    }
    int pos = s->position;
    size_t cache_row = (size_t)c->kv_heads * c->head_dim;
    for (int l = 0; l < c->layers; ++l) {
        const orc_tensor* t = &m->layer[l * T_PER_LAYER];
        for (int i = 0; i < T_PER_LAYER; ++i) if (!t[i].bytes) { rc = -1; goto done; }
        orc_rms_norm(hidden, as_f32(&t[T_ATTN_NORM]), H, c->eps, normed);
        orc_gemv(t[T_Q].type, t[T_Q].bytes, H, QD, normed, q);
        orc_gemv(t[T_K].type, t[T_K].bytes, H, KD, normed, k);
        orc_gemv(t[T_V].type, t[T_V].bytes, H, KD, normed, v);
        for (int h = 0; h < c->q_heads; ++h) {
            orc_rms_norm(q + h * c->head_dim, as_f32(&t[T_Q_NORM]), c->head_dim, c->eps, tmp);
            memcpy(q + h * c->head_dim, tmp, sizeof(float) * c->head_dim);
        }
        for (int h = 0; h < c->kv_heads; ++h) {
            orc_rms_norm(k + h * c->head_dim, as_f32(&t[T_K_NORM]), c->head_dim, c->eps, tmp);
            memcpy(k + h * c->head_dim, tmp, sizeof(float) * c->head_dim);
        }
        orc_rope_neox(q, c->q_heads, c->head_dim, c->head_dim, c->rope_base, pos);
        orc_rope_neox(k, c->kv_heads, c->head_dim, c->head_dim, c->rope_base, pos);
        uint16_t* lk = s->keys + (size_t)l * c->context * cache_row;
        uint16_t* lv = s->values + (size_t)l * c->context * cache_row;
        for (size_t i = 0; i < cache_row; ++i) {
            lk[(size_t)pos * cache_row + i] = orc_f32_to_f16(k[i]);
            lv[(size_t)pos * cache_row + i] = orc_f32_to_f16(v[i]);
        }
        orc_attention(q, lk, lv, pos + 1, c->q_heads, c->kv_heads, c->head_dim, attn);
        orc_gemv(t[T_O].type, t[T_O].bytes, QD, H, attn, proj);
        for (int i = 0; i < H; ++i) hidden[i] += proj[i];
        orc_rms_norm(hidden, as_f32(&t[T_FFN_NORM]), H, c->eps, normed);
        orc_gemv(t[T_GATE].type, t[T_GATE].bytes, H, F, normed, gate);
        orc_gemv(t[T_UP].type, t[T_UP].bytes, H, F, normed, up);
        orc_silu_mul(gate, up, F, gate);
        orc_gemv(t[T_DOWN].type, t[T_DOWN].bytes, F, H, gate, proj);
        for (int i = 0; i < H; ++i) hidden[i] += proj[i];
    }
    if (hidden_out) memcpy(hidden_out, hidden, sizeof(float) * H);
    if (logits) {
        if (!m->output_norm.bytes || !m->output.bytes) { rc = -1; goto done; }
        orc_rms_norm(hidden, as_f32(&m->output_norm), H, c->eps, normed);
        orc_gemv(m->output.type, m->output.bytes, H, c->vocab, normed, logits);
    }
    s->position = pos + 1;
done:
    free(hidden); free(normed); free(q); free(k); free(v); free(attn); free(proj);
    free(gate); free(up); free(tmp);
    return rc;
}

/* Read back one layer's cached K or V row (F16 bits) for parity checks. */
ORC_API const uint16_t* orc_qwen3_seq_cache(const orc_qwen3_seq* s, int layer, int which) {
    const orc_qwen3_config* c = &s->model->cfg;
    size_t per_layer = (size_t)c->context * c->kv_heads * c->head_dim;
    return (which ? s->values : s->keys) + (size_t)layer * per_layer;
}
