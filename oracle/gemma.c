/* CPU restatement of the reference's host Gemma-4 text decoder (BF16 storage, FP32 arithmetic, one BF16
 * rounding after every operation).  TEST INFRASTRUCTURE ONLY: the shipped library never links or calls
 * this file; tests, the smoke check and the bench's CPU-baseline leg use it as the checker.
 *
 * Each function names the reference source it follows (paths inside the reference project):
 *   crates/gemma4/src/cpu/linear.rs       bf16 (10-16), project (23-66)
 *   crates/gemma4/src/cpu/norm.rs         rms_norm / rms_norm_scale_free (12-82)
 *   crates/gemma4/src/cpu/rotary.rs       factors (33-93), apply_rotary (95-140)
 *   crates/gemma4/src/cpu/attention.rs    attention (26-277)
 *   crates/gemma4/src/cpu/elementwise.rs  add, multiply, scale, gelu_tanh, softcap, ple_combine
 *   crates/gemma4/src/cpu/decoder.rs      step / run_body / layer_forward / attention_forward /
 *                                         feedforward_forward / project_logits / argmax (133-626)
 *   crates/gemma4/src/config.rs           rotary_inverse_frequency (200-247), layer geometry (296-385)
 *
 * Pinned by the reference's own known answers (crates/gemma4/tests/cpu_ops.rs:21-135,
 * cpu_attention.rs:23-100, rotary.rs with tests/fixtures/rotary.json); no end-to-end Gemma vector
 * exists in the reference without its 14.9 GB checkpoint, so whole-model parity is "unpinned" and this
 * restatement is the end-to-end oracle.
 *
 * Build: -O2 -ffp-contract=off (no fused multiply-add, source-order accumulation).  OpenMP, when
 * present, splits independent output elements only, which changes no bit. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

static inline float gm_load(uint16_t bits) {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* linear.rs:10-16: round to nearest even, NaN -> 0x7fc0 */
ORC_API uint16_t orc_gm_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    return (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

ORC_API float orc_gm_bf16_to_f32(uint16_t bits) { return gm_load(bits); }

/* linear.rs:23-66: out[m][n] = bf16(sum_k in[m][k] * w[n][k]), FP32, source order */
ORC_API void orc_gm_project(const uint16_t* in, int rows, const uint16_t* w, int64_t n, int64_t k, uint16_t* out) {
    for (int r = 0; r < rows; ++r) {
        const uint16_t* x = in + (int64_t)r * k;
#pragma omp parallel for schedule(static)
        for (int64_t c = 0; c < n; ++c) {
            const uint16_t* row = w + c * k;
            float sum = 0.0f;
            for (int64_t i = 0; i < k; ++i) sum += gm_load(x[i]) * gm_load(row[i]);
            out[(int64_t)r * n + c] = orc_gm_bf16(sum);
        }
    }
}

/* norm.rs:38-82: FP32 energy in source order, powf(mean + eps, -0.5), optional direct scale, one rounding */
ORC_API void orc_gm_rms_norm(const uint16_t* in, int rows, int width, float eps, const uint16_t* scale, uint16_t* out) {
    for (int r = 0; r < rows; ++r) {
        const uint16_t* x = in + (int64_t)r * width;
        float energy = 0.0f;
        for (int i = 0; i < width; ++i) {
            const float v = gm_load(x[i]);
            energy += v * v;
        }
        const float mean = energy / (float)width;
        const float inverse = powf(mean + eps, -0.5f);
        for (int i = 0; i < width; ++i) {
            float v = gm_load(x[i]) * inverse;
            if (scale) v *= gm_load(scale[i]);
            out[(int64_t)r * width + i] = orc_gm_bf16(v);
        }
    }
}

/* config.rs:200-247: FP32 exponent (2 pair) / head_dim, 1 / powf(theta, exponent); a proportional layer
 * rotates the first quarter of the pairs and pads the rest with +0 */
ORC_API float orc_gm_inverse_frequency(int head_dim, float theta, int proportional, int pair) {
    const int pairs = head_dim / 2;
    const int active = proportional ? pairs / 4 : pairs;
    if (pair >= active) return 0.0f;
    const float exponent = (float)(pair * 2) / (float)head_dim;
    return 1.0f / powf(theta, exponent);
}

/* rotary.rs:33-93: BF16 cos / sin of the FP32 phase, both halves duplicated */
ORC_API void orc_gm_factors(int head_dim, float theta, int proportional, const uint32_t* positions, int rows,
                            uint16_t* cosine, uint16_t* sine) {
    const int half = head_dim / 2;
    for (int r = 0; r < rows; ++r) {
        const float position = (float)positions[r];
        for (int p = 0; p < half; ++p) {
            const float phase = position * orc_gm_inverse_frequency(head_dim, theta, proportional, p);
            const uint16_t c = orc_gm_bf16(cosf(phase)), s = orc_gm_bf16(sinf(phase));
            cosine[r * head_dim + p] = c;
            cosine[r * head_dim + p + half] = c;
            sine[r * head_dim + p] = s;
            sine[r * head_dim + p + half] = s;
        }
    }
}

static inline float gm_mul_round(float a, float b) { return gm_load(orc_gm_bf16(a * b)); }

/* rotary.rs:95-140: each product rounded to BF16, FP32 addition, sum rounded */
ORC_API void orc_gm_apply_rotary(const uint16_t* in, int rows, int heads, int width, const uint16_t* cosine,
                                 const uint16_t* sine, uint16_t* out) {
    const int half = width / 2;
    for (int r = 0; r < rows; ++r) {
        for (int h = 0; h < heads; ++h) {
            const int64_t base = ((int64_t)r * heads + h) * width;
            for (int j = 0; j < half; ++j) {
                const int f = r * width + j;
                const float a = gm_load(in[base + j]), b = gm_load(in[base + j + half]);
                const float c1 = gm_load(cosine[f]), s1 = gm_load(sine[f]);
                const float c2 = gm_load(cosine[f + half]), s2 = gm_load(sine[f + half]);
                const float first = gm_mul_round(a, c1) + gm_mul_round(-b, s1);
                const float second = gm_mul_round(b, c2) + gm_mul_round(a, s2);
                out[base + j] = orc_gm_bf16(first);
                out[base + j + half] = orc_gm_bf16(second);
            }
        }
    }
}

/* attention.rs:203-277: BF16 scores (scaling 1.0), FP32 softmax, BF16 weights, FP32 accumulation over keys
 * in order, one BF16 rounding.  window 0 = full attention.  query [seq][heads * width], keys / values
 * [kv_seq][kv_heads * width]; key i has absolute position key_start + i. */
ORC_API int orc_gm_attention(const uint16_t* query, int seq, const uint16_t* keys, const uint16_t* values, int kv_seq,
                             int heads, int kv_heads, int width, int window, int query_start, int key_start,
                             uint16_t* out) {
    if (heads <= 0 || kv_heads <= 0 || width <= 0 || heads % kv_heads || seq <= 0 || kv_seq <= 0 || window < 0) return -1;
    if (query_start + seq > key_start + kv_seq || query_start < key_start) return -1;
    const int groups = heads / kv_heads;
    const int64_t head_step = (int64_t)heads * width, kv_step = (int64_t)kv_heads * width;
    int failed = 0;
#pragma omp parallel for collapse(2) schedule(static)
    for (int p = 0; p < seq; ++p) {
        for (int h = 0; h < heads; ++h) {
            float* scores = (float*)malloc(sizeof(float) * (size_t)kv_seq);
            float* acc = (float*)malloc(sizeof(float) * (size_t)width);
            if (!scores || !acc) { failed = 1; free(scores); free(acc); continue; }
            const int absolute = query_start + p;
            int last = absolute - key_start;
            if (last > kv_seq - 1) last = kv_seq - 1;
            int first = 0;
            if (window > 0) {
                int lo = absolute - (window - 1);
                if (lo < 0) lo = 0;
                lo -= key_start;
                if (lo < 0) lo = 0;
                first = lo < last ? lo : last;
            }
            const int kv_head = h / groups;
            const uint16_t* q = query + p * head_step + (int64_t)h * width;
            float maximum = -INFINITY;
            for (int t = first; t <= last; ++t) {
                const uint16_t* key = keys + t * kv_step + (int64_t)kv_head * width;
                float sum = 0.0f;
                for (int c = 0; c < width; ++c) sum += gm_load(q[c]) * gm_load(key[c]);
                scores[t] = gm_load(orc_gm_bf16(sum));
                maximum = fmaxf(maximum, scores[t]);
            }
            float total = 0.0f;
            for (int t = first; t <= last; ++t) {
                scores[t] = expf(scores[t] - maximum);
                total += scores[t];
            }
            for (int c = 0; c < width; ++c) acc[c] = 0.0f;
            for (int t = first; t <= last; ++t) {
                const float weight = gm_load(orc_gm_bf16(scores[t] / total));
                const uint16_t* value = values + t * kv_step + (int64_t)kv_head * width;
                for (int c = 0; c < width; ++c) acc[c] += weight * gm_load(value[c]);
            }
            uint16_t* o = out + p * head_step + (int64_t)h * width;
            for (int c = 0; c < width; ++c) o[c] = orc_gm_bf16(acc[c]);
            free(scores);
            free(acc);
        }
    }
    return failed ? -2 : 0;
}

/* elementwise.rs: every function rounds once per step it names */
ORC_API void orc_gm_add(const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_gm_bf16(gm_load(a[i]) + gm_load(b[i]));
}
ORC_API void orc_gm_multiply(const uint16_t* a, const uint16_t* b, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_gm_bf16(gm_load(a[i]) * gm_load(b[i]));
}
ORC_API void orc_gm_scale(const uint16_t* a, float factor, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_gm_bf16(gm_load(a[i]) * factor);
}
/* elementwise.rs:66-83 */
ORC_API void orc_gm_gelu_tanh(const uint16_t* a, int64_t n, uint16_t* out) {
    const float alpha = 0.7978846f, cubic = 0.044715f;
    for (int64_t i = 0; i < n; ++i) {
        const float x = gm_load(a[i]);
        const float inner = alpha * x * (1.0f + cubic * x * x);
        out[i] = orc_gm_bf16(0.5f * x * (1.0f + tanhf(inner)));
    }
}
/* elementwise.rs:85-107: divide, tanh, multiply, each rounded */
ORC_API void orc_gm_softcap(const uint16_t* a, float cap, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) {
        const uint16_t divided = orc_gm_bf16(gm_load(a[i]) / cap);
        const uint16_t hyperbolic = orc_gm_bf16(tanhf(gm_load(divided)));
        out[i] = orc_gm_bf16(gm_load(hyperbolic) * cap);
    }
}
/* elementwise.rs:109-115: (context + token) * 2^-1/2, two roundings */
ORC_API void orc_gm_ple_combine(const uint16_t* context, const uint16_t* token, int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) {
        const uint16_t sum = orc_gm_bf16(gm_load(context[i]) + gm_load(token[i]));
        out[i] = orc_gm_bf16(gm_load(sum) * 0.70710678118654752440f);
    }
}
/* decoder.rs:316-332: first maximum wins; a NaN never replaces the incumbent */
ORC_API uint32_t orc_gm_argmax(const uint16_t* logits, int64_t n) {
    int64_t best = 0;
    for (int64_t i = 1; i < n; ++i) {
        if (gm_load(logits[i]) > gm_load(logits[best])) best = i;
    }
    return (uint32_t)best;
}

/* ------------------------------------------------------------------------------------------------
 * Whole decoder (decoder.rs).  One model object holds BF16 tensors by name; one sequence object holds
 * the per-owner key / value history and the position.
 * ---------------------------------------------------------------------------------------------- */
#define GM_MAX_LAYERS 64

typedef struct {
    int32_t layers, hidden, heads, kv_heads, head_dim, global_head_dim, ffn, vocab, ple, ple_vocab, window, context,
        kv_shared;
    float eps, softcap, theta_local, theta_global;
    int32_t full[GM_MAX_LAYERS]; /* 1 = full attention (global head width, proportional rotary) */
} orc_gemma_config;

enum { G_EMBED, G_PLE_EMBED, G_PLE_PROJ, G_PLE_NORM, G_NORM, G_COUNT };
enum { L_Q, L_K, L_V, L_O, L_QNORM, L_KNORM, L_IN, L_POST_ATTN, L_PRE_FFN, L_POST_FFN, L_GATE, L_UP, L_DOWN, L_PLE_GATE,
       L_PLE_PROJ, L_POST_PLE, L_SCALAR, L_COUNT };
static const char* const g_names[G_COUNT] = {"embed_tokens", "embed_tokens_per_layer", "per_layer_model_projection",
                                             "per_layer_projection_norm", "norm"};
static const char* const l_names[L_COUNT] = {"q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "input_layernorm",
                                             "post_attention_layernorm", "pre_feedforward_layernorm",
                                             "post_feedforward_layernorm", "gate_proj", "up_proj", "down_proj",
                                             "per_layer_input_gate", "per_layer_projection",
                                             "post_per_layer_input_norm", "layer_scalar"};

typedef struct {
    orc_gemma_config cfg;
    uint16_t* g[G_COUNT];
    uint16_t* l[GM_MAX_LAYERS][L_COUNT];
    int owner[GM_MAX_LAYERS];
} orc_gemma;

typedef struct {
    const orc_gemma* m;
    uint16_t* keys[GM_MAX_LAYERS];
    uint16_t* values[GM_MAX_LAYERS];
    int position;
} orc_gemma_seq;

static int gm_width(const orc_gemma_config* c, int layer) { return c->full[layer] ? c->global_head_dim : c->head_dim; }

/* config.rs:296-385: layers past the owner prefix reuse the last owner of their own kind */
static int gm_owner(const orc_gemma_config* c, int layer) {
    const int owners = c->layers - c->kv_shared;
    if (layer < owners) return layer;
    for (int i = owners - 1; i >= 0; --i) {
        if (c->full[i] == c->full[layer]) return i;
    }
    return -1;
}

/* expected element count of a tensor, 0 when the layer does not hold it */
static int64_t gm_global_count(const orc_gemma_config* c, int id) {
    const int64_t packed = (int64_t)c->layers * c->ple;
    switch (id) {
        case G_EMBED: return (int64_t)c->vocab * c->hidden;
        case G_PLE_EMBED: return (int64_t)c->ple_vocab * packed;
        case G_PLE_PROJ: return packed * c->hidden;
        case G_PLE_NORM: return c->ple;
        default: return c->hidden;
    }
}
static int64_t gm_layer_count(const orc_gemma_config* c, int layer, int id) {
    const int64_t w = gm_width(c, layer), h = c->hidden;
    switch (id) {
        case L_Q: case L_O: return (int64_t)c->heads * w * h;
        case L_K: case L_V: return (int64_t)c->kv_heads * w * h;
        case L_QNORM: case L_KNORM: return w;
        case L_GATE: case L_UP: case L_DOWN: return (int64_t)c->ffn * h;
        case L_PLE_GATE: case L_PLE_PROJ: return (int64_t)c->ple * h;
        case L_SCALAR: return 1;
        default: return h;
    }
}

ORC_API orc_gemma* orc_gemma_create(const orc_gemma_config* cfg) {
    if (!cfg || cfg->layers <= 0 || cfg->layers > GM_MAX_LAYERS || cfg->kv_shared >= cfg->layers || cfg->kv_shared < 0 ||
        cfg->hidden <= 0 || cfg->heads <= 0 || cfg->kv_heads <= 0 || cfg->heads % cfg->kv_heads || cfg->head_dim % 2 ||
        cfg->global_head_dim % 8 || cfg->ple <= 0 || cfg->ple_vocab < cfg->vocab || !cfg->full[cfg->layers - 1]) {
        return NULL;
    }
    orc_gemma* m = (orc_gemma*)calloc(1, sizeof(orc_gemma));
    if (!m) return NULL;
    m->cfg = *cfg;
    for (int i = 0; i < cfg->layers; ++i) {
        m->owner[i] = gm_owner(cfg, i);
        if (m->owner[i] < 0) { free(m); return NULL; }
    }
    return m;
}

ORC_API void orc_gemma_destroy(orc_gemma* m) {
    if (!m) return;
    for (int i = 0; i < G_COUNT; ++i) free(m->g[i]);
    for (int l = 0; l < GM_MAX_LAYERS; ++l) for (int i = 0; i < L_COUNT; ++i) free(m->l[l][i]);
    free(m);
}

/* names: "embed_tokens", ..., "layers.<i>.<role>"; count must equal the shape the configuration implies */
ORC_API int orc_gemma_set_tensor(orc_gemma* m, const char* name, const uint16_t* data, int64_t count) {
    uint16_t** slot = NULL;
    int64_t expect = 0;
    for (int i = 0; i < G_COUNT; ++i) {
        if (strcmp(name, g_names[i]) == 0) { slot = &m->g[i]; expect = gm_global_count(&m->cfg, i); }
    }
    if (!slot && strncmp(name, "layers.", 7) == 0) {
        char* end = NULL;
        const long layer = strtol(name + 7, &end, 10);
        if (end && *end == '.' && layer >= 0 && layer < m->cfg.layers) {
            for (int i = 0; i < L_COUNT; ++i) {
                if (strcmp(end + 1, l_names[i]) == 0) { slot = &m->l[layer][i]; expect = gm_layer_count(&m->cfg, (int)layer, i); }
            }
        }
    }
    if (!slot || count != expect) return -1;
    free(*slot);
    *slot = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)count);
    if (!*slot) return -2;
    memcpy(*slot, data, sizeof(uint16_t) * (size_t)count);
    return 0;
}

/* decoder.rs:36-71, 194-313: every tensor the configuration needs is present */
ORC_API int orc_gemma_ready(const orc_gemma* m) {
    for (int i = 0; i < G_COUNT; ++i) if (!m->g[i]) return 0;
    for (int l = 0; l < m->cfg.layers; ++l) {
        for (int i = 0; i < L_COUNT; ++i) {
            const int kv_only = i == L_K || i == L_V || i == L_KNORM;
            if (!m->l[l][i] && !(kv_only && m->owner[l] != l)) return 0;
        }
    }
    return 1;
}

ORC_API orc_gemma_seq* orc_gemma_seq_create(const orc_gemma* m) {
    if (!m || !orc_gemma_ready(m)) return NULL;
    orc_gemma_seq* s = (orc_gemma_seq*)calloc(1, sizeof(orc_gemma_seq));
    if (!s) return NULL;
    s->m = m;
    for (int l = 0; l < m->cfg.layers; ++l) {
        if (m->owner[l] != l) continue;
        const size_t n = (size_t)m->cfg.context * m->cfg.kv_heads * gm_width(&m->cfg, l);
        s->keys[l] = (uint16_t*)malloc(sizeof(uint16_t) * n);
        s->values[l] = (uint16_t*)malloc(sizeof(uint16_t) * n);
    }
    return s;
}

ORC_API void orc_gemma_seq_destroy(orc_gemma_seq* s) {
    if (!s) return;
    for (int l = 0; l < GM_MAX_LAYERS; ++l) { free(s->keys[l]); free(s->values[l]); }
    free(s);
}

ORC_API int orc_gemma_seq_position(const orc_gemma_seq* s) { return s->position; }
ORC_API void orc_gemma_seq_reset(orc_gemma_seq* s) { s->position = 0; }

static uint16_t* gm_alloc(int64_t n) { return (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(n > 0 ? n : 1)); }

/* decoder.rs:458-568 */
static int gm_attention_forward(orc_gemma_seq* s, int layer, int seq, const uint32_t* positions, const uint16_t* hidden,
                                uint16_t* out) {
    const orc_gemma* m = s->m;
    const orc_gemma_config* c = &m->cfg;
    const int H = c->hidden, heads = c->heads, kvh = c->kv_heads, w = gm_width(c, layer), owner = m->owner[layer];
    uint16_t* const* L = m->l[layer];
    uint16_t* normed = gm_alloc((int64_t)seq * H);
    uint16_t* q = gm_alloc((int64_t)seq * heads * w);
    uint16_t* q2 = gm_alloc((int64_t)seq * heads * w);
    uint16_t* cosine = gm_alloc((int64_t)seq * w);
    uint16_t* sine = gm_alloc((int64_t)seq * w);
    uint16_t* k = gm_alloc((int64_t)seq * kvh * w);
    uint16_t* k2 = gm_alloc((int64_t)seq * kvh * w);
    uint16_t* attended = gm_alloc((int64_t)seq * heads * w);
    uint16_t* projected = gm_alloc((int64_t)seq * H);
    int rc = 0;
    orc_gm_rms_norm(hidden, seq, H, c->eps, L[L_IN], normed);
    orc_gm_project(normed, seq, L[L_Q], (int64_t)heads * w, H, q);
    orc_gm_rms_norm(q, seq * heads, w, c->eps, L[L_QNORM], q2);
    orc_gm_factors(w, c->full[layer] ? c->theta_global : c->theta_local, c->full[layer], positions, seq, cosine, sine);
    orc_gm_apply_rotary(q2, seq, heads, w, cosine, sine, q);
    if (owner == layer) {
        const int64_t at = (int64_t)s->position * kvh * w;
        orc_gm_project(normed, seq, L[L_K], (int64_t)kvh * w, H, k);
        orc_gm_rms_norm(k, seq * kvh, w, c->eps, L[L_KNORM], k2);
        orc_gm_apply_rotary(k2, seq, kvh, w, cosine, sine, s->keys[layer] + at);
        orc_gm_project(normed, seq, L[L_V], (int64_t)kvh * w, H, k);
        orc_gm_rms_norm(k, seq * kvh, w, c->eps, NULL, s->values[layer] + at);
    }
    rc = orc_gm_attention(q, seq, s->keys[owner], s->values[owner], s->position + seq, heads, kvh, w,
                          c->full[layer] ? 0 : c->window, s->position, 0, attended);
    orc_gm_project(attended, seq, L[L_O], H, (int64_t)heads * w, projected);
    orc_gm_rms_norm(projected, seq, H, c->eps, L[L_POST_ATTN], normed);
    orc_gm_add(hidden, normed, (int64_t)seq * H, out);
    free(normed); free(q); free(q2); free(cosine); free(sine); free(k); free(k2); free(attended); free(projected);
    return rc;
}

/* decoder.rs:570-626 */
static void gm_feedforward_forward(const orc_gemma* m, int layer, int seq, const uint16_t* hidden, const uint16_t* per_layer,
                                   uint16_t* out) {
    const orc_gemma_config* c = &m->cfg;
    const int H = c->hidden, F = c->ffn, P = c->ple;
    uint16_t* const* L = m->l[layer];
    uint16_t* normed = gm_alloc((int64_t)seq * H);
    uint16_t* gate = gm_alloc((int64_t)seq * F);
    uint16_t* up = gm_alloc((int64_t)seq * F);
    uint16_t* down = gm_alloc((int64_t)seq * H);
    uint16_t* mid = gm_alloc((int64_t)seq * H);
    uint16_t* pg = gm_alloc((int64_t)seq * P);
    orc_gm_rms_norm(hidden, seq, H, c->eps, L[L_PRE_FFN], normed);
    orc_gm_project(normed, seq, L[L_GATE], F, H, gate);
    orc_gm_project(normed, seq, L[L_UP], F, H, up);
    orc_gm_gelu_tanh(gate, (int64_t)seq * F, gate);
    orc_gm_multiply(gate, up, (int64_t)seq * F, gate);
    orc_gm_project(gate, seq, L[L_DOWN], H, F, down);
    orc_gm_rms_norm(down, seq, H, c->eps, L[L_POST_FFN], normed);
    orc_gm_add(hidden, normed, (int64_t)seq * H, mid);
    /* per-layer embedding gate */
    orc_gm_project(mid, seq, L[L_PLE_GATE], P, H, pg);
    orc_gm_gelu_tanh(pg, (int64_t)seq * P, pg);
    orc_gm_multiply(pg, per_layer, (int64_t)seq * P, pg);
    orc_gm_project(pg, seq, L[L_PLE_PROJ], H, P, down);
    orc_gm_rms_norm(down, seq, H, c->eps, L[L_POST_PLE], normed);
    orc_gm_add(mid, normed, (int64_t)seq * H, down);
    orc_gm_scale(down, gm_load(L[L_SCALAR][0]), (int64_t)seq * H, out);
    free(normed); free(gate); free(up); free(down); free(mid); free(pg);
}

/* decoder.rs:133-192, 334-445: process `n` tokens; logits (vocab BF16 values of the last token, after the
 * soft cap) may be NULL (advance_prefill).  hidden_out, when given, receives the last token's final hidden
 * row.  Returns 0, or a negative code with the sequence unchanged. */
ORC_API int orc_gemma_step(orc_gemma_seq* s, const uint32_t* tokens, int n, uint16_t* logits, uint16_t* hidden_out) {
    const orc_gemma* m = s->m;
    const orc_gemma_config* c = &m->cfg;
    if (n <= 0 || s->position + n > c->context) return -1;
    for (int i = 0; i < n; ++i) if (tokens[i] >= (uint32_t)c->vocab) return -1;
    const int H = c->hidden, P = c->ple, packed = c->layers * c->ple;
    const float embed_scale = gm_load(orc_gm_bf16(sqrtf((float)H)));
    const float ple_embed_scale = gm_load(orc_gm_bf16(sqrtf((float)P)));
    const float ple_projection_scale = 1.0f / sqrtf((float)H);
    uint16_t* hidden = gm_alloc((int64_t)n * H);
    uint16_t* next = gm_alloc((int64_t)n * H);
    uint16_t* identity = gm_alloc((int64_t)n * packed);
    uint16_t* projection = gm_alloc((int64_t)n * packed);
    uint16_t* per_layer = gm_alloc((int64_t)c->layers * n * P);
    uint16_t* slice = gm_alloc((int64_t)n * P);
    uint16_t* ident = gm_alloc((int64_t)n * P);
    uint32_t* positions = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)n);
    int rc = 0;
    for (int i = 0; i < n; ++i) {
        orc_gm_scale(m->g[G_EMBED] + (int64_t)tokens[i] * H, embed_scale, H, hidden + (int64_t)i * H);
        orc_gm_scale(m->g[G_PLE_EMBED] + (int64_t)tokens[i] * packed, ple_embed_scale, packed, identity + (int64_t)i * packed);
        positions[i] = (uint32_t)(s->position + i);
    }
    orc_gm_project(hidden, n, m->g[G_PLE_PROJ], packed, H, projection);
    orc_gm_scale(projection, ple_projection_scale, (int64_t)n * packed, projection);
    for (int l = 0; l < c->layers; ++l) {
        for (int i = 0; i < n; ++i) {
            memcpy(slice + (int64_t)i * P, projection + (int64_t)i * packed + l * P, sizeof(uint16_t) * (size_t)P);
            memcpy(ident + (int64_t)i * P, identity + (int64_t)i * packed + l * P, sizeof(uint16_t) * (size_t)P);
        }
        orc_gm_rms_norm(slice, n, P, c->eps, m->g[G_PLE_NORM], slice);
        orc_gm_ple_combine(slice, ident, (int64_t)n * P, per_layer + (int64_t)l * n * P);
    }
    for (int l = 0; l < c->layers && rc == 0; ++l) {
        rc = gm_attention_forward(s, l, n, positions, hidden, next);
        if (rc == 0) gm_feedforward_forward(m, l, n, next, per_layer + (int64_t)l * n * P, hidden);
    }
    if (rc == 0) {
        const uint16_t* last = hidden + (int64_t)(n - 1) * H;
        if (hidden_out) memcpy(hidden_out, last, sizeof(uint16_t) * (size_t)H);
        if (logits) {
            /* decoder.rs:410-428: final norm, tied head, soft cap */
            orc_gm_rms_norm(last, 1, H, c->eps, m->g[G_NORM], next);
            orc_gm_project(next, 1, m->g[G_EMBED], c->vocab, H, logits);
            orc_gm_softcap(logits, c->softcap, c->vocab, logits);
        }
        s->position += n;
    }
    free(hidden); free(next); free(identity); free(projection); free(per_layer); free(slice); free(ident); free(positions);
    return rc;
}
