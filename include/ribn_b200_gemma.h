/*
 * ribn_b200 — C ABI of the B200-native (sm_100a) Gemma-4 text decoder that stands behind the
 * reference's `GemmaDecode` backend trait (crates/gemma4/src/executor/backend.rs:10-34) and, batched
 * across sequences, behind its `GenerationExecutor` for Gemma (crates/gemma4/src/executor.rs:55-294).
 *
 * Arithmetic policy is the reference host decoder's (crates/gemma4/src/cpu): BF16 storage, FP32
 * arithmetic, one BF16 round-to-nearest-even after every operation.  All tensors cross this boundary as
 * BF16 bit patterns (uint16_t).  The library owns all device memory; callers own their host arrays only
 * for the duration of a call.  One thread per model object.  There is no CPU fallback.
 */
#ifndef RIBN_B200_GEMMA_H
#define RIBN_B200_GEMMA_H

#include <stddef.h>
#include <stdint.h>

#include "ribn_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define RIBN_B200_GEMMA_MAX_LAYERS 64

/* Text configuration (crates/gemma4/src/config.rs:33-124, accessors 154-198).  `full[i]` = 1 marks a
 * full-attention layer (global head width, proportional quarter rotary); 0 a sliding-window layer.  The
 * last `kv_shared` layers reuse the keys / values of the last earlier layer of their kind
 * (config.rs:296-385).  Widths (hidden, ffn, ple, both head widths) must be multiples of 8. */
/* Passes of 16 or more rows (prefill chunks) run their projections on the tensor cores: BF16 products
 * accumulated in FP32 in the tensor core's order, one BF16 rounding per output.  Off by default: the
 * default projections add in source order like the reference's host decoder (linear.rs:23-66) and
 * reproduce its bits; with the flag a logit can move by a rounding step of an intermediate. */
#define RIBN_B200_GEMMA_FLAG_TENSOR_CORE_PREFILL 1

typedef struct ribn_b200_gemma_config {
    int32_t layers, hidden, heads, kv_heads, head_dim, global_head_dim, ffn, vocab;
    int32_t ple;        /* hidden_size_per_layer_input */
    int32_t ple_vocab;  /* vocab_size_per_layer_input, >= vocab */
    int32_t window;     /* sliding_window */
    int32_t context;    /* max_position_embeddings served by this object */
    int32_t kv_shared;  /* num_kv_shared_layers */
    float eps, softcap, theta_local, theta_global;
    int32_t full[RIBN_B200_GEMMA_MAX_LAYERS];
    int32_t max_sequences;     /* concurrently open continuations */
    int32_t max_batch_tokens;  /* rows processed per pass; longer chunks run as several passes */
    int32_t device;
    int32_t flags;             /* RIBN_B200_GEMMA_FLAG_* */
} ribn_b200_gemma_config;

typedef struct ribn_b200_gemma ribn_b200_gemma;

/* One row of a batched step: `n_tokens` consecutive tokens appended to `sequence`.  With want_output
 * the row yields the greedy token (first maximum, crates/gemma4/src/cpu/decoder.rs:316-332) of the
 * logits after its last token, as `prefill` / `decode` do; without, it is `advance_prefill`. */
typedef struct ribn_b200_gemma_row {
    uint64_t sequence;
    const uint32_t* tokens;
    uint32_t n_tokens;
    uint32_t want_output;
} ribn_b200_gemma_row;

RIBN_B200_API int ribn_b200_gemma_create(const ribn_b200_gemma_config* config, ribn_b200_gemma** out, char* error,
                                         size_t error_capacity);
RIBN_B200_API int ribn_b200_gemma_destroy(ribn_b200_gemma* model);
RIBN_B200_API const char* ribn_b200_gemma_last_error(const ribn_b200_gemma* model);

/* Weights.  Names: "embed_tokens", "embed_tokens_per_layer", "per_layer_model_projection",
 * "per_layer_projection_norm", "norm", and "layers.<i>.<role>" with role one of q_proj, k_proj, v_proj,
 * o_proj, q_norm, k_norm, input_layernorm, post_attention_layernorm, pre_feedforward_layernorm,
 * post_feedforward_layernorm, gate_proj, up_proj, down_proj, per_layer_input_gate, per_layer_projection,
 * post_per_layer_input_norm, layer_scalar (the reference's inventory, crates/gemma4/src/cpu/decoder.rs:
 * 205-313).  `count` must equal the element count the configuration implies. */
RIBN_B200_API int ribn_b200_gemma_load_tensor(ribn_b200_gemma* model, const char* name, const uint16_t* values,
                                              size_t count);
/* Seeded N(0, 0.02) matrices rounded to BF16; norm scales and layer scalars 1.0. */
RIBN_B200_API int ribn_b200_gemma_init_synthetic(ribn_b200_gemma* model, uint64_t seed);
RIBN_B200_API int ribn_b200_gemma_read_tensor(ribn_b200_gemma* model, const char* name, uint16_t* out, size_t capacity,
                                              size_t* count);
/* Checks the inventory and builds the rotary factor tables; required before any sequence opens. */
RIBN_B200_API int ribn_b200_gemma_finalize(ribn_b200_gemma* model);

/* `GemmaDecode` (backend.rs:10-34), one continuation per sequence id. */
RIBN_B200_API int ribn_b200_gemma_open(ribn_b200_gemma* model, uint64_t* sequence);
RIBN_B200_API int ribn_b200_gemma_advance_prefill(ribn_b200_gemma* model, uint64_t sequence, const uint32_t* tokens,
                                                  uint32_t n_tokens);
/* logits: vocab BF16 values after the soft cap, or NULL; token: their greedy choice, or NULL. */
RIBN_B200_API int ribn_b200_gemma_prefill(ribn_b200_gemma* model, uint64_t sequence, const uint32_t* tokens,
                                          uint32_t n_tokens, uint16_t* logits, uint32_t* token);
RIBN_B200_API int ribn_b200_gemma_decode(ribn_b200_gemma* model, uint64_t sequence, uint32_t input, uint16_t* logits,
                                         uint32_t* token);
RIBN_B200_API int ribn_b200_gemma_position(const ribn_b200_gemma* model, uint64_t sequence, uint32_t* position);
RIBN_B200_API int ribn_b200_gemma_close(ribn_b200_gemma* model, uint64_t sequence);

/* Batched step over rows of distinct sequences (what one `GenerationExecutor::submit` maps to): weights
 * are read once for all rows.  tokens_out[i] receives row i's greedy token when it wants output.
 * logits_out, when not NULL, receives vocab BF16 values per row that wants output, in row order.
 * REJECTED (nothing advanced): unknown sequence, out-of-range token, context exceeded, duplicate sequence. */
RIBN_B200_API int ribn_b200_gemma_step(ribn_b200_gemma* model, const ribn_b200_gemma_row* rows, uint32_t n_rows,
                                       uint32_t* tokens_out, uint16_t* logits_out);
RIBN_B200_API int ribn_b200_gemma_synchronize(ribn_b200_gemma* model);
/* Kernel launches and device milliseconds of the last step (measurement aid). */
RIBN_B200_API int ribn_b200_gemma_last_step_stats(const ribn_b200_gemma* model, float* milliseconds, uint32_t* launches);

#ifdef __cplusplus
}
#endif

#endif /* RIBN_B200_GEMMA_H */
