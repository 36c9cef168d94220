/*
 * ribn_b200 — C ABI of the B200-native (sm_100a) batched decode / chunked-prefill
 * executor that stands behind ribn's `GenerationExecutor` trait.
 *
 * Every entry point takes plain pointers and sizes; the library owns all
 * device memory; the caller owns its host arrays only for the duration of a
 * call.  All calls on one executor must come from one thread (the reference's
 * trait is `Send`, not `Sync`: crates/runtime/src/executor.rs:171).
 *
 * There is no CPU fallback: every compute entry point runs CUDA kernels and
 * returns RIBN_B200_ERROR when no usable device exists.
 */
#ifndef RIBN_B200_H
#define RIBN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define RIBN_B200_API __attribute__((visibility("default")))
#else
#define RIBN_B200_API
#endif

/* GGML tensor value types accepted by the loader (crates/gguf/src/lib.rs
 * tensor_layout; numbering is GGUF's). */
enum {
    RIBN_B200_F32 = 0,
    RIBN_B200_F16 = 1,
    RIBN_B200_Q8_0 = 8,
    RIBN_B200_Q4_K = 12,
    RIBN_B200_Q6_K = 14
};

/* Return codes.  ERROR corresponds to `Err(ExecutionError)` (faults the
 * engine); REJECTED / DEFERRED to `Admission::Rejected` / `Admission::Deferred`
 * (crates/runtime/src/executor.rs:109-129); PENDING to `poll -> Ok(None)`. */
enum {
    RIBN_B200_OK = 0,
    RIBN_B200_PENDING = 1,
    RIBN_B200_REJECTED = 2,
    RIBN_B200_DEFERRED = 3,
    RIBN_B200_SELECTED = 4,  /* prepare_rows: BatchPreparation::Selected, one decision per offered row */
    RIBN_B200_ERROR = -1
};

/* StepKind (crates/runtime/src/executor.rs:35-39). */
enum { RIBN_B200_PREFILL = 0, RIBN_B200_DECODE = 1 };

/* Quantisation schemes of the seeded synthetic checkpoints. */
enum {
    RIBN_B200_SCHEME_Q8_0 = 0,   /* every matrix Q8_0 */
    RIBN_B200_SCHEME_Q4_K_M = 1  /* Q4_K; Q6_K for attn_v, ffn_down, output */
};

typedef struct ribn_b200_executor ribn_b200_executor;

/* Dense Qwen3-architecture geometry plus the executor's scheduling limits
 * (GenerationLimits, crates/runtime/src/executor.rs:43-51; QwenLoadOptions,
 * crates/qwen/src/loading.rs:29-81). */
typedef struct {
    int32_t layers;
    int32_t hidden;
    int32_t q_heads;
    int32_t kv_heads;
    int32_t head_dim;
    int32_t ffn;
    int32_t vocab;
    float rope_base;
    float rms_eps;
    int32_t context_tokens;   /* longest prompt + output of one sequence */
    int32_t max_sequences;    /* concurrent sequences */
    int32_t max_batch_tokens; /* tokens per submitted batch */
    int32_t kv_pages;         /* 16-token pages in the shared KV arena; 0 = enough for
                                 max_sequences full contexts */
    int32_t device;           /* CUDA ordinal */
    int32_t flags;            /* RIBN_B200_FLAG_* */
    int32_t tp_size;          /* tensor-parallel group size: 0 or 1 = none, else 2, 4 or 8 */
    int32_t tp_rank;          /* this executor's rank in the group */
} ribn_b200_config;

enum {
    RIBN_B200_FLAG_KEEP_LOGITS = 1,   /* keep F32 logits of sampling rows for copy_logits */
    RIBN_B200_FLAG_REFERENCE_KERNELS = 2, /* run the plain one-warp-per-row CUDA kernels
                                             (slow; used to cross-check the fast path) */
    RIBN_B200_FLAG_NO_GRAPH = 4,      /* launch kernels directly instead of replaying graphs */
    RIBN_B200_FLAG_NO_TCGEN05 = 8,    /* batches of 3+ rows on the integer mma.sync kernel instead of tcgen05 */
    RIBN_B200_FLAG_KV_ON_DEMAND = 16, /* admit reserves the prompt's KV pages only; prepare takes the pages a row's
                                         range needs and defers the rows the arena cannot serve */
    RIBN_B200_FLAG_OPERAND_CACHE = 32 /* finalize also keeps every Q4_K / Q6_K matrix as tcgen05 operands (binary16
                                         integers, 2 or 4 bytes of HBM per weight); steps of 3+ rows then copy operand
                                         stages instead of converting packed tiles.  Same results bit for bit. */
};

/* GenerationLimits (crates/runtime/src/executor.rs:43-51). */
typedef struct {
    uint32_t context_tokens;
    uint32_t max_sequences;
    uint32_t max_batch_tokens;
    uint32_t max_decode_tokens; /* always 1 */
    uint32_t kv_page_tokens;    /* 16: crates/qwen/src/gguf.rs:16 */
    uint32_t kv_pages_total;
    uint32_t kv_pages_free;
} ribn_b200_limits;

/* BatchItem (crates/runtime/src/executor.rs:67-79). */
typedef struct {
    uint64_t sequence;
    uint32_t kind;          /* RIBN_B200_PREFILL / RIBN_B200_DECODE */
    uint32_t prefix;
    uint32_t token_budget;
    uint32_t output_budget;
} ribn_b200_batch_item;

/* TokenRequest.options.sampling: Sampling{temperature, top_p, top_k, seed}
 * (crates/runtime/src/executor.rs, crates/qwen/src/execution.rs:107-111).  Only greedy selection
 * (temperature 0) is executed; anything else is Admission::Rejected, as in the reference. */
typedef struct {
    float temperature;
    float top_p;
    uint32_t top_k;
    uint32_t reserved;
    uint64_t seed;
} ribn_b200_sampling;

/* PreparedRow (crates/runtime/src/executor.rs:97-105): the decision for one offered row.  READY rows keep
 * identity, kind and prefix; their budgets may have shrunk, never to zero.  DEFERRED rows retain nothing
 * new and should be offered again after a release.  REJECTED is reserved for request-local refusals. */
enum { RIBN_B200_ROW_READY = 0, RIBN_B200_ROW_DEFERRED = 1, RIBN_B200_ROW_REJECTED = 2 };
typedef struct {
    uint32_t state;
    uint32_t token_budget;
    uint32_t output_budget;
    uint32_t reserved;
} ribn_b200_prepared_row;

/* StepCompletion (crates/runtime/src/executor.rs:101-106); max_decode_tokens
 * is 1, so a row carries at most one sampled token. */
typedef struct {
    uint64_t sequence;
    uint32_t prefix;    /* absolute prefix after this step */
    uint32_t n_tokens;  /* 0 or 1 */
    uint32_t token;
    uint32_t reserved;
} ribn_b200_completion;

/* ---- lifecycle ---------------------------------------------------------- */

/* Replaces QwenCuda::load_gguf's executor construction
 * (crates/qwen/src/cuda.rs:16-53, crates/qwen/src/loading.rs:93-190). */
RIBN_B200_API int ribn_b200_create(const ribn_b200_config* config, ribn_b200_executor** out,
                                   char* error, size_t error_capacity);
/* Drop (crates/qwen/src/cuda.rs:111-121): synchronises, then frees. */
RIBN_B200_API int ribn_b200_destroy(ribn_b200_executor* executor);

/* Upload one GGUF tensor's encoded bytes verbatim.  Matrices are
 * `[rows = out][cols = in, contiguous]` blocks, norms are F32 vectors with
 * rows = 1.  Names are GGUF's (`blk.N.attn_q.weight`, `token_embd.weight`,
 * `output_norm.weight`, `output.weight`, ...).  Replaces
 * CudaQwen35Weights::stage (crates/nvidia/src/staging.rs:263-315,
 * crates/nvidia/src/cuda.rs:320-387). */
RIBN_B200_API int ribn_b200_load_tensor(ribn_b200_executor* executor, const char* name,
                                        int32_t ggml_type, int64_t rows, int64_t cols,
                                        const void* bytes, size_t byte_count);
/* Fill every tensor with seeded N(0, 0.02) weights quantised on the device
 * (norm weights 1.0).  No reference counterpart: the reference has no
 * quantiser; the encoded bytes are the ground truth shared with any checker. */
RIBN_B200_API int ribn_b200_init_synthetic(ribn_b200_executor* executor, uint64_t seed, int32_t scheme);
/* Copy a loaded tensor's encoded GGUF bytes back to the host
 * (CudaWeightStore::copy_quantized_to_host, crates/nvidia/tests/cuda_reference.rs:244-248).
 * Any of the out pointers may be NULL; `bytes` may be NULL to query the size. */
RIBN_B200_API int ribn_b200_read_tensor(ribn_b200_executor* executor, const char* name,
                                        int32_t* ggml_type, int64_t* rows, int64_t* cols,
                                        void* bytes, size_t capacity, size_t* byte_count);
/* Validate the model plan, repack weights for the fast kernels, allocate the
 * KV arena and step scratch (validate_model_plan, crates/nvidia/src/decode.rs:364-368;
 * loading.rs:93-190).  Must be called once before admit. */
RIBN_B200_API int ribn_b200_finalize(ribn_b200_executor* executor);

/* ---- GenerationExecutor (crates/runtime/src/executor.rs:171-254) -------- */

/* info() */
RIBN_B200_API int ribn_b200_info(ribn_b200_executor* executor, ribn_b200_limits* out);
/* admit(): OK = Admission::Ready (pages for prompt + max_output reserved; with
 * RIBN_B200_FLAG_KV_ON_DEMAND the prompt's pages only), REJECTED, DEFERRED, or ERROR (duplicate
 * sequence / faulted executor).  `sampling` may be NULL (greedy).
 * Semantics follow QwenExecution::admit (crates/qwen/src/execution.rs:80-162). */
RIBN_B200_API int ribn_b200_admit(ribn_b200_executor* executor, uint64_t request_id, uint64_t sequence,
                                  const uint32_t* tokens, uint32_t token_count,
                                  uint32_t max_output_tokens, const ribn_b200_sampling* sampling,
                                  const uint32_t* stop_tokens, uint32_t stop_count);
/* prepare(): OK = BatchPreparation::Ready.  Never advances state
 * (crates/qwen/src/execution.rs:164-269).  A batch the KV arena cannot serve whole is an error
 * here; prepare_rows reports it per row. */
RIBN_B200_API int ribn_b200_prepare(ribn_b200_executor* executor, const ribn_b200_batch_item* items,
                                    uint32_t count);
/* prepare() with the per-row report of BatchPreparation (crates/runtime/src/executor.rs:97-105, 195-204):
 * OK = Ready (every row accepted unchanged), RIBN_B200_SELECTED = Selected (`rows[i]` holds the decision
 * for `items[i]`: a row whose range needs KV pages the arena cannot give is DEFERRED and retains nothing
 * new; READY rows carry their granted budgets, which this executor never shrinks).  Pages granted to
 * READY rows stay with their sequences.  submit() then takes exactly the READY rows, in offered order,
 * with their granted budgets; when none is READY call abandon_preparation().  `rows` may be NULL, which
 * makes this ribn_b200_prepare. */
RIBN_B200_API int ribn_b200_prepare_rows(ribn_b200_executor* executor, const ribn_b200_batch_item* items,
                                         uint32_t count, ribn_b200_prepared_row* rows);
/* abandon_preparation(): idempotent. */
RIBN_B200_API int ribn_b200_abandon_preparation(ribn_b200_executor* executor);
/* submit(): asynchronous; must repeat the prepared rows
 * (crates/qwen/src/execution.rs:275-316). */
RIBN_B200_API int ribn_b200_submit(ribn_b200_executor* executor, const ribn_b200_batch_item* items,
                                   uint32_t count, uint64_t* submission);
/* poll(): PENDING while the device is busy, else OK with exactly one row per
 * submitted row, in order (crates/qwen/src/execution.rs:329-414). */
RIBN_B200_API int ribn_b200_poll(ribn_b200_executor* executor, uint64_t submission,
                                 ribn_b200_completion* rows, uint32_t capacity, uint32_t* count);
/* release(): idempotent (crates/qwen/src/execution.rs:416-440).  A sequence named by the outstanding
 * preparation is refused ("cannot release prepared Qwen state").  A sequence the pending submission
 * still reads is parked and retired when that submission completes at poll()
 * (deferred_releases, crates/nvidia/src/serving.rs:1082-1096, 1231-1251); the call returns OK. */
RIBN_B200_API int ribn_b200_release(ribn_b200_executor* executor, uint64_t sequence);
/* synchronize(): block until every queued launch has finished. */
RIBN_B200_API int ribn_b200_synchronize(ribn_b200_executor* executor);
/* ExecutionError text of the last failing call, at most 4096 bytes
 * (crates/runtime/src/executor.rs:134-152).  Returns the length written. */
RIBN_B200_API size_t ribn_b200_last_error(ribn_b200_executor* executor, char* buffer, size_t capacity);

/* ---- tensor parallelism (one executor per GPU, one process per GPU) ------- */
/* No reference counterpart: the reference runs on one device (docs/architecture.md).  With tp_size > 1 an
 * executor holds one shard of every layer: q / k / v split by head and ffn gate / up by output column, the
 * attention output and ffn down projections split along K on 256-input block boundaries (the ffn blocks are
 * dealt out as evenly as they go: FFN 25600 = 100 blocks gives 13,13,13,13,12,12,12,12 at eight ranks), the KV
 * cache by kv head; norms, the embedding and the output head are replicated (every rank selects the same token).
 * After the attention output and the ffn down projection the ranks' F32 partial sums `[tokens, hidden]` meet in an
 * NCCL all-reduce(sum) on the executor's stream (captured into the step graphs), then join the residual stream.
 * Every rank must be driven with the same admit / prepare / submit sequence.
 * load_tensor takes the WHOLE tensor on every rank and keeps its shard; read_tensor returns the shard. */
typedef struct { char bytes[128]; } ribn_b200_nccl_id;   /* ncclUniqueId */
/* Rank 0: make the group's id with the NCCL library at `nccl_library` (a path to libnccl.so.2) and hand it to the
 * other ranks out of band (the host's own channel: a store, a pipe, a gloo broadcast). */
RIBN_B200_API int ribn_b200_tp_unique_id(const char* nccl_library, ribn_b200_nccl_id* id, char* error,
                                         size_t error_capacity);
/* Every rank, after create and before finalize: join the group (collective: returns once all ranks called). */
RIBN_B200_API int ribn_b200_tp_init(ribn_b200_executor* executor, const char* nccl_library,
                                    const ribn_b200_nccl_id* id);
/* Measurement aid (collective: every rank calls it with the same arguments): average device time of one
 * all-reduce of `tokens` x hidden F32 values on the executor's stream, as the step issues it. */
RIBN_B200_API int ribn_b200_tp_time_allreduce(ribn_b200_executor* executor, uint32_t tokens, uint32_t repeats,
                                              float* average_us);
/* Which part of a whole tensor a rank keeps (no device work): rows [row0, row0 + rows) and columns
 * [col0, col0 + cols) of the `[full_rows][full_cols]` tensor `name`, for config->tp_rank of config->tp_size. */
RIBN_B200_API int ribn_b200_tp_shard(const ribn_b200_config* config, const char* name, int64_t full_rows,
                                     int64_t full_cols, int64_t* row0, int64_t* rows, int64_t* col0, int64_t* cols);

/* ---- parity / measurement taps ------------------------------------------ */

/* F32 logits of sampling row `row` of the last completed submission
 * (CudaQwen35Decode::copy_logits, crates/nvidia/src/decode.rs:788).
 * Needs RIBN_B200_FLAG_KEEP_LOGITS. */
RIBN_B200_API int ribn_b200_copy_logits(ribn_b200_executor* executor, uint32_t row, float* out,
                                        size_t capacity);
/* F16 K (which = 0) or V (which = 1) rows of one layer for the first `tokens`
 * positions of a sequence, gathered through its page table into
 * `[token][kv_head][head_dim]`. */
RIBN_B200_API int ribn_b200_copy_kv(ribn_b200_executor* executor, uint64_t sequence, int32_t layer,
                                    int32_t which, uint32_t tokens, uint16_t* out);
/* Measurement aid: mark `tokens` positions of an admitted sequence as already
 * consumed, with its KV pages filled with seeded F16 values and `next_token`
 * as its pending decode input, so steady-state decode at a long context can
 * be timed without running the prefill. */
RIBN_B200_API int ribn_b200_debug_set_context(ribn_b200_executor* executor, uint64_t sequence,
                                              uint32_t tokens, uint32_t next_token, uint64_t seed);
/* Device time (CUDA events on the executor's stream) of the last completed
 * submission, and how many kernels it launched. */
RIBN_B200_API int ribn_b200_last_step_stats(ribn_b200_executor* executor, float* device_ms,
                                            uint32_t* kernel_launches);
/* Algorithmic HBM bytes of one decode step: quantised weight bytes read once
 * plus `context_tokens_total` tokens of F16 K and V over all layers. */
RIBN_B200_API int ribn_b200_step_bytes(ribn_b200_executor* executor, uint64_t context_tokens_total,
                                       uint64_t* weight_bytes, uint64_t* kv_bytes);

/* Measurement aid: enqueue `repeats` launches of one of the decode step's projection kernels for a
 * single row (which: 0 = q|k|v, 1 = attention output, 2 = gate|up, 3 = down, 4 = output head),
 * launch r on layer r % layers so that every launch streams its weights from HBM, and report the
 * average device time per launch from CUDA events on the executor's stream together with the
 * encoded weight bytes one launch reads.  Overwrites the step's activation buffers; call it only
 * between steps.  Counterpart of the reference's device-side kernel timing loop in
 * crates/nvidia/examples/qwen_decode_bench.rs. */
RIBN_B200_API int ribn_b200_time_projection(ribn_b200_executor* executor, int32_t which, uint32_t repeats,
                                            float* average_us, uint64_t* bytes_per_launch);

/* ---- failure detection aids (no GPU fault is involved in any of them) ------ */

/* Host-side fault injection, the counterpart of the switches of the reference's contract tests
 * (crates/runtime/tests/contract.rs:12-31).  ALLOC_REFUSAL: the next `value` device allocations of this
 * executor fail as if the device were out of memory.  ERROR_WORD: the next submitted step ends with
 * `value` in the word that a kernel's expired bounded wait writes.  BAD_ROW: the next `value` submits
 * corrupt one row record before the host-side check of the step plan.  Each surfaces as RIBN_B200_ERROR
 * with a message in last_error and leaves the executor faulted. */
enum { RIBN_B200_INJECT_ALLOC_REFUSAL = 1, RIBN_B200_INJECT_ERROR_WORD = 2, RIBN_B200_INJECT_BAD_ROW = 3 };
RIBN_B200_API int ribn_b200_debug_inject(ribn_b200_executor* executor, int32_t kind, int32_t value);
/* Launches one small kernel whose only thread waits, through the kernels' bounded wait, on a barrier that
 * nothing completes; after `spin_limit` polls (1 .. 2^20) the wait gives up, writes code 99 to the
 * executor's error word and the kernel returns.  The call waits for the kernel and returns OK: the
 * context stays usable.  The next poll() of a submission reports the expired wait and faults the
 * executor.  No reference counterpart (its kernels do not wait on one another). */
RIBN_B200_API int ribn_b200_debug_wait_expiry(ribn_b200_executor* executor, uint32_t spin_limit);

/* ---- single operators (host pointers in, host pointers out) ------------- */
/* Each runs the same device kernels the executor uses, on `device`, and is
 * what the per-primitive parity tests call.  They replace the operator
 * wrappers of crates/nvidia/src/quantized.rs and crates/nvidia/src/model_ops.rs. */

/* Diagnostic of the calling thread's last failed ribn_b200_op_* call (the CUDA error and the step that
 * raised it).  Returns the message length; copies at most capacity - 1 bytes plus a terminator.
 * The operator wrappers of the reference return the same information as their Err value. */
RIBN_B200_API size_t ribn_b200_op_last_error(char* buffer, size_t capacity);

/* dequantize_block over `rows x cols` (crates/gguf/src/lib.rs:508-535), bit-exact. */
RIBN_B200_API int ribn_b200_op_dequantize(int32_t device, int32_t ggml_type, const void* bytes,
                                          int64_t rows, int64_t cols, float* out);
/* The same decode, but FROM the tile-major packed form that the tensor-core kernels stream (`packed` =
 * output of ribn_b200_debug_repack), through the weight decoder of the decode-and-split tcgen05 kernel.
 * Must equal dequantize_block bit for bit: the repack is judged only by the values it decodes to. */
RIBN_B200_API int ribn_b200_debug_unpack(int32_t device, int32_t ggml_type, const void* packed,
                                         int64_t rows, int64_t cols, float* out);
/* q4_k_embedding(_batch) and its Q8_0 / Q6_K forms (crates/nvidia/src/kernels/quantized/q4_k.cu:1-60):
 * out[i][:] = dequantised row tokens[i] of the raw-layout `[vocab][hidden]` table, bit-exact. */
RIBN_B200_API int ribn_b200_op_embedding(int32_t device, int32_t ggml_type, const void* table, int32_t vocab,
                                         int32_t hidden, const uint32_t* tokens, int32_t count, float* out);
/* y[m][n] = sum_k deq(W[n][k]) x[m][k] (CudaQuantizedGemv::execute_warp /
 * gemv_batch, crates/nvidia/src/quantized.rs:303-436).  variant 0 = fast
 * GEMV kernels (members in pairs), 1 = one-warp-per-row reference kernels,
 * 2 = the batched integer tensor-core kernel (up to 64 members per launch),
 * 3 = the tcgen05 / tensor-memory kernels (K-quant integer form for Q4_K / Q6_K,
 * decode-and-split form for Q8_0), 4 = the decode-and-split form for every type,
 * 5 = the K-quant form over operands converted once (what RIBN_B200_FLAG_OPERAND_CACHE
 * runs; Q4_K / Q6_K only; bit-identical to variant 3). */
RIBN_B200_API int ribn_b200_op_gemv(int32_t device, int32_t ggml_type, const void* weights,
                                    int64_t rows, int64_t cols, const float* x, int32_t members,
                                    float* y, int32_t variant);
/* rms_norm(_batch) (crates/nvidia/src/model_ops.rs:108-201). */
RIBN_B200_API int ribn_b200_op_rms_norm(int32_t device, const float* x, const float* weight,
                                        int32_t members, int32_t length, float eps, float* out);
/* Decode steps of a Gated-DeltaNet recurrent layer behind its projections (the Qwen3.5 hybrid model's
 * linear-attention layers), for `members` sequences each with its own state and `tokens` consecutive tokens per
 * sequence (1: a decode step; more: a prefill chunk, advanced token by token inside the kernel with the state
 * in registers, bit for bit what that many single steps give; rows below = members * tokens, member-major): scalar gates, depth-4 causal
 * convolution + SiLU with history shift, l2-normalised q / k heads tiled over the value heads, the per-head
 * state update and read, and the gated norm.  Replaces the reference's gdn_scalar_gate, gdn_conv_silu,
 * l2_norm_heads, gdn_state_update and gdn_gated_norm launches (crates/nvidia/src/model_ops.rs:372-394,
 * 614-820, 983-1040; host equations crates/nvidia/src/qwen_reference.rs:202-278).  Host pointers:
 * qkv [rows][(2 k_heads + v_heads) * head_dim], z [rows][v_heads * head_dim], beta_raw / alpha_raw
 * [rows][v_heads], dt_bias / a [v_heads], conv_weight [channels][4] (tap fastest), norm_weight
 * [head_dim]; conv_state [members][channels][3] (oldest first) and state [members][v_heads][head_dim]
 * [head_dim] (row major) are updated in place.  Outputs: out [rows][v_heads * head_dim] (what the
 * output projection reads) and, when not NULL, decay, beta [rows][v_heads], conv_act
 * [rows][channels], attn_out [rows][v_heads * head_dim] (before the gated norm).  head_dim 64 or 128.
 * The reference's chunk-parallel scan (gdn_chunk_scan: another summation order) and the hybrid model's executor
 * are not part of this library. */
RIBN_B200_API int ribn_b200_op_gdn_step(int32_t device, int32_t members, int32_t tokens, int32_t k_heads,
                                        int32_t v_heads, int32_t head_dim, const float* qkv, const float* z,
                                        const float* beta_raw, const float* alpha_raw, const float* dt_bias,
                                        const float* a, const float* conv_weight, const float* norm_weight,
                                        float* conv_state, float* state, float l2_eps, float norm_eps,
                                        float* decay, float* beta, float* conv_act, float* attn_out, float* out);
/* Output gate of the gated full-attention layers: out[r][h][i] = attn[r][h][i] * sigmoid(gate), the gate being
 * the second half of head h's [q | gate] projection q_gate[r][h][2 * head_dim]
 * (crates/nvidia/src/model_ops.rs:463-473, crates/nvidia/src/qwen_reference.rs:386-392, 462-472). */
RIBN_B200_API int ribn_b200_op_attention_gate(int32_t device, const float* attn, const float* q_gate, int64_t rows,
                                              int32_t heads, int32_t head_dim, float* out);
/* silu_mul (model_ops.rs:318-330). */
RIBN_B200_API int ribn_b200_op_silu_mul(int32_t device, const float* gate, const float* up,
                                        int64_t length, float* out);
/* argmax(_batch) (model_ops.rs:203-316): lowest index on ties, NaN skipped. */
RIBN_B200_API int ribn_b200_op_argmax(int32_t device, const float* logits, int32_t members,
                                      int64_t length, uint32_t* out);
/* rope_neox(_batch) (model_ops.rs:395-425, 1178-1211): in place on
 * `[members][heads][head_dim]`, one position per member. */
RIBN_B200_API int ribn_b200_op_rope_neox(int32_t device, float* values, const int64_t* positions,
                                         int32_t members, int32_t heads, int32_t head_dim,
                                         int32_t rot_dims, float base);
/* f32_to_f16_bits as used by kv_append_f16 (model_ops.rs:1213-1277). */
RIBN_B200_API int ribn_b200_op_f32_to_f16(int32_t device, const float* in, int64_t length,
                                          uint16_t* out);
/* attn_score_gqa_paged without the Qwen3.5 output gate (model_ops.rs:441-589):
 * `rows` consecutive query positions of one sequence whose cache holds
 * `tokens` keys; row r attends tokens - rows + 1 + r keys.  K/V are F16
 * `[physical_token][kv_head][head_dim]`, `page_table[logical / page_tokens]`
 * gives the physical page.  window = 0 means full causal attention;
 * variant as in op_gemv. */
RIBN_B200_API int ribn_b200_op_attention(int32_t device, const float* q, const uint16_t* keys,
                                         const uint16_t* values, const int32_t* page_table,
                                         int32_t page_tokens, int32_t physical_tokens,
                                         int32_t tokens, int32_t rows, int32_t q_heads,
                                         int32_t kv_heads, int32_t head_dim, int32_t window,
                                         float* out, int32_t variant);
/* strided_rms_norm + rope_neox + kv_append_f16 for every token of a step (model_ops.rs:662, 395-425,
 * 1258-1277): per-head RMSNorm of q `[tokens][q_heads][head_dim]` and k `[tokens][kv_heads][head_dim]`
 * with the shared `[head_dim]` weights, full-width NeoX rotary at positions[t] (both in place), then the
 * F16 (round-to-nearest-even) append of k and v at row kv_slots[t] of the `[physical_tokens][kv_heads][head_dim]`
 * caches. */
RIBN_B200_API int ribn_b200_op_qk_norm_rope_append(int32_t device, float* q, float* k, const float* v,
                                                   const float* q_norm, const float* k_norm,
                                                   const int32_t* positions, const int32_t* kv_slots,
                                                   int32_t tokens, int32_t q_heads, int32_t kv_heads,
                                                   int32_t head_dim, float rope_base, float eps,
                                                   uint16_t* cache_k, uint16_t* cache_v, int32_t physical_tokens);
/* The decode step's fused form of the above plus attention (one new token per sequence): raw q / k / v
 * projections of `members` sequences, token m at positions[m] of sequence m, whose page-table row is
 * page_tables[m][..].  Normalises and rotates q and k, appends k and v to the caches (updated in place on
 * return) and attends keys [0, positions[m]].  out is `[members][q_heads * head_dim]`.
 * Replaces the member-by-member sequence of BatchStates::attend
 * (crates/nvidia/src/decode/member_state.rs:194-324). */
RIBN_B200_API int ribn_b200_op_attention_decode(int32_t device, const float* q, const float* k, const float* v,
                                                const float* q_norm, const float* k_norm, float rope_base,
                                                float eps, uint16_t* cache_k, uint16_t* cache_v,
                                                int32_t physical_tokens, const int32_t* page_tables,
                                                int32_t pages_per_sequence, const int32_t* positions,
                                                int32_t members, int32_t q_heads, int32_t kv_heads,
                                                int32_t head_dim, float* out);
/* Ragged batch metadata built on the device from per-row (prefix, tokens)
 * records: cu_seqlens[rows + 1], and per token its row, position and physical
 * KV slot.  Supersedes the host-built DescriptorPacket
 * (crates/nvidia/src/member_descriptor.rs:6-108). */
RIBN_B200_API int ribn_b200_op_batch_metadata(int32_t device, const int32_t* row_slot,
                                              const int32_t* row_prefix, const int32_t* row_tokens,
                                              int32_t rows, const int32_t* page_tables,
                                              int32_t pages_per_sequence, int32_t page_tokens,
                                              int32_t* cu_seqlens, int32_t* token_row,
                                              int32_t* token_position, int32_t* token_kv_slot);

/* Paged split-KV attention for callers that cannot allocate device memory (code running while a
 * stream is being captured, or under a start-up-only allocation policy).  It has no counterpart
 * in the reference.  Same arithmetic as ribn_b200_op_attention, but every pointer is a DEVICE
 * pointer supplied by the caller, the work is enqueued on `stream` (a cudaStream_t), and the
 * per-span scratch is an 8 MiB array built into the library, so the call performs no cudaMalloc,
 * cudaFree or allocating library routine.  `token_pos[r]` is the position of query row r (it
 * attends keys [0, token_pos[r]], or the last `window` of them); `max_tokens` is 1 + the largest
 * position.  That is a hard precondition the host cannot check (the positions live on the device):
 * a position >= max_tokens makes the merge read span slots no block wrote.  The launch is made with
 * `device` current; the caller's current device is restored before the call returns.  Refused with a message when rows * q_heads * ceil(keys / 64) * (head_dim + 2)
 * exceeds 2 Mi floats.  Calls share the scratch: do not let two of them overlap on the GPU.
 * The first call on a device resolves the scratch address; make it before any stream capture. */
RIBN_B200_API int ribn_b200_attention_noalloc(int32_t device, void* stream, const float* q,
                                              const uint16_t* keys, const uint16_t* values,
                                              const int32_t* page_table, const int32_t* token_pos,
                                              int32_t rows, int32_t max_tokens, int32_t q_heads,
                                              int32_t kv_heads, int32_t head_dim, int32_t window,
                                              float* out, char* error, size_t error_capacity);

/* Host-side tile-major repack used by finalize (no device work): writes the
 * packed form of raw GGUF rows and returns its size; `out` may be NULL to
 * query the size.  No reference counterpart: the reference uploads GGUF bytes
 * verbatim (crates/nvidia/src/cuda.rs:320-387). */
RIBN_B200_API int ribn_b200_debug_repack(int32_t ggml_type, const void* raw, int64_t rows, int64_t cols,
                                         void* out, size_t capacity, size_t* byte_count);

/* Library build identification (git-free; the CUDA arch it was built for). */
RIBN_B200_API const char* ribn_b200_build_info(void);

#ifdef __cplusplus
}
#endif
#endif /* RIBN_B200_H */
