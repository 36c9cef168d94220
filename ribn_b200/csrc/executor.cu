// The executor behind the C ABI: model plan, paged KV arena, admission,
// prepare / submit / poll, and the per-step launch sequence.
//
// Protocol semantics follow QwenExecution (crates/qwen/src/execution.rs) and
// the GenerationExecutor contract (crates/runtime/src/executor.rs:171-254).
// The device side is new: one ragged batch of T tokens (decode rows and
// prefill chunks together) flows through every layer in a single launch
// sequence, with the batch metadata built on the device from 32-byte row
// records, instead of the reference's one-launch-sequence-per-member decode
// (crates/nvidia/src/decode.rs:550-640, 2161-2334).
#include "executor.h"

#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <thread>

#include "blocks.cuh"

using namespace ribn;

namespace {

constexpr size_t kMaxError = 4096;  // ExecutionError bound, crates/runtime/src/executor.rs:134-152

int fail(ribn_b200_executor* ex, const char* fmt, ...) {
    char buf[kMaxError];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    ex->error = buf;
    return RIBN_B200_ERROR;
}

int soft(ribn_b200_executor* ex, int code, const char* fmt, ...) {
    char buf[kMaxError];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    ex->error = buf;
    return code;
}

#define CU_TRY(ex, expr)                                                                       \
    do {                                                                                       \
        cudaError_t e_ = (expr);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            (ex)->faulted = true;                                                              \
            return fail((ex), "CUDA error %s at %s:%d (%s)", cudaGetErrorString(e_), __FILE__, \
                        __LINE__, #expr);                                                      \
        }                                                                                      \
    } while (0)

template <typename T>
cudaError_t dev_alloc(ribn_b200_executor* ex, T** out, size_t count) {
    void* p = nullptr;
    if (ex->inject_alloc_failures > 0) {  // host-side fault injection: the allocator refuses
        --ex->inject_alloc_failures;
        return cudaErrorMemoryAllocation;
    }
    cudaError_t e = cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T));
    if (e == cudaSuccess) {
        ex->allocations.push_back(p);
        *out = (T*)p;
    }
    return e;
}

const char* kLayerNames[kLayerTensors] = {
    "attn_norm.weight", "attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_q_norm.weight",
    "attn_k_norm.weight", "attn_output.weight", "ffn_norm.weight", "ffn_gate.weight", "ffn_up.weight",
    "ffn_down.weight"};

Tensor* find_tensor(ribn_b200_executor* ex, const char* name) {
    if (!strcmp(name, "token_embd.weight")) return &ex->token_embd;
    if (!strcmp(name, "output_norm.weight")) return &ex->output_norm;
    if (!strcmp(name, "output.weight")) return &ex->output;
    int layer = -1;
    char rest[64];
    if (sscanf(name, "blk.%d.%63s", &layer, rest) != 2 || layer < 0 || layer >= ex->cfg.layers) return nullptr;
    for (int i = 0; i < kLayerTensors; ++i) {
        if (!strcmp(rest, kLayerNames[i])) return &ex->lt(layer, i);
    }
    return nullptr;
}

// Expected (rows, cols) of every tensor of the dense-Qwen3 plan.
void expected_shape(const ribn_b200_config& c, int which, long long* rows, long long* cols) {
    const long long H = c.hidden, QD = (long long)c.q_heads * c.head_dim, KD = (long long)c.kv_heads * c.head_dim,
                    F = c.ffn;
    switch (which) {
        case kAttnNorm: case kFfnNorm: *rows = 1; *cols = H; break;
        case kAttnQ: *rows = QD; *cols = H; break;
        case kAttnK: case kAttnV: *rows = KD; *cols = H; break;
        case kAttnQNorm: case kAttnKNorm: *rows = 1; *cols = c.head_dim; break;
        case kAttnOutput: *rows = H; *cols = QD; break;
        case kFfnGate: case kFfnUp: *rows = F; *cols = H; break;
        case kFfnDown: *rows = H; *cols = F; break;
    }
}

bool is_norm(int which) {
    return which == kAttnNorm || which == kFfnNorm || which == kAttnQNorm || which == kAttnKNorm;
}

int set_tensor_storage(ribn_b200_executor* ex, Tensor* t, int type, long long rows, long long cols) {
    const int elems = block_elems(type);
    if (elems == 0 || rows <= 0 || cols <= 0 || cols % elems != 0) {
        return fail(ex, "tensor type %d with shape [%lld, %lld] is not supported", type, rows, cols);
    }
    const size_t bytes = (size_t)rows * (size_t)(cols / elems) * (size_t)block_bytes(type);
    if (t->raw == nullptr || t->bytes != bytes) {
        // A replaced tensor's old storage stays owned by the executor until destroy.
        CU_TRY(ex, dev_alloc(ex, &t->raw, bytes));
    }
    t->type = type;
    t->rows = rows;
    t->cols = cols;
    t->bytes = bytes;
    t->packed = PackedMatrix{};
    return RIBN_B200_OK;
}

int check_open(ribn_b200_executor* ex) {
    if (ex == nullptr) return RIBN_B200_ERROR;
    if (ex->faulted) return fail(ex, "executor is faulted");
    return RIBN_B200_OK;
}

// ---- tensor parallelism: which part of a whole tensor a rank keeps -----------------------------------------
constexpr int kRoleEmbedding = 100, kRoleOutputNorm = 101, kRoleOutput = 102;

int role_from_name(const char* name) {
    if (name == nullptr) return -1;
    if (!strcmp(name, "token_embd.weight")) return kRoleEmbedding;
    if (!strcmp(name, "output_norm.weight")) return kRoleOutputNorm;
    if (!strcmp(name, "output.weight")) return kRoleOutput;
    int layer = -1;
    char rest[64];
    if (sscanf(name, "blk.%d.%63s", &layer, rest) != 2 || layer < 0) return -1;
    for (int i = 0; i < kLayerTensors; ++i) if (!strcmp(rest, kLayerNames[i])) return i;
    return -1;
}

// The ffn dimension is dealt out in 256-column blocks, the first (blocks % ranks) ranks taking one block more.
void ffn_shard(int ffn, int tp, int rank, int* first, int* count) {
    const int blocks = ffn / 256, base = blocks / tp, rem = blocks % tp;
    *first = (rank * base + std::min(rank, rem)) * 256;
    *count = (base + (rank < rem ? 1 : 0)) * 256;
}

// `full` is the whole model's geometry.  Rows and columns are those of the tensor as stored ([out][in]).
void shard_of(const ribn_b200_config& full, int tp, int rank, int role, long long full_rows, long long full_cols,
              long long* r0, long long* nr, long long* c0, long long* nc) {
    *r0 = 0; *nr = full_rows; *c0 = 0; *nc = full_cols;
    if (tp <= 1) return;
    const long long qd = (long long)(full.q_heads / tp) * full.head_dim, kd = (long long)(full.kv_heads / tp) * full.head_dim;
    int f0 = 0, fn = 0;
    ffn_shard(full.ffn, tp, rank, &f0, &fn);
    switch (role) {
        case kAttnQ: *r0 = rank * qd; *nr = qd; break;                  // by query head
        case kAttnK: case kAttnV: *r0 = rank * kd; *nr = kd; break;    // by kv head
        case kFfnGate: case kFfnUp: *r0 = f0; *nr = fn; break;         // by output column
        case kAttnOutput: *c0 = rank * qd; *nc = qd; break;            // along K: the heads this rank attends
        case kFfnDown: *c0 = f0; *nc = fn; break;                      // along K: this rank's ffn columns
        default: break;                                                // norms, embedding, output head: replicated
    }
}

bool load_nccl(NcclApi& api, const char* path, std::string& why) {
    if (api.handle != nullptr) return true;
    void* h = dlopen(path != nullptr && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) { why = std::string("cannot load the NCCL library: ") + dlerror(); return false; }
    api.get_unique_id = (int (*)(void*))dlsym(h, "ncclGetUniqueId");
    api.comm_init_rank = (int (*)(void**, int, ribn_b200_nccl_id, int))dlsym(h, "ncclCommInitRank");
    api.all_reduce = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t))dlsym(h, "ncclAllReduce");
    api.comm_destroy = (int (*)(void*))dlsym(h, "ncclCommDestroy");
    api.get_error_string = (const char* (*)(int))dlsym(h, "ncclGetErrorString");
    if (!api.get_unique_id || !api.comm_init_rank || !api.all_reduce || !api.comm_destroy || !api.get_error_string) {
        why = "the NCCL library lacks an expected entry point";
        return false;
    }
    api.handle = h;
    return true;
}

int pages_for(uint32_t tokens) { return (int)((tokens + kPageTokens - 1) / kPageTokens); }

// ---------------------------------------------------------------------------
// the step
// ---------------------------------------------------------------------------
struct StepPlan {
    int n_rows = 0, n_tokens = 0, n_sample = 0, n_prompt_tokens = 0;
    int max_keys = 0;  // longest prefix + tokens of any row
    int run_first = -1, run_count = 0;  // the longest row's tokens: consecutive positions of one sequence (a prefill chunk)
};

#define STEP_TRY(expr)                          \
    do {                                        \
        cudaError_t e_ = (expr);                \
        if (e_ != cudaSuccess) return e_;       \
        ++launches;                             \
    } while (0)

// Tensor parallelism: the ranks' partial sums `proj` [tokens][hidden] meet in one NCCL all-reduce(sum) on the
// executor's stream, then join the residual stream.
cudaError_t tp_reduce_add(ribn_b200_executor* ex, int tokens, int& launches) {
    constexpr int kNcclFloat = 7, kNcclSum = 0;
    const size_t count = (size_t)tokens * ex->cfg.hidden;
    if (ex->nccl.all_reduce(ex->proj, ex->proj, count, kNcclFloat, kNcclSum, ex->comm, ex->stream) != 0) {
        return cudaErrorUnknown;
    }
    ++launches;
    cudaError_t e = launch_residual_add(ex->stream, ex->hidden, ex->proj, (long long)count);
    if (e == cudaSuccess) ++launches;
    return e;
}

// ---- reference family: plain kernels over raw GGUF blocks, any number of tokens ----------
cudaError_t run_layers_reference(ribn_b200_executor* ex, const StepPlan& plan, int& launches) {
    const ribn_b200_config& c = ex->cfg;
    cudaStream_t s = ex->stream;
    const int T = plan.n_tokens;
    const bool plain_attention = (c.flags & RIBN_B200_FLAG_REFERENCE_KERNELS) != 0;
    for (int l = 0; l < c.layers; ++l) {
        Tensor* t = &ex->lt(l, 0);
        STEP_TRY(launch_rms_norm(s, ex->hidden, (const float*)t[kAttnNorm].raw, T, c.hidden, c.rms_eps, ex->normed));
        STEP_TRY(launch_gemv_ref(s, t[kAttnQ].type, t[kAttnQ].raw, t[kAttnQ].rows, c.hidden, ex->normed, T, ex->q, false));
        STEP_TRY(launch_gemv_ref(s, t[kAttnK].type, t[kAttnK].raw, t[kAttnK].rows, c.hidden, ex->normed, T, ex->k, false));
        STEP_TRY(launch_gemv_ref(s, t[kAttnV].type, t[kAttnV].raw, t[kAttnV].rows, c.hidden, ex->normed, T, ex->v, false));
        __half* ck = ex->cache_k + (long long)l * ex->layer_stride;
        __half* cv = ex->cache_v + (long long)l * ex->layer_stride;
        STEP_TRY(launch_qk_norm_rope_append(s, ex->q, ex->k, ex->v, (const float*)t[kAttnQNorm].raw,
                                            (const float*)t[kAttnKNorm].raw, ex->inv_freq, ex->meta.token_pos,
                                            ex->meta.token_slot, T, c.q_heads, c.kv_heads, c.head_dim, c.rms_eps,
                                            ck, cv));
        if (plain_attention) {
            STEP_TRY(launch_attention_ref(s, ex->q, ck, cv, ex->d_page_tables, ex->pages_per_sequence,
                                          ex->meta.token_seq, ex->meta.token_pos, T, c.q_heads, c.kv_heads,
                                          c.head_dim, 0, ex->attn));
        } else {
            cudaError_t e = launch_attention(s, ex->q, ck, cv, ex->d_page_tables, ex->pages_per_sequence,
                                             ex->meta.token_seq, ex->meta.token_pos, T, c.q_heads, c.kv_heads,
                                             c.head_dim, 0, plan.max_keys, ex->scratch.attn_partial,
                                             ex->scratch.attn_partial_bytes, ex->attn, &launches, plan.run_first, plan.run_count);
            if (e != cudaSuccess) return e;
        }
        if (ex->tp > 1) {
            STEP_TRY(launch_gemv_ref(s, t[kAttnOutput].type, t[kAttnOutput].raw, c.hidden, t[kAttnOutput].cols, ex->attn, T,
                                     ex->proj, false));
            cudaError_t e = tp_reduce_add(ex, T, launches);
            if (e != cudaSuccess) return e;
        } else {
            STEP_TRY(launch_gemv_ref(s, t[kAttnOutput].type, t[kAttnOutput].raw, c.hidden, t[kAttnOutput].cols, ex->attn, T,
                                     ex->hidden, true));
        }
        STEP_TRY(launch_rms_norm(s, ex->hidden, (const float*)t[kFfnNorm].raw, T, c.hidden, c.rms_eps, ex->normed));
        STEP_TRY(launch_gemv_ref(s, t[kFfnGate].type, t[kFfnGate].raw, c.ffn, c.hidden, ex->normed, T, ex->gate, false));
        STEP_TRY(launch_gemv_ref(s, t[kFfnUp].type, t[kFfnUp].raw, c.ffn, c.hidden, ex->normed, T, ex->up, false));
        STEP_TRY(launch_silu_mul(s, ex->gate, ex->up, (long long)T * c.ffn, ex->gate));
        if (ex->tp > 1) {
            STEP_TRY(launch_gemv_ref(s, t[kFfnDown].type, t[kFfnDown].raw, c.hidden, c.ffn, ex->gate, T, ex->proj, false));
            cudaError_t e = tp_reduce_add(ex, T, launches);
            if (e != cudaSuccess) return e;
        } else {
            STEP_TRY(launch_gemv_ref(s, t[kFfnDown].type, t[kFfnDown].raw, c.hidden, c.ffn, ex->gate, T, ex->hidden, true));
        }
    }
    if (plan.n_sample > 0) {
        // Only sampling rows reach the head (crates/nvidia/src/decode.rs:686-704).
        STEP_TRY(launch_rms_norm_gather(s, ex->hidden, ex->meta.sample_token, (const float*)ex->output_norm.raw,
                                        plan.n_sample, c.hidden, c.rms_eps, ex->head_in));
        STEP_TRY(launch_gemv_ref(s, ex->output.type, ex->output.raw, ex->output.rows, ex->output.cols, ex->head_in,
                                 plan.n_sample, ex->logits, false));
    }
    return cudaSuccess;
}

// ---- decode family: tensor-core GEMV chain over operand-form activations (<= 2 tokens) ---------
GemvSegment segment_of(const Tensor& t, float* y) {
    return GemvSegment{t.packed.data, t.type, (int)t.rows, t.packed.row_tiles, y};
}

// The decode step's projections as GEMV arguments (T = 1 or 2 rows).
GemvArgs base_args(ribn_b200_executor* ex, int T) {
    GemvArgs a{};
    a.members = T;
    a.eps = ex->cfg.rms_eps;
    a.error_flag = ex->d_error;
    return a;
}
// q | k | v from the normalised residual stream
GemvArgs qkv_args(ribn_b200_executor* ex, int l, int T) {
    Tensor* t = &ex->lt(l, 0);
    GemvArgs a = base_args(ex, T);
    a.n_segments = 3;
    a.seg[0] = segment_of(t[kAttnQ], ex->q);
    a.seg[1] = segment_of(t[kAttnK], ex->k);
    a.seg[2] = segment_of(t[kAttnV], ex->v);
    a.k = ex->cfg.hidden;
    a.in = ex->op_hidden;
    a.in_has_norm = 1;
    a.epilogue = kStore;
    return a;
}
// attention output projection, residual add, operand form of ffn_norm(hidden)
GemvArgs o_args(ribn_b200_executor* ex, int l, int T) {
    Tensor* t = &ex->lt(l, 0);
    GemvArgs a = base_args(ex, T);
    a.n_segments = 1;
    a.seg[0] = segment_of(t[kAttnOutput], ex->tp > 1 ? ex->proj : ex->hidden);
    a.k = ex->cfg.q_heads * ex->cfg.head_dim;
    a.in = ex->op_attn;
    a.in_has_norm = 0;
    if (ex->tp > 1) {
        a.epilogue = kStore;   // tensor parallel: a partial sum for the all-reduce; the operand form follows it
    } else {
        a.epilogue = kResidual;
        a.out = ex->op_hidden;
        a.out_norm_weight = (const float*)t[kFfnNorm].raw;
    }
    return a;
}
// gate | up with the SwiGLU epilogue, operand form of the gated product
GemvArgs gate_up_args(ribn_b200_executor* ex, int l, int T) {
    Tensor* t = &ex->lt(l, 0);
    GemvArgs a = base_args(ex, T);
    a.n_segments = 2;
    a.seg[0] = segment_of(t[kFfnGate], ex->gate);
    a.seg[1] = segment_of(t[kFfnUp], ex->up);
    a.k = ex->cfg.hidden;
    a.in = ex->op_hidden;
    a.in_has_norm = 1;
    a.epilogue = kSwiGLU;
    a.out = ex->op_act;
    return a;
}
// down projection, residual add, operand form of the next norm (next layer's or the output norm)
GemvArgs down_args(ribn_b200_executor* ex, int l, int T) {
    const ribn_b200_config& c = ex->cfg;
    Tensor* t = &ex->lt(l, 0);
    GemvArgs a = base_args(ex, T);
    a.n_segments = 1;
    a.seg[0] = segment_of(t[kFfnDown], ex->tp > 1 ? ex->proj : ex->hidden);
    a.k = c.ffn;
    a.in = ex->op_act;
    a.in_has_norm = 0;
    if (ex->tp > 1) {
        a.epilogue = kStore;
    } else {
        a.epilogue = kResidual;
        a.out = ex->op_hidden;
        a.out_norm_weight = l + 1 < c.layers ? (const float*)ex->lt(l + 1, kAttnNorm).raw : (const float*)ex->output_norm.raw;
    }
    return a;
}
// output head over `rows` already normalised rows
GemvArgs head_args(ribn_b200_executor* ex, int rows, const ActOperand& in) {
    GemvArgs a = base_args(ex, rows);
    a.n_segments = 1;
    a.seg[0] = segment_of(ex->output, ex->logits);
    a.k = ex->cfg.hidden;
    a.in = in;
    a.in_has_norm = 1;
    a.epilogue = kStore;
    return a;
}

cudaError_t run_layers_decode(ribn_b200_executor* ex, const StepPlan& plan, int& launches) {
    const ribn_b200_config& c = ex->cfg;
    cudaStream_t s = ex->stream;
    const int T = plan.n_tokens;
    const bool pdl = !(c.flags & RIBN_B200_FLAG_NO_GRAPH);
    STEP_TRY(launch_to_operand(s, ex->hidden, nullptr, (const float*)ex->lt(0, kAttnNorm).raw, T, c.hidden,
                               ex->op_hidden));
    STEP_TRY(launch_gemv_mma(s, qkv_args(ex, 0, T), pdl));
    for (int l = 0; l < c.layers; ++l) {
        Tensor* t = &ex->lt(l, 0);
        __half* ck = ex->cache_k + (long long)l * ex->layer_stride;
        __half* cv = ex->cache_v + (long long)l * ex->layer_stride;
        if (plan.n_rows == T && c.head_dim >= 64) {
            // every row adds one token: norm, rotary, cache append, attention and operand form in one pass
            DecodeAttention d{};
            d.q = ex->q; d.k = ex->k; d.v = ex->v;
            d.q_norm = (const float*)t[kAttnQNorm].raw; d.k_norm = (const float*)t[kAttnKNorm].raw;
            d.inv_freq = ex->inv_freq; d.eps = c.rms_eps;
            d.cache_k = ck; d.cache_v = cv;
            d.page_tables = ex->d_page_tables; d.pages_per_sequence = ex->pages_per_sequence;
            d.token_seq = ex->meta.token_seq; d.token_pos = ex->meta.token_pos; d.token_slot = ex->meta.token_slot;
            d.n_tokens = T; d.q_heads = c.q_heads; d.kv_heads = c.kv_heads; d.head_dim = c.head_dim;
            d.window = 0; d.max_keys = plan.max_keys;
            d.partial = ex->scratch.attn_partial; d.partial_bytes = ex->scratch.attn_partial_bytes;
            d.out = ex->attn; d.operand = ex->op_attn;
            d.programmatic = pdl;
            cudaError_t e = launch_attention_decode(s, d, &launches);
            if (e != cudaSuccess) return e;
        } else {
            STEP_TRY(launch_qk_norm_rope_append(s, ex->q, ex->k, ex->v, (const float*)t[kAttnQNorm].raw,
                                                (const float*)t[kAttnKNorm].raw, ex->inv_freq, ex->meta.token_pos,
                                                ex->meta.token_slot, T, c.q_heads, c.kv_heads, c.head_dim,
                                                c.rms_eps, ck, cv));
            cudaError_t e = launch_attention(s, ex->q, ck, cv, ex->d_page_tables, ex->pages_per_sequence,
                                             ex->meta.token_seq, ex->meta.token_pos, T, c.q_heads, c.kv_heads,
                                             c.head_dim, 0, plan.max_keys, ex->scratch.attn_partial,
                                             ex->scratch.attn_partial_bytes, ex->attn, &launches, plan.run_first, plan.run_count);
            if (e != cudaSuccess) return e;
            STEP_TRY(launch_to_operand(s, ex->attn, nullptr, nullptr, T, c.q_heads * c.head_dim, ex->op_attn));
        }
        STEP_TRY(launch_gemv_mma(s, o_args(ex, l, T), pdl));
        if (ex->tp > 1) {
            cudaError_t e = tp_reduce_add(ex, T, launches);
            if (e != cudaSuccess) return e;
            STEP_TRY(launch_to_operand(s, ex->hidden, nullptr, (const float*)t[kFfnNorm].raw, T, c.hidden, ex->op_hidden));
        }
        STEP_TRY(launch_gemv_mma(s, gate_up_args(ex, l, T), pdl));
        STEP_TRY(launch_gemv_mma(s, down_args(ex, l, T), pdl));
        if (ex->tp > 1) {
            cudaError_t e = tp_reduce_add(ex, T, launches);
            if (e != cudaSuccess) return e;
            const float* next_norm = l + 1 < c.layers ? (const float*)ex->lt(l + 1, kAttnNorm).raw : (const float*)ex->output_norm.raw;
            STEP_TRY(launch_to_operand(s, ex->hidden, nullptr, next_norm, T, c.hidden, ex->op_hidden));
        }
        if (l + 1 < c.layers) STEP_TRY(launch_gemv_mma(s, qkv_args(ex, l + 1, T), pdl));
    }
    if (plan.n_sample > 0) {
        ActOperand head = ex->op_hidden;  // already normalised with output_norm
        if (plan.n_sample != T) {
            STEP_TRY(launch_to_operand(s, ex->hidden, ex->meta.sample_token, (const float*)ex->output_norm.raw,
                                       plan.n_sample, c.hidden, ex->op_head));
            head = ex->op_head;
        }
        const GemvArgs a = head_args(ex, plan.n_sample, head);
        STEP_TRY(launch_gemv_mma(s, a, pdl));
    }
    return cudaSuccess;
}

// ---- batch family: integer tensor-core GEMM over batch-operand activations (3+ tokens) --------
// Tokens go through each projection in groups of up to kGemmMaxMembers; weights are read once per group.
cudaError_t batch_project(ribn_b200_executor* ex, int& launches, const float* x, const int32_t* index,
                          const float* norm_weight, int tokens, int k, const Tensor* const* mats, float* const* ys,
                          int n_mats, int epilogue) {
    cudaStream_t s = ex->stream;
    const bool tensor_memory = !(ex->cfg.flags & RIBN_B200_FLAG_NO_TCGEN05);
    GemvSegment probe[3];
    for (int i = 0; i < n_mats; ++i) probe[i] = GemvSegment{nullptr, mats[i]->type, 0, 0, nullptr};
    const bool kquant = tensor_memory && gemm_tc_kquant(probe, n_mats, 1);
    const int group = !tensor_memory ? kGemmMaxMembers : kquant ? 64 : kGemmTcMaxMembers;
    // K-quant form: one conversion of every row of the step, laid out as one operand per group
    const bool converted = kquant && tokens > group;
    if (converted) {
        cudaError_t e = launch_to_tc_operand_groups(s, x, index, norm_weight, tokens, group, k, ex->cfg.rms_eps, ex->op_tc);
        if (e != cudaSuccess) return e;
        launches += 1;
    }
    // ... and its whole groups in one launch: a weight tile then meets every group while it is in L2
    const int fused_groups = converted ? tokens / group : 0;
    for (int base = 0; base < tokens; base += group) {
        const bool fused = fused_groups > 1 && base == 0;
        if (fused_groups > 1 && base > 0 && base < fused_groups * group) continue;  // covered by the fused launch
        const int m = std::min(group, tokens - base);
        GemmArgs a{};
        a.n_segments = n_mats;
        for (int i = 0; i < n_mats; ++i) {
            a.seg[i] = GemvSegment{mats[i]->packed.data, mats[i]->type, (int)mats[i]->rows, mats[i]->packed.row_tiles,
                                   ys[i] + (size_t)base * mats[i]->rows, mats[i]->op_a, mats[i]->op_meta};
        }
        a.k = k;
        a.members = m;
        a.error_flag = ex->d_error;
        if (tensor_memory) {
            // tcgen05 dequant-GEMM; SwiGLU runs as a separate elementwise pass over gate and up
            if (!converted) {
                cudaError_t e = launch_to_tc_operand(s, index ? x : x + (size_t)base * k, index ? index + base : nullptr,
                                                     norm_weight, m, k, ex->cfg.rms_eps, kquant, ex->op_tc);
                if (e != cudaSuccess) return e;
                launches += kquant ? 1 : 2;
                a.chunks = (const signed char*)ex->op_tc.chunks;
                a.member_scale = ex->op_tc.member_scale;
            } else {
                a.chunks = (const signed char*)ex->op_tc.chunks + (size_t)(base / group) * tc_operand_bytes(group, k);
                a.member_scale = ex->op_tc.member_scale + base;
                if (fused) {
                    a.groups = fused_groups;
                    a.group_chunk_bytes = tc_operand_bytes(group, k);
                }
            }
            a.kquant = kquant ? 1 : 0;
            a.partial = ex->tc_partial;
            a.partial_floats = ex->tc_partial_floats;
            a.epilogue = epilogue == kSwiGLU ? kStore : epilogue;
            STEP_TRY(launch_gemm_tc(s, a));
            launches += gemm_tc_last_launches() - 1;
            if (epilogue == kSwiGLU) {
                float* gate = ys[0] + (size_t)base * mats[0]->rows;
                float* up = ys[1] + (size_t)base * mats[1]->rows;
                const long long rows_done = fused ? (long long)fused_groups * group : m;
                STEP_TRY(launch_silu_mul(s, gate, up, rows_done * mats[0]->rows, gate));
            }
        } else {
            cudaError_t e = launch_to_batch_operand(s, index ? x : x + (size_t)base * k, index ? index + base : nullptr,
                                                    norm_weight, m, k, ex->cfg.rms_eps, ex->op_batch);
            if (e != cudaSuccess) return e;
            launches += 2;
            a.chunks = ex->op_batch.chunks;
            a.member_scale = ex->op_batch.member_scale;
            a.epilogue = epilogue;
            STEP_TRY(launch_gemm_imma(s, a));
        }
    }
    return cudaSuccess;
}

cudaError_t run_layers_batch(ribn_b200_executor* ex, const StepPlan& plan, int& launches) {
    const ribn_b200_config& c = ex->cfg;
    cudaStream_t s = ex->stream;
    const int T = plan.n_tokens;
    const int QD = c.q_heads * c.head_dim;
    for (int l = 0; l < c.layers; ++l) {
        Tensor* t = &ex->lt(l, 0);
        {
            const Tensor* mats[3] = {&t[kAttnQ], &t[kAttnK], &t[kAttnV]};
            float* ys[3] = {ex->q, ex->k, ex->v};
            cudaError_t e = batch_project(ex, launches, ex->hidden, nullptr, (const float*)t[kAttnNorm].raw, T, c.hidden,
                                          mats, ys, 3, kStore);
            if (e != cudaSuccess) return e;
        }
        __half* ck = ex->cache_k + (long long)l * ex->layer_stride;
        __half* cv = ex->cache_v + (long long)l * ex->layer_stride;
        if (plan.n_rows == T && c.head_dim >= 64) {
            DecodeAttention d{};
            d.q = ex->q; d.k = ex->k; d.v = ex->v;
            d.q_norm = (const float*)t[kAttnQNorm].raw; d.k_norm = (const float*)t[kAttnKNorm].raw;
            d.inv_freq = ex->inv_freq; d.eps = c.rms_eps;
            d.cache_k = ck; d.cache_v = cv;
            d.page_tables = ex->d_page_tables; d.pages_per_sequence = ex->pages_per_sequence;
            d.token_seq = ex->meta.token_seq; d.token_pos = ex->meta.token_pos; d.token_slot = ex->meta.token_slot;
            d.n_tokens = T; d.q_heads = c.q_heads; d.kv_heads = c.kv_heads; d.head_dim = c.head_dim;
            d.window = 0; d.max_keys = plan.max_keys;
            d.partial = ex->scratch.attn_partial; d.partial_bytes = ex->scratch.attn_partial_bytes;
            d.out = ex->attn;
            d.programmatic = false;
            cudaError_t e = launch_attention_decode(s, d, &launches);
            if (e != cudaSuccess) return e;
        } else {
            STEP_TRY(launch_qk_norm_rope_append(s, ex->q, ex->k, ex->v, (const float*)t[kAttnQNorm].raw,
                                                (const float*)t[kAttnKNorm].raw, ex->inv_freq, ex->meta.token_pos,
                                                ex->meta.token_slot, T, c.q_heads, c.kv_heads, c.head_dim,
                                                c.rms_eps, ck, cv));
            cudaError_t e = launch_attention(s, ex->q, ck, cv, ex->d_page_tables, ex->pages_per_sequence,
                                             ex->meta.token_seq, ex->meta.token_pos, T, c.q_heads, c.kv_heads,
                                             c.head_dim, 0, plan.max_keys, ex->scratch.attn_partial,
                                             ex->scratch.attn_partial_bytes, ex->attn, &launches, plan.run_first, plan.run_count);
            if (e != cudaSuccess) return e;
        }
        {
            const Tensor* mats[1] = {&t[kAttnOutput]};
            float* ys[1] = {ex->tp > 1 ? ex->proj : ex->hidden};
            cudaError_t e = batch_project(ex, launches, ex->attn, nullptr, nullptr, T, QD, mats, ys, 1, ex->tp > 1 ? kStore : kResidual);
            if (e == cudaSuccess && ex->tp > 1) e = tp_reduce_add(ex, T, launches);
            if (e != cudaSuccess) return e;
        }
        {
            const Tensor* mats[2] = {&t[kFfnGate], &t[kFfnUp]};
            float* ys[2] = {ex->gate, ex->up};
            cudaError_t e = batch_project(ex, launches, ex->hidden, nullptr, (const float*)t[kFfnNorm].raw, T, c.hidden,
                                          mats, ys, 2, kSwiGLU);
            if (e != cudaSuccess) return e;
        }
        {
            const Tensor* mats[1] = {&t[kFfnDown]};
            float* ys[1] = {ex->tp > 1 ? ex->proj : ex->hidden};
            cudaError_t e = batch_project(ex, launches, ex->gate, nullptr, nullptr, T, c.ffn, mats, ys, 1, ex->tp > 1 ? kStore : kResidual);
            if (e == cudaSuccess && ex->tp > 1) e = tp_reduce_add(ex, T, launches);
            if (e != cudaSuccess) return e;
        }
    }
    if (plan.n_sample > 0) {
        // Only sampling rows reach the head (crates/nvidia/src/decode.rs:686-704).
        const Tensor* mats[1] = {&ex->output};
        float* ys[1] = {ex->logits};
        cudaError_t e = batch_project(ex, launches, ex->hidden, ex->meta.sample_token, (const float*)ex->output_norm.raw,
                                      plan.n_sample, c.hidden, mats, ys, 1, kStore);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

bool packed_family_applies(const ribn_b200_executor* ex) {
    if (ex->cfg.flags & RIBN_B200_FLAG_REFERENCE_KERNELS) return false;
    if (!ex->output.packed.ready()) return false;
    for (const Tensor& t : ex->layer_tensors) {
        if (t.type != kF32 && !t.packed.ready()) return false;
    }
    return true;
}

bool decode_family_applies(const ribn_b200_executor* ex, const StepPlan& plan) {
    return plan.n_tokens <= kGemvMaxMembers && packed_family_applies(ex);
}

cudaError_t run_step(ribn_b200_executor* ex, const StepPlan& plan, int& launches) {
    const ribn_b200_config& c = ex->cfg;
    cudaStream_t s = ex->stream;
    const int T = plan.n_tokens;
    launches = 0;
    STEP_TRY(launch_step_metadata(s, ex->d_rows, plan.n_rows, T, ex->d_tokens, ex->d_next_token,
                                  ex->d_page_tables, ex->pages_per_sequence, ex->meta));
    STEP_TRY(launch_embedding(s, ex->token_embd.type, ex->token_embd.raw, c.hidden, c.vocab, ex->meta.token_id, T,
                              ex->hidden));
    cudaError_t e = decode_family_applies(ex, plan) ? run_layers_decode(ex, plan, launches)
                    : packed_family_applies(ex)     ? run_layers_batch(ex, plan, launches)
                                                    : run_layers_reference(ex, plan, launches);
    if (e != cudaSuccess) return e;
    if (plan.n_sample > 0) {
        STEP_TRY(launch_argmax(s, ex->logits, plan.n_sample, c.vocab, ex->d_sampled, ex->meta.sample_slot,
                               ex->d_next_token));
    }
    return cudaSuccess;
}

}  // namespace

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" {

#define RIBN_STR2(x) #x
#define RIBN_STR(x) RIBN_STR2(x)
const char* ribn_b200_build_info(void) {
    return "ribn_b200 sm_100a cuda " RIBN_STR(__CUDACC_VER_MAJOR__) "." RIBN_STR(__CUDACC_VER_MINOR__);
}

int ribn_b200_create(const ribn_b200_config* config, ribn_b200_executor** out, char* error, size_t error_capacity) {
    auto report = [&](const char* msg) {
        if (error != nullptr && error_capacity > 0) snprintf(error, error_capacity, "%s", msg);
        return RIBN_B200_ERROR;
    };
    if (config == nullptr || out == nullptr) return report("null argument");
    const ribn_b200_config& c = *config;
    if (c.layers <= 0 || c.hidden <= 0 || c.q_heads <= 0 || c.kv_heads <= 0 || c.head_dim <= 0 || c.ffn <= 0 ||
        c.vocab <= 0 || c.q_heads % c.kv_heads != 0) {
        return report("model geometry must be positive and q_heads a multiple of kv_heads");
    }
    if (c.head_dim != 32 && c.head_dim != 64 && c.head_dim != 128 && c.head_dim != 256) {
        return report("head_dim must be 32, 64, 128 or 256");
    }
    // GenerationLimits::validate, crates/runtime/src/executor.rs:53-63
    if (c.context_tokens <= 0 || c.max_sequences <= 0 || c.max_batch_tokens <= 0) {
        return report("prepared model limits must be nonzero");
    }
    if (c.max_sequences > 1024) return report("max_sequences above 1024 is not supported");
    const int tp = c.tp_size > 1 ? c.tp_size : 1;
    if (tp > 1) {
        // heads split by rank; K splits must fall on 256-input block boundaries (K-quant super-blocks)
        if (c.tp_rank < 0 || c.tp_rank >= tp) return report("tp_rank out of range");
        if (c.q_heads % tp != 0 || c.kv_heads % tp != 0) return report("tensor parallelism needs q_heads and kv_heads divisible by tp_size");
        if (((c.q_heads / tp) * c.head_dim) % 256 != 0) return report("tensor parallelism needs (q_heads / tp_size) * head_dim to be a multiple of 256");
        if (c.ffn % 256 != 0 || c.ffn / 256 < tp) return report("tensor parallelism needs ffn to be a multiple of 256 with at least one block per rank");
    }
    if (c.context_tokens > kAttnMaxSpans * kAttnSpanKeys) {
        return report("context_tokens above 65536 is not supported (1024 attention spans of 64 keys)");
    }
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        return report("no CUDA device: this library has no CPU path");
    }
    if (c.device < 0 || c.device >= count) return report("CUDA device ordinal out of range");
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, c.device) != cudaSuccess) return report("cannot query the CUDA device");
    if (prop.major != 10) {
        return report("kernels are built for sm_100a only; this device is not a Blackwell B200-class GPU");
    }
    if (cudaSetDevice(c.device) != cudaSuccess) return report("cannot select the CUDA device");
    auto* ex = new ribn_b200_executor();
    ex->cfg = c;
    ex->full = c;
    ex->tp = tp;
    ex->rank = tp > 1 ? c.tp_rank : 0;
    if (tp > 1) {
        // this rank's shard: the step's kernels see the local geometry
        int count = 0;
        ffn_shard(c.ffn, tp, ex->rank, &ex->ffn_first, &count);
        ex->cfg.q_heads = c.q_heads / tp;
        ex->cfg.kv_heads = c.kv_heads / tp;
        ex->cfg.ffn = count;
    }
    ex->layer_tensors.resize((size_t)c.layers * kLayerTensors);
    if (cudaStreamCreateWithFlags(&ex->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreate(&ex->ev_start) != cudaSuccess || cudaEventCreate(&ex->ev_done) != cudaSuccess) {
        delete ex;
        return report("cannot create CUDA stream/events");
    }
    *out = ex;
    return RIBN_B200_OK;
}

int ribn_b200_destroy(ribn_b200_executor* ex) {
    if (ex == nullptr) return RIBN_B200_OK;
    cudaSetDevice(ex->cfg.device);
    // Never free device memory while completion is uncertain: leak instead
    // (crates/runtime/src/engine.rs:597-607).
    if (cudaStreamSynchronize(ex->stream) != cudaSuccess) return RIBN_B200_ERROR;
    for (auto& g : ex->graphs) cudaGraphExecDestroy(g.second.exec);
    if (ex->comm != nullptr && ex->nccl.comm_destroy != nullptr) ex->nccl.comm_destroy(ex->comm);
    for (void* p : ex->allocations) cudaFree(p);
    if (ex->h_rows) cudaFreeHost(ex->h_rows);
    if (ex->h_tokens) cudaFreeHost(ex->h_tokens);
    if (ex->h_sampled) cudaFreeHost(ex->h_sampled);
    if (ex->h_error) cudaFreeHost(ex->h_error);
    cudaEventDestroy(ex->ev_start);
    cudaEventDestroy(ex->ev_done);
    cudaStreamDestroy(ex->stream);
    delete ex;
    return RIBN_B200_OK;
}

size_t ribn_b200_last_error(ribn_b200_executor* ex, char* buffer, size_t capacity) {
    if (ex == nullptr || buffer == nullptr || capacity == 0) return 0;
    const size_t n = std::min(std::min(ex->error.size(), capacity - 1), kMaxError);
    memcpy(buffer, ex->error.data(), n);
    buffer[n] = 0;
    return n;
}

// Role of a tensor slot of this executor (a LayerTensor index, or one of the kRole* constants).
static int role_of(ribn_b200_executor* ex, const Tensor* t) {
    if (t == &ex->token_embd) return kRoleEmbedding;
    if (t == &ex->output_norm) return kRoleOutputNorm;
    if (t == &ex->output) return kRoleOutput;
    return (int)((t - ex->layer_tensors.data()) % kLayerTensors);
}

// Copies this rank's shard of a whole tensor (`src`: host or device memory holding [rows][cols] blocks) into `t`.
static int store_shard(ribn_b200_executor* ex, Tensor* t, int type, long long rows, long long cols, const unsigned char* src,
                       cudaMemcpyKind kind) {
    long long r0, nr, c0, nc;
    shard_of(ex->full, ex->tp, ex->rank, role_of(ex, t), rows, cols, &r0, &nr, &c0, &nc);
    const int elems = block_elems(type);
    if (elems == 0 || cols % elems != 0 || c0 % elems != 0 || nc % elems != 0) {
        return fail(ex, "tensor type %d with shape [%lld, %lld] cannot be split for this rank", type, rows, cols);
    }
    if (set_tensor_storage(ex, t, type, nr, nc) != RIBN_B200_OK) return RIBN_B200_ERROR;
    const size_t bb = (size_t)block_bytes(type);
    const size_t src_pitch = (size_t)(cols / elems) * bb, dst_pitch = (size_t)(nc / elems) * bb;
    const unsigned char* from = src + (size_t)r0 * src_pitch + (size_t)(c0 / elems) * bb;
    CU_TRY(ex, cudaMemcpy2DAsync(t->raw, dst_pitch, from, src_pitch, dst_pitch, (size_t)nr, kind, ex->stream));
    return RIBN_B200_OK;
}

int ribn_b200_load_tensor(ribn_b200_executor* ex, const char* name, int32_t type, int64_t rows, int64_t cols,
                          const void* bytes, size_t byte_count) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (ex->finalized) return fail(ex, "tensors cannot change after finalize");
    cudaSetDevice(ex->cfg.device);
    Tensor* t = name ? find_tensor(ex, name) : nullptr;
    if (t == nullptr) return fail(ex, "unknown tensor name '%s'", name ? name : "(null)");
    const int elems = block_elems(type);
    if (elems == 0 || rows <= 0 || cols <= 0 || cols % elems != 0) {
        return fail(ex, "tensor type %d with shape [%lld, %lld] is not supported", type, (long long)rows, (long long)cols);
    }
    const size_t whole = (size_t)rows * (size_t)(cols / elems) * (size_t)block_bytes(type);
    if (byte_count != whole || bytes == nullptr) {
        return fail(ex, "tensor '%s' needs %zu encoded bytes, got %zu", name, whole, byte_count);
    }
    // The caller passes the whole tensor; a tensor-parallel rank keeps its shard of it.
    if (store_shard(ex, t, type, rows, cols, (const unsigned char*)bytes, cudaMemcpyHostToDevice) != RIBN_B200_OK) {
        return RIBN_B200_ERROR;
    }
    CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    return RIBN_B200_OK;
}

int ribn_b200_init_synthetic(ribn_b200_executor* ex, uint64_t seed, int32_t scheme) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (ex->finalized) return fail(ex, "tensors cannot change after finalize");
    if (scheme != RIBN_B200_SCHEME_Q8_0 && scheme != RIBN_B200_SCHEME_Q4_K_M) return fail(ex, "unknown scheme");
    cudaSetDevice(ex->cfg.device);
    const ribn_b200_config& c = ex->cfg;
    const int base = scheme == RIBN_B200_SCHEME_Q8_0 ? kQ8_0 : kQ4_K;
    const int wide = scheme == RIBN_B200_SCHEME_Q8_0 ? kQ8_0 : kQ6_K;  // attn_v, ffn_down, output
    uint64_t index = 0;
    // Every rank generates the WHOLE tensor from the same seed (into a scratch buffer when it keeps only a shard),
    // so the shards of a tensor-parallel group are slices of the one-GPU checkpoint with the same seed.
    unsigned char* scratch = nullptr;
    size_t scratch_bytes = 0;
    auto fill = [&](Tensor* t, int type, long long rows, long long cols) -> int {
        const uint64_t tensor_seed = seed * 0x9e3779b97f4a7c15ull + (++index) * 0xd1342543de82ef95ull;
        long long r0, nr, c0, nc;
        shard_of(ex->full, ex->tp, ex->rank, role_of(ex, t), rows, cols, &r0, &nr, &c0, &nc);
        const bool whole = nr == rows && nc == cols;
        unsigned char* target = nullptr;
        if (whole) {
            if (set_tensor_storage(ex, t, type, rows, cols) != RIBN_B200_OK) return RIBN_B200_ERROR;
            target = t->raw;
        } else {
            const size_t need = (size_t)rows * (size_t)(cols / block_elems(type)) * (size_t)block_bytes(type);
            if (need > scratch_bytes) {
                if (scratch != nullptr) { CU_TRY(ex, cudaStreamSynchronize(ex->stream)); cudaFree(scratch); scratch = nullptr; }
                CU_TRY(ex, cudaMalloc((void**)&scratch, need));
                scratch_bytes = need;
            }
            target = scratch;
        }
        if (type == kF32) {
            CU_TRY(ex, launch_fill_f32(ex->stream, (float*)target, rows * cols, 1.0f));
        } else {
            CU_TRY(ex, launch_synth_quantized(ex->stream, type, target, rows, cols, tensor_seed, 0.02f));
        }
        if (!whole && store_shard(ex, t, type, rows, cols, scratch, cudaMemcpyDeviceToDevice) != RIBN_B200_OK) return RIBN_B200_ERROR;
        return RIBN_B200_OK;
    };
    for (int l = 0; l < c.layers; ++l) {
        for (int w = 0; w < kLayerTensors; ++w) {
            long long rows, cols;
            expected_shape(ex->full, w, &rows, &cols);
            int type = is_norm(w) ? kF32 : ((w == kAttnV || w == kFfnDown) ? wide : base);
            if (fill(&ex->lt(l, w), type, rows, cols) != RIBN_B200_OK) return RIBN_B200_ERROR;
        }
    }
    if (fill(&ex->token_embd, base, c.vocab, c.hidden) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (fill(&ex->output_norm, kF32, 1, c.hidden) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (fill(&ex->output, wide, c.vocab, c.hidden) != RIBN_B200_OK) return RIBN_B200_ERROR;
    CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    if (scratch != nullptr) cudaFree(scratch);
    return RIBN_B200_OK;
}

int ribn_b200_read_tensor(ribn_b200_executor* ex, const char* name, int32_t* type, int64_t* rows, int64_t* cols,
                          void* bytes, size_t capacity, size_t* byte_count) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    cudaSetDevice(ex->cfg.device);
    Tensor* t = name ? find_tensor(ex, name) : nullptr;
    if (t == nullptr || !t->loaded()) return fail(ex, "tensor '%s' is not loaded", name ? name : "(null)");
    if (type) *type = t->type;
    if (rows) *rows = t->rows;
    if (cols) *cols = t->cols;
    if (byte_count) *byte_count = t->bytes;
    if (bytes != nullptr) {
        if (capacity < t->bytes) return fail(ex, "buffer too small for tensor '%s'", name);
        CU_TRY(ex, cudaMemcpyAsync(bytes, t->raw, t->bytes, cudaMemcpyDeviceToHost, ex->stream));
        CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    }
    return RIBN_B200_OK;
}

int ribn_b200_finalize(ribn_b200_executor* ex) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (ex->finalized) return fail(ex, "finalize called twice");
    if (ex->tp > 1 && ex->comm == nullptr) return fail(ex, "a tensor-parallel executor must join its group (tp_init) before finalize");
    cudaSetDevice(ex->cfg.device);
    const ribn_b200_config& c = ex->cfg;
    // Model plan validation (validate_model_plan, crates/nvidia/src/decode.rs:364-368).
    for (int l = 0; l < c.layers; ++l) {
        for (int w = 0; w < kLayerTensors; ++w) {
            const Tensor& t = ex->lt(l, w);
            long long rows, cols;
            expected_shape(c, w, &rows, &cols);
            if (!t.loaded()) return fail(ex, "missing tensor blk.%d.%s", l, kLayerNames[w]);
            if (t.rows * t.cols != rows * cols || (!is_norm(w) && (t.rows != rows || t.cols != cols))) {
                return fail(ex, "tensor blk.%d.%s has shape [%lld, %lld], expected [%lld, %lld]", l, kLayerNames[w],
                            t.rows, t.cols, rows, cols);
            }
            if (is_norm(w) ? t.type != kF32 : (t.type != kQ8_0 && t.type != kQ4_K && t.type != kQ6_K)) {
                return fail(ex, "tensor blk.%d.%s has unsupported type %d", l, kLayerNames[w], t.type);
            }
        }
    }
    if (!ex->token_embd.loaded() || ex->token_embd.rows != c.vocab || ex->token_embd.cols != c.hidden) {
        return fail(ex, "token_embd.weight must be [vocab, hidden]");
    }
    if (!ex->output_norm.loaded() || ex->output_norm.type != kF32 || ex->output_norm.rows * ex->output_norm.cols != c.hidden) {
        return fail(ex, "output_norm.weight must be F32 [hidden]");
    }
    if (!ex->output.loaded() || ex->output.rows != c.vocab || ex->output.cols != c.hidden ||
        (ex->output.type != kQ8_0 && ex->output.type != kQ4_K && ex->output.type != kQ6_K)) {
        return fail(ex, "output.weight must be a quantised [vocab, hidden] matrix");
    }

    // Tile-major repack for the tensor-core GEMV.
    if (!(c.flags & RIBN_B200_FLAG_REFERENCE_KERNELS)) {
        std::vector<Tensor*> mats;
        for (int l = 0; l < c.layers; ++l) {
            for (int w = 0; w < kLayerTensors; ++w) if (!is_norm(w)) mats.push_back(&ex->lt(l, w));
        }
        mats.push_back(&ex->output);
        size_t largest = 0;
        for (Tensor* t : mats) if (packable(t->type, t->rows, t->cols)) largest = std::max(largest, t->bytes);
        std::vector<unsigned char> raw(largest), packed;
        const int threads = (int)std::max(1u, std::min(32u, std::thread::hardware_concurrency()));
        for (Tensor* t : mats) {
            if (!packable(t->type, t->rows, t->cols)) continue;
            PackedMatrix& p = t->packed;
            p.type = t->type; p.n = t->rows; p.k = t->cols;
            p.row_tiles = (int)((t->rows + kTileRows - 1) / kTileRows);
            p.k_tiles = (int)(t->cols / kTileCols);
            p.bytes = packed_bytes(t->type, t->rows, t->cols);
            packed.resize(p.bytes);
            CU_TRY(ex, cudaMemcpy(raw.data(), t->raw, t->bytes, cudaMemcpyDeviceToHost));
            repack_host(t->type, raw.data(), t->rows, t->cols, packed.data(), threads);
            CU_TRY(ex, dev_alloc(ex, &p.data, p.bytes));
            CU_TRY(ex, cudaMemcpy(p.data, packed.data(), p.bytes, cudaMemcpyHostToDevice));
            // the tensor-memory GEMM's operands, converted once instead of on every use
            if ((c.flags & RIBN_B200_FLAG_OPERAND_CACHE) && !(c.flags & RIBN_B200_FLAG_NO_TCGEN05) &&
                (t->type == kQ4_K || t->type == kQ6_K)) {
                CU_TRY(ex, dev_alloc(ex, &t->op_a, tc_cache_a_bytes(t->type, t->rows, t->cols)));
                CU_TRY(ex, dev_alloc(ex, &t->op_meta, tc_cache_meta_bytes(t->rows, t->cols)));
                CU_TRY(ex, launch_tc_cache(ex->stream, t->type, p.data, t->rows, t->cols, t->op_a, t->op_meta));
            }
        }
        CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    }

    CU_TRY(ex, gemv_prepare());

    // Rotary table on the host, with the host libm's powf, so theta matches
    // `pos as f32 * base.powf(-(2 pair) / rot)` bit for bit
    // (crates/nvidia/src/qwen_reference.rs:414-415).
    {
        std::vector<float> table((size_t)c.head_dim / 2);
        for (int p = 0; p < c.head_dim / 2; ++p) {
            table[p] = powf(c.rope_base, -(2.0f * (float)p) / (float)c.head_dim);
        }
        CU_TRY(ex, dev_alloc(ex, &ex->inv_freq, table.size()));
        CU_TRY(ex, cudaMemcpy(ex->inv_freq, table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice));
    }

    // Paged KV arena (KvStateSpec, crates/core/src/state.rs:37-173): one shared
    // pool of 16-token pages; a sequence's table maps logical to physical pages.
    ex->pages_per_sequence = pages_for((uint32_t)c.context_tokens);
    ex->kv_pages = c.kv_pages > 0 ? c.kv_pages : ex->pages_per_sequence * c.max_sequences;
    const long long row_elems = (long long)c.kv_heads * c.head_dim;
    ex->layer_stride = (long long)ex->kv_pages * kPageTokens * row_elems;
    CU_TRY(ex, dev_alloc(ex, &ex->cache_k, (size_t)ex->layer_stride * c.layers));
    CU_TRY(ex, dev_alloc(ex, &ex->cache_v, (size_t)ex->layer_stride * c.layers));
    CU_TRY(ex, cudaMemsetAsync(ex->cache_k, 0, (size_t)ex->layer_stride * c.layers * sizeof(__half), ex->stream));
    CU_TRY(ex, cudaMemsetAsync(ex->cache_v, 0, (size_t)ex->layer_stride * c.layers * sizeof(__half), ex->stream));
    ex->free_pages.resize(ex->kv_pages);
    for (int i = 0; i < ex->kv_pages; ++i) ex->free_pages[i] = ex->kv_pages - 1 - i;
    ex->free_slots.resize(c.max_sequences);
    for (int i = 0; i < c.max_sequences; ++i) ex->free_slots[i] = c.max_sequences - 1 - i;
    CU_TRY(ex, dev_alloc(ex, &ex->d_page_tables, (size_t)c.max_sequences * ex->pages_per_sequence));
    CU_TRY(ex, cudaMemsetAsync(ex->d_page_tables, 0, (size_t)c.max_sequences * ex->pages_per_sequence * 4, ex->stream));
    CU_TRY(ex, dev_alloc(ex, &ex->d_next_token, (size_t)c.max_sequences));
    CU_TRY(ex, cudaMemsetAsync(ex->d_next_token, 0, (size_t)c.max_sequences * 4, ex->stream));

    // Step buffers.
    const size_t T = (size_t)c.max_batch_tokens, S = (size_t)c.max_sequences;
    const size_t QD = (size_t)c.q_heads * c.head_dim, KD = (size_t)c.kv_heads * c.head_dim;
    CU_TRY(ex, cudaMallocHost((void**)&ex->h_rows, S * sizeof(RowDesc)));
    CU_TRY(ex, cudaMallocHost((void**)&ex->h_tokens, T * sizeof(uint32_t)));
    CU_TRY(ex, cudaMallocHost((void**)&ex->h_sampled, S * sizeof(uint32_t)));
    CU_TRY(ex, dev_alloc(ex, &ex->d_rows, S));
    CU_TRY(ex, dev_alloc(ex, &ex->d_tokens, T));
    CU_TRY(ex, dev_alloc(ex, &ex->d_sampled, S));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.cu_seqlens, S + 1));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.token_row, T));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.token_pos, T));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.token_slot, T));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.token_id, T));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.token_seq, T));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.sample_token, S));
    CU_TRY(ex, dev_alloc(ex, &ex->meta.sample_slot, S));
    CU_TRY(ex, dev_alloc(ex, &ex->hidden, T * c.hidden));
    CU_TRY(ex, dev_alloc(ex, &ex->normed, T * std::max<size_t>(c.hidden, 1)));
    CU_TRY(ex, dev_alloc(ex, &ex->q, T * QD));
    CU_TRY(ex, dev_alloc(ex, &ex->k, T * KD));
    CU_TRY(ex, dev_alloc(ex, &ex->v, T * KD));
    CU_TRY(ex, dev_alloc(ex, &ex->attn, T * QD));
    CU_TRY(ex, dev_alloc(ex, &ex->gate, T * c.ffn));
    CU_TRY(ex, dev_alloc(ex, &ex->up, T * c.ffn));
    if (ex->tp > 1) CU_TRY(ex, dev_alloc(ex, &ex->proj, T * c.hidden));
    CU_TRY(ex, dev_alloc(ex, &ex->head_in, S * c.hidden));
    CU_TRY(ex, dev_alloc(ex, &ex->logits, S * c.vocab));
    {
        // Span accumulators: enough for every token of a full batch when that is small, capped at 256 MiB
        // (longer batches run the attention in several launches).
        const size_t spans = ((size_t)c.context_tokens + kAttnSpanKeys - 1) / kAttnSpanKeys;
        const size_t per_token = (size_t)c.q_heads * spans * (c.head_dim + 2) * sizeof(float);
        ex->scratch.attn_partial_bytes = std::max(per_token, std::min(per_token * T, (size_t)256 << 20));
        CU_TRY(ex, dev_alloc(ex, (unsigned char**)&ex->scratch.attn_partial, ex->scratch.attn_partial_bytes));
    }
    {
        auto alloc_operand = [&](ActOperand* op, int k) -> cudaError_t {
            cudaError_t e = dev_alloc(ex, &op->dig, (size_t)kGemvMaxMembers * 3 * k);
            if (e == cudaSuccess) e = dev_alloc(ex, &op->sx, (size_t)kGemvMaxMembers * (k / 32));
            if (e == cudaSuccess) e = dev_alloc(ex, &op->sxs16, (size_t)kGemvMaxMembers * (k / 16));
            if (e == cudaSuccess) e = dev_alloc(ex, &op->ss32, (size_t)kGemvMaxMembers * (k / 32));
            return e;
        };
        CU_TRY(ex, alloc_operand(&ex->op_hidden, c.hidden));
        CU_TRY(ex, alloc_operand(&ex->op_attn, c.q_heads * c.head_dim));
        CU_TRY(ex, alloc_operand(&ex->op_act, c.ffn));
        CU_TRY(ex, alloc_operand(&ex->op_head, c.hidden));
        {
            const int kmax = std::max(std::max(c.hidden, c.ffn), c.q_heads * c.head_dim);
            if (kmax % 256 == 0) {
                CU_TRY(ex, dev_alloc(ex, &ex->op_batch.chunks, batch_operand_bytes(kGemmMaxMembers, kmax)));
                // room for every 64-row group of the largest step (one conversion per projection), or one 128-row operand
                const size_t tc_groups = ((size_t)c.max_batch_tokens + 63) / 64;
                const size_t tc_rows = std::max<size_t>(tc_groups * 64, kGemmTcMaxMembers);
                CU_TRY(ex, dev_alloc(ex, (unsigned char**)&ex->op_tc.chunks,
                                     std::max(tc_operand_bytes(kGemmTcMaxMembers, kmax), tc_groups * tc_operand_bytes(64, kmax))));
                CU_TRY(ex, dev_alloc(ex, &ex->op_tc.scale_in, tc_rows));
                // room for four K slices of the widest fused projection at 64 rows
                ex->tc_partial_floats = (size_t)4 * 64 * (size_t)std::max(std::max(2 * c.ffn, c.hidden), (c.q_heads + 2 * c.kv_heads) * c.head_dim);
                CU_TRY(ex, dev_alloc(ex, &ex->tc_partial, ex->tc_partial_floats));
                CU_TRY(ex, dev_alloc(ex, &ex->op_tc.member_scale, tc_rows));
                CU_TRY(ex, dev_alloc(ex, &ex->op_batch.member_scale, kGemmMaxMembers));
                CU_TRY(ex, dev_alloc(ex, &ex->op_batch.digit_inv, kGemmMaxMembers));
            }
        }
        CU_TRY(ex, dev_alloc(ex, &ex->d_error, 1));
        CU_TRY(ex, cudaMemsetAsync(ex->d_error, 0, sizeof(int), ex->stream));
        CU_TRY(ex, cudaMallocHost((void**)&ex->h_error, sizeof(int)));
        *ex->h_error = 0;
    }
    CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    ex->finalized = true;
    return RIBN_B200_OK;
}

int ribn_b200_tp_unique_id(const char* nccl_library, ribn_b200_nccl_id* id, char* error, size_t error_capacity) {
    auto report = [&](const char* msg) {
        if (error != nullptr && error_capacity > 0) snprintf(error, error_capacity, "%s", msg);
        return RIBN_B200_ERROR;
    };
    if (id == nullptr) return report("null argument");
    static NcclApi api;  // the process's one NCCL library
    std::string why;
    if (!load_nccl(api, nccl_library, why)) return report(why.c_str());
    const int rc = api.get_unique_id(id);
    if (rc != 0) return report(api.get_error_string(rc));
    return RIBN_B200_OK;
}

int ribn_b200_tp_init(ribn_b200_executor* ex, const char* nccl_library, const ribn_b200_nccl_id* id) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (ex->tp <= 1) return fail(ex, "this executor was created without tensor parallelism");
    if (ex->comm != nullptr) return fail(ex, "the executor already joined its group");
    if (id == nullptr) return fail(ex, "null group id");
    std::string why;
    if (!load_nccl(ex->nccl, nccl_library, why)) return fail(ex, "%s", why.c_str());
    cudaSetDevice(ex->cfg.device);
    const int rc = ex->nccl.comm_init_rank(&ex->comm, ex->tp, *id, ex->rank);
    if (rc != 0) {
        ex->comm = nullptr;
        return fail(ex, "ncclCommInitRank failed: %s", ex->nccl.get_error_string(rc));
    }
    return RIBN_B200_OK;
}

int ribn_b200_tp_time_allreduce(ribn_b200_executor* ex, uint32_t tokens, uint32_t repeats, float* average_us) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (ex->tp <= 1 || ex->comm == nullptr || !ex->finalized || ex->pending.active) return fail(ex, "time_allreduce: no idle tensor-parallel executor");
    if (tokens == 0 || tokens > (uint32_t)ex->cfg.max_batch_tokens || repeats == 0 || average_us == nullptr) return fail(ex, "time_allreduce: bad argument");
    cudaSetDevice(ex->cfg.device);
    CU_TRY(ex, cudaMemsetAsync(ex->proj, 0, (size_t)tokens * ex->cfg.hidden * sizeof(float), ex->stream));
    for (int warm = 0; warm < 3; ++warm) {
        if (ex->nccl.all_reduce(ex->proj, ex->proj, (size_t)tokens * ex->cfg.hidden, 7, 0, ex->comm, ex->stream) != 0) return fail(ex, "ncclAllReduce failed");
    }
    CU_TRY(ex, cudaEventRecord(ex->ev_start, ex->stream));
    for (uint32_t r = 0; r < repeats; ++r) {
        if (ex->nccl.all_reduce(ex->proj, ex->proj, (size_t)tokens * ex->cfg.hidden, 7, 0, ex->comm, ex->stream) != 0) return fail(ex, "ncclAllReduce failed");
    }
    CU_TRY(ex, cudaEventRecord(ex->ev_done, ex->stream));
    CU_TRY(ex, cudaEventSynchronize(ex->ev_done));
    float ms = 0.0f;
    CU_TRY(ex, cudaEventElapsedTime(&ms, ex->ev_start, ex->ev_done));
    *average_us = ms * 1000.0f / (float)repeats;

    return RIBN_B200_OK;
}

int ribn_b200_tp_shard(const ribn_b200_config* config, const char* name, int64_t full_rows, int64_t full_cols,
                       int64_t* row0, int64_t* rows, int64_t* col0, int64_t* cols) {
    if (config == nullptr || row0 == nullptr || rows == nullptr || col0 == nullptr || cols == nullptr) return RIBN_B200_ERROR;
    const int role = role_from_name(name);
    const int tp = config->tp_size > 1 ? config->tp_size : 1;
    if (role < 0 || config->tp_rank < 0 || config->tp_rank >= tp) return RIBN_B200_ERROR;
    if (tp > 1 && (config->q_heads % tp != 0 || config->kv_heads % tp != 0 || config->ffn % 256 != 0 || config->ffn / 256 < tp)) {
        return RIBN_B200_ERROR;
    }
    long long r0, nr, c0, nc;
    shard_of(*config, tp, config->tp_rank, role, full_rows, full_cols, &r0, &nr, &c0, &nc);
    *row0 = r0; *rows = nr; *col0 = c0; *cols = nc;
    return RIBN_B200_OK;
}

int ribn_b200_info(ribn_b200_executor* ex, ribn_b200_limits* out) {
    if (ex == nullptr || out == nullptr) return RIBN_B200_ERROR;
    out->context_tokens = (uint32_t)ex->cfg.context_tokens;
    out->max_sequences = (uint32_t)ex->cfg.max_sequences;
    out->max_batch_tokens = (uint32_t)ex->cfg.max_batch_tokens;
    out->max_decode_tokens = 1;
    out->kv_page_tokens = kPageTokens;
    out->kv_pages_total = (uint32_t)ex->kv_pages;
    out->kv_pages_free = (uint32_t)ex->free_pages.size();
    return RIBN_B200_OK;
}

}  // extern "C"

namespace {

// Take `count` more pages from the arena for a sequence and publish its page-table row.
int grow_pages(ribn_b200_executor* ex, Sequence& seq, int count) {
    const int first = (int)seq.pages.size();
    for (int i = 0; i < count; ++i) {
        seq.pages.push_back(ex->free_pages.back());
        ex->free_pages.pop_back();
    }
    if (count == 0) return RIBN_B200_OK;
    cudaSetDevice(ex->cfg.device);
    cudaError_t e = cudaMemcpyAsync(ex->d_page_tables + (size_t)seq.slot * ex->pages_per_sequence + first,
                                    seq.pages.data() + first, (size_t)count * sizeof(int32_t), cudaMemcpyHostToDevice,
                                    ex->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ex->stream);  // pageable source: keep it simple and safe
    if (e != cudaSuccess) {
        for (int i = 0; i < count; ++i) { ex->free_pages.push_back(seq.pages.back()); seq.pages.pop_back(); }
        ex->faulted = true;
        return fail(ex, "page table upload failed: %s", cudaGetErrorString(e));
    }
    return RIBN_B200_OK;
}

// Returns a sequence's pages and slot to the executor.
void retire_sequence(ribn_b200_executor* ex, uint64_t sequence) {
    auto found = ex->sequences.find(sequence);
    if (found == ex->sequences.end()) return;
    for (int32_t page : found->second.pages) ex->free_pages.push_back(page);
    ex->free_slots.push_back(found->second.slot);
    ex->sequences.erase(found);
}

}  // namespace

extern "C" {

int ribn_b200_admit(ribn_b200_executor* ex, uint64_t request_id, uint64_t sequence, const uint32_t* tokens,
                    uint32_t token_count, uint32_t max_output_tokens, const ribn_b200_sampling* sampling,
                    const uint32_t* stop_tokens, uint32_t stop_count) {
    (void)request_id;
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (!ex->finalized) return fail(ex, "executor is not finalized");
    if (ex->sequences.count(sequence)) return fail(ex, "duplicate sequence");
    const ribn_b200_config& c = ex->cfg;
    const uint64_t total = (uint64_t)token_count + max_output_tokens;
    bool bad = token_count == 0 || max_output_tokens == 0 || total > (uint64_t)c.context_tokens ||
               (token_count > 0 && tokens == nullptr) || (stop_count > 0 && stop_tokens == nullptr);
    for (uint32_t i = 0; !bad && i < token_count; ++i) bad = tokens[i] >= (uint32_t)c.vocab;
    for (uint32_t i = 0; !bad && i < stop_count; ++i) bad = stop_tokens[i] >= (uint32_t)c.vocab;
    if (bad) return soft(ex, RIBN_B200_REJECTED, "Qwen input/output limits or token IDs are invalid");
    // Sampling::is_greedy (crates/qwen/src/execution.rs:107-111): temperature 0 selects the first maximum;
    // top_p / top_k / seed are carried for non-greedy selection, which this executor rejects as the reference does.
    if (sampling != nullptr && sampling->temperature != 0.0f) {
        return soft(ex, RIBN_B200_REJECTED, "the executor currently supports greedy sampling only");
    }
    if ((int)ex->sequences.size() >= c.max_sequences || ex->free_slots.empty()) {
        return soft(ex, RIBN_B200_DEFERRED, "all sequence slots are in use");
    }
    const int envelope = pages_for((uint32_t)total);
    if (envelope > ex->kv_pages) {
        return soft(ex, RIBN_B200_REJECTED, "request needs %d KV pages, above the %d-page arena", envelope, ex->kv_pages);
    }
    // Reserve the request-reachable envelope atomically (execution.rs:125-149), or, with
    // RIBN_B200_FLAG_KV_ON_DEMAND, only the prompt's pages: decode pages are then taken at prepare.
    const bool on_demand = (c.flags & RIBN_B200_FLAG_KV_ON_DEMAND) != 0;
    const int need = on_demand ? pages_for(token_count) : envelope;
    if (need > (int)ex->free_pages.size()) return soft(ex, RIBN_B200_DEFERRED, "KV arena has no free pages");
    Sequence seq;
    seq.id = sequence;
    seq.slot = ex->free_slots.back();
    seq.prompt.assign(tokens, tokens + token_count);
    seq.prompt_len = token_count;
    seq.max_output = max_output_tokens;
    if (grow_pages(ex, seq, need) != RIBN_B200_OK) return RIBN_B200_ERROR;
    ex->free_slots.pop_back();
    ex->sequences.emplace(sequence, std::move(seq));
    return RIBN_B200_OK;
}

int ribn_b200_prepare_rows(ribn_b200_executor* ex, const ribn_b200_batch_item* items, uint32_t count,
                           ribn_b200_prepared_row* rows) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (!ex->finalized) return fail(ex, "executor is not finalized");
    if (ex->pending.active || ex->prepared) return fail(ex, "Qwen execution is faulted or busy");
    const ribn_b200_config& c = ex->cfg;
    uint64_t tokens = 0;
    for (uint32_t i = 0; i < count; ++i) tokens += items[i].token_budget;
    if (count == 0 || items == nullptr || count > (uint32_t)c.max_sequences || tokens > (uint64_t)c.max_batch_tokens) {
        return fail(ex, "Qwen batch exceeds prepared limits");
    }
    for (uint32_t i = 0; i < count; ++i) {
        const ribn_b200_batch_item& it = items[i];
        auto found = ex->sequences.find(it.sequence);
        if (found == ex->sequences.end() || found->second.released) return fail(ex, "unknown Qwen sequence");
        const Sequence& s = found->second;
        if (s.in_flight) return fail(ex, "Qwen sequence is in flight");
        for (uint32_t j = 0; j < i; ++j) {
            if (items[j].sequence == it.sequence) return fail(ex, "duplicate sequence in batch");
        }
        const uint64_t end = (uint64_t)it.prefix + it.token_budget;
        if (it.token_budget == 0 || s.position != it.prefix || end > (uint64_t)c.context_tokens) {
            return fail(ex, "Qwen work does not match the sequence prefix/capacity");
        }
        if (it.kind == RIBN_B200_PREFILL) {
            if (end > s.prompt_len || it.output_budget != (end == s.prompt_len ? 1u : 0u)) {
                return fail(ex, "Qwen prefill boundary/output mismatch");
            }
        } else if (it.kind == RIBN_B200_DECODE) {
            if (it.token_budget != 1 || it.output_budget != 1 || it.prefix < s.prompt_len) {
                return fail(ex, "Qwen adapter only supports one-token ordinary decode");
            }
            if (!s.has_next) return fail(ex, "Qwen decode has no next token");
            if (end > (uint64_t)s.prompt_len + s.max_output) {
                return fail(ex, "Qwen work does not match the sequence prefix/capacity");
            }
        } else {
            return fail(ex, "unknown step kind");
        }
    }
    // Every offered row is valid.  A row whose range reaches past the pages its sequence holds takes pages from
    // the arena now (the executor keeps them; nothing else of the sequence changes); a row the arena cannot
    // serve is Deferred and retains nothing new (PreparedRow, crates/runtime/src/executor.rs:97-105).  Prompt
    // pages are held since admission, so only decode rows of an on-demand executor can be deferred.
    ex->prepared_items.clear();
    bool unchanged = true;
    for (uint32_t i = 0; i < count; ++i) {
        const ribn_b200_batch_item& it = items[i];
        Sequence& s = ex->sequences.find(it.sequence)->second;
        ribn_b200_prepared_row row{RIBN_B200_ROW_READY, it.token_budget, it.output_budget, 0};
        const int need = pages_for(it.prefix + it.token_budget) - (int)s.pages.size();
        if (need > (int)ex->free_pages.size()) {
            row.state = RIBN_B200_ROW_DEFERRED;
            row.token_budget = row.output_budget = 0;
            unchanged = false;
        } else {
            if (need > 0 && grow_pages(ex, s, need) != RIBN_B200_OK) return RIBN_B200_ERROR;
            ex->prepared_items.push_back(it);
        }
        if (rows != nullptr) rows[i] = row;
    }
    if (!unchanged && rows == nullptr) {
        ex->prepared_items.clear();
        return fail(ex, "KV arena cannot serve every offered row; prepare_rows reports the decision per row");
    }
    ex->prepared = true;
    if (!unchanged) ex->error = "KV arena has no free pages for some rows";
    return unchanged ? RIBN_B200_OK : RIBN_B200_SELECTED;
}

int ribn_b200_prepare(ribn_b200_executor* ex, const ribn_b200_batch_item* items, uint32_t count) {
    return ribn_b200_prepare_rows(ex, items, count, nullptr);
}

int ribn_b200_abandon_preparation(ribn_b200_executor* ex) {
    if (ex == nullptr) return RIBN_B200_ERROR;
    ex->prepared = false;
    ex->prepared_items.clear();
    return RIBN_B200_OK;
}

int ribn_b200_submit(ribn_b200_executor* ex, const ribn_b200_batch_item* items, uint32_t count, uint64_t* submission) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (!ex->prepared) return fail(ex, "submit without a preparation");
    if (count == 0 || items == nullptr || submission == nullptr) return fail(ex, "submit needs at least one prepared row");
    if (count != ex->prepared_items.size() ||
        memcmp(items, ex->prepared_items.data(), count * sizeof(ribn_b200_batch_item)) != 0) {
        return fail(ex, "submitted rows differ from the prepared rows");
    }
    // The prepared rows name live sequences (release refuses a prepared sequence); look them up defensively all the same.
    for (uint32_t i = 0; i < count; ++i) {
        if (ex->sequences.find(items[i].sequence) == ex->sequences.end()) {
            ex->prepared = false;
            ex->prepared_items.clear();
            return fail(ex, "unknown Qwen sequence in the prepared rows");
        }
    }
    cudaSetDevice(ex->cfg.device);
    Pending& p = ex->pending;
    p.items = ex->prepared_items;
    p.sample_row.assign(count, -1);
    StepPlan plan;
    plan.n_rows = (int)count;
    for (uint32_t i = 0; i < count; ++i) {
        const ribn_b200_batch_item& it = items[i];
        Sequence& s = ex->sequences.find(it.sequence)->second;
        RowDesc& r = ex->h_rows[i];
        r.slot = s.slot;
        r.prefix = (int32_t)it.prefix;
        r.tokens = (int32_t)it.token_budget;
        if (it.kind == RIBN_B200_PREFILL) {
            r.token_offset = plan.n_prompt_tokens;
            memcpy(ex->h_tokens + plan.n_prompt_tokens, s.prompt.data() + it.prefix, it.token_budget * sizeof(uint32_t));
            plan.n_prompt_tokens += (int)it.token_budget;
        } else {
            r.token_offset = -1;
        }
        r.sample_row = it.output_budget > 0 ? plan.n_sample++ : -1;
        p.sample_row[i] = r.sample_row;
        r.pad[0] = r.pad[1] = r.pad[2] = 0;
        if ((int)it.token_budget > plan.run_count) { plan.run_first = plan.n_tokens; plan.run_count = (int)it.token_budget; }
        plan.n_tokens += (int)it.token_budget;
        plan.max_keys = std::max(plan.max_keys, (int)(it.prefix + it.token_budget));
    }
    p.n_sample = plan.n_sample;
    if (ex->inject_bad_row > 0) {  // host-side fault injection: a corrupted row record
        --ex->inject_bad_row;
        ex->h_rows[0].slot = ex->cfg.max_sequences + 7;
    }
    // What is about to be uploaded must describe the plan: slots in range, ranges inside the context, token counts
    // adding up.  A record that does not is never sent to the device.
    {
        long long total = 0;
        bool sane = true;
        for (uint32_t i = 0; i < count; ++i) {
            const RowDesc& r = ex->h_rows[i];
            sane = sane && r.slot >= 0 && r.slot < ex->cfg.max_sequences && r.prefix >= 0 && r.tokens > 0 &&
                   (long long)r.prefix + r.tokens <= ex->cfg.context_tokens &&
                   (r.token_offset < 0 || r.token_offset + r.tokens <= ex->cfg.max_batch_tokens);
            total += r.tokens;
        }
        if (!sane || total != plan.n_tokens) {
            ex->faulted = true;
            return fail(ex, "malformed row record in the step plan");
        }
    }
    // Mark ownership before the first launch: if anything below fails the
    // executor faults and keeps everything until synchronize.
    for (uint32_t i = 0; i < count; ++i) ex->sequences.find(items[i].sequence)->second.in_flight = true;
    ex->prepared = false;
    p.active = true;
    p.id = ex->next_submission++;
    // Everything the step does on the stream, in order: row records and prompt tokens in, kernels,
    // sampled tokens and the error word out.
    auto enqueue = [&](int& launches) -> cudaError_t {
        cudaError_t e = cudaMemcpyAsync(ex->d_rows, ex->h_rows, count * sizeof(RowDesc), cudaMemcpyHostToDevice, ex->stream);
        if (e == cudaSuccess && plan.n_prompt_tokens > 0) {
            e = cudaMemcpyAsync(ex->d_tokens, ex->h_tokens, (size_t)plan.n_prompt_tokens * sizeof(uint32_t),
                                cudaMemcpyHostToDevice, ex->stream);
        }
        if (e == cudaSuccess) e = run_step(ex, plan, launches);
        if (e == cudaSuccess && plan.n_sample > 0) {
            e = cudaMemcpyAsync(ex->h_sampled, ex->d_sampled, (size_t)plan.n_sample * sizeof(uint32_t),
                                cudaMemcpyDeviceToHost, ex->stream);
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(ex->h_error, ex->d_error, sizeof(int), cudaMemcpyDeviceToHost, ex->stream);
        return e;
    };
    if (ex->inject_error_word != 0) {  // host-side fault injection: the error word a kernel's expired wait would leave
        CU_TRY(ex, cudaMemcpyAsync(ex->d_error, &ex->inject_error_word, sizeof(int), cudaMemcpyHostToDevice, ex->stream));
        CU_TRY(ex, cudaStreamSynchronize(ex->stream));
        ex->inject_error_word = 0;
    }
    int launches = 0;
    // Decode-only steps replay captured graphs: always for one or two rows; for larger batches (several hundred
    // launches per step, whose launch gaps a graph closes) once the same shape has come up three times, and while
    // the executor holds fewer than kMaxStepGraphs graphs.
    constexpr size_t kMaxStepGraphs = 192;
    bool graphable = !(ex->cfg.flags & RIBN_B200_FLAG_NO_GRAPH) && packed_family_applies(ex) &&
                     plan.n_rows == plan.n_tokens && plan.n_prompt_tokens == 0;
    if (graphable && !decode_family_applies(ex, plan)) {
        const int bucket = (plan.max_keys + 511) / 512;
        const uint64_t key = (uint64_t)plan.n_tokens | ((uint64_t)plan.n_sample << 16) | ((uint64_t)bucket << 32);
        if (ex->graphs.find(key) == ex->graphs.end()) {
            graphable = ++ex->graph_seen[key] >= 3 && ex->graphs.size() < kMaxStepGraphs;
        }
    }
    CU_TRY(ex, cudaEventRecord(ex->ev_start, ex->stream));
    if (graphable) {
        // Decode-only steps replay a captured graph.  The attention grid is sized by a bucket of the
        // longest context (results do not depend on it), so a graph serves 512 consecutive positions.
        const int bucket = (plan.max_keys + 511) / 512;
        plan.max_keys = std::min(bucket * 512, ex->cfg.context_tokens);
        const uint64_t key = (uint64_t)plan.n_tokens | ((uint64_t)plan.n_sample << 16) | ((uint64_t)bucket << 32);
        auto found = ex->graphs.find(key);
        if (found == ex->graphs.end()) {
            cudaGraph_t graph = nullptr;
            CU_TRY(ex, cudaStreamBeginCapture(ex->stream, cudaStreamCaptureModeThreadLocal));
            cudaError_t e = enqueue(launches);
            cudaError_t end = cudaStreamEndCapture(ex->stream, &graph);
            CU_TRY(ex, e);
            CU_TRY(ex, end);
            ribn_b200_executor::StepGraph entry;
            entry.launches = launches;
            cudaError_t inst = cudaGraphInstantiate(&entry.exec, graph, 0);
            cudaGraphDestroy(graph);
            CU_TRY(ex, inst);
            found = ex->graphs.emplace(key, entry).first;
        }
        launches = found->second.launches;
        CU_TRY(ex, cudaGraphLaunch(found->second.exec, ex->stream));
    } else {
        CU_TRY(ex, enqueue(launches));
    }
    p.launches = launches;
    CU_TRY(ex, cudaEventRecord(ex->ev_done, ex->stream));
    *submission = p.id;
    return RIBN_B200_OK;
}

int ribn_b200_poll(ribn_b200_executor* ex, uint64_t submission, ribn_b200_completion* rows, uint32_t capacity,
                   uint32_t* count) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    Pending& p = ex->pending;
    if (!p.active) return fail(ex, "unknown Qwen submission");
    if (p.id != submission) return fail(ex, "Qwen submission identity mismatch");
    cudaSetDevice(ex->cfg.device);
    cudaError_t q = cudaEventQuery(ex->ev_done);
    if (q == cudaErrorNotReady) return RIBN_B200_PENDING;
    if (q != cudaSuccess) {
        // Any status other than NOT_READY is a fault (crates/nvidia/src/serving.rs:624-635).
        ex->faulted = true;
        return fail(ex, "device work failed: %s", cudaGetErrorString(q));
    }
    if (*ex->h_error != 0) {
        ex->faulted = true;
        return fail(ex, "a device-side bounded wait expired (code %d)", *ex->h_error);
    }
    if (capacity < p.items.size()) return fail(ex, "completion buffer too small");
    cudaEventElapsedTime(&ex->last_ms, ex->ev_start, ex->ev_done);
    ex->last_launches = (uint32_t)p.launches;
    ex->last_n_sample = p.n_sample;
    for (size_t i = 0; i < p.items.size(); ++i) {
        const ribn_b200_batch_item& it = p.items[i];
        Sequence& s = ex->sequences.find(it.sequence)->second;
        ribn_b200_completion& out = rows[i];
        out.sequence = it.sequence;
        out.prefix = it.prefix + it.token_budget;
        out.n_tokens = 0;
        out.token = 0;
        out.reserved = 0;
        if (p.sample_row[i] >= 0) {
            const uint32_t token = ex->h_sampled[p.sample_row[i]];
            if (token >= (uint32_t)ex->cfg.vocab) {
                ex->faulted = true;
                return fail(ex, "Qwen completion does not match submitted work");
            }
            out.n_tokens = 1;
            out.token = token;
            s.has_next = true;
        }
        s.position = out.prefix;
        s.in_flight = false;
        if (s.position >= s.prompt_len) std::vector<uint32_t>().swap(s.prompt);
    }
    *count = (uint32_t)p.items.size();
    p.active = false;
    // Sequences released while this submission referenced them are retired now
    // (drain_deferred_releases, crates/nvidia/src/serving.rs:1082-1096).
    for (uint64_t sequence : ex->deferred_releases) retire_sequence(ex, sequence);
    ex->deferred_releases.clear();
    return RIBN_B200_OK;
}

int ribn_b200_release(ribn_b200_executor* ex, uint64_t sequence) {
    if (ex == nullptr) return RIBN_B200_ERROR;
    auto found = ex->sequences.find(sequence);
    if (found == ex->sequences.end() || found->second.released) return RIBN_B200_OK;  // idempotent
    if (ex->prepared) {
        for (const ribn_b200_batch_item& it : ex->prepared_items) {
            if (it.sequence == sequence) return fail(ex, "cannot release prepared Qwen state");
        }
    }
    if (found->second.in_flight) {
        // Queued device work still reads this sequence's pages: park the release until the referencing
        // submission completes (release_inference_state, crates/nvidia/src/serving.rs:1231-1251).
        found->second.released = true;
        ex->deferred_releases.push_back(sequence);
        return RIBN_B200_OK;
    }
    retire_sequence(ex, sequence);
    return RIBN_B200_OK;
}

int ribn_b200_synchronize(ribn_b200_executor* ex) {
    if (ex == nullptr) return RIBN_B200_ERROR;
    cudaSetDevice(ex->cfg.device);
    ex->prepared = false;
    cudaError_t e = cudaStreamSynchronize(ex->stream);
    if (e != cudaSuccess) {
        ex->faulted = true;
        return fail(ex, "synchronize failed: %s", cudaGetErrorString(e));
    }
    return RIBN_B200_OK;
}

int ribn_b200_copy_logits(ribn_b200_executor* ex, uint32_t row, float* out, size_t capacity) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (ex->pending.active) return fail(ex, "a submission is still pending");
    if ((int)row >= ex->last_n_sample) return fail(ex, "no logits for row %u", row);
    if (capacity < (size_t)ex->cfg.vocab) return fail(ex, "logit buffer too small");
    cudaSetDevice(ex->cfg.device);
    CU_TRY(ex, cudaMemcpyAsync(out, ex->logits + (size_t)row * ex->cfg.vocab, (size_t)ex->cfg.vocab * sizeof(float),
                               cudaMemcpyDeviceToHost, ex->stream));
    CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    return RIBN_B200_OK;
}

int ribn_b200_copy_kv(ribn_b200_executor* ex, uint64_t sequence, int32_t layer, int32_t which, uint32_t tokens,
                      uint16_t* out) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    auto found = ex->sequences.find(sequence);
    if (found == ex->sequences.end()) return fail(ex, "unknown Qwen sequence");
    const ribn_b200_config& c = ex->cfg;
    if (layer < 0 || layer >= c.layers || tokens > (uint32_t)found->second.pages.size() * kPageTokens) {
        return fail(ex, "copy_kv range is outside the sequence's reservation");
    }
    cudaSetDevice(c.device);
    const int row_elems = c.kv_heads * c.head_dim;
    __half* tmp = nullptr;
    CU_TRY(ex, cudaMalloc((void**)&tmp, std::max<size_t>((size_t)tokens * row_elems, 1) * sizeof(__half)));
    const __half* cache = (which ? ex->cache_v : ex->cache_k) + (long long)layer * ex->layer_stride;
    cudaError_t e = launch_gather_kv(ex->stream, cache, ex->d_page_tables + (size_t)found->second.slot * ex->pages_per_sequence,
                                     (int)tokens, row_elems, tmp);
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, tmp, (size_t)tokens * row_elems * 2, cudaMemcpyDeviceToHost, ex->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ex->stream);
    cudaFree(tmp);
    CU_TRY(ex, e);
    return RIBN_B200_OK;
}

int ribn_b200_debug_set_context(ribn_b200_executor* ex, uint64_t sequence, uint32_t tokens, uint32_t next_token,
                                uint64_t seed) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    auto found = ex->sequences.find(sequence);
    if (found == ex->sequences.end()) return fail(ex, "unknown Qwen sequence");
    Sequence& s = found->second;
    if (s.in_flight || tokens != s.prompt_len || next_token >= (uint32_t)ex->cfg.vocab) {
        return fail(ex, "set_context needs an idle sequence, tokens == prompt length and a valid token");
    }
    cudaSetDevice(ex->cfg.device);
    const ribn_b200_config& c = ex->cfg;
    CU_TRY(ex, launch_synth_kv(ex->stream, ex->cache_k, ex->cache_v, ex->layer_stride, c.layers,
                               ex->d_page_tables + (size_t)s.slot * ex->pages_per_sequence, (int)tokens,
                               c.kv_heads * c.head_dim, seed));
    CU_TRY(ex, cudaMemcpyAsync(ex->d_next_token + s.slot, &next_token, sizeof(uint32_t), cudaMemcpyHostToDevice,
                               ex->stream));
    CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    s.position = tokens;
    s.has_next = true;
    std::vector<uint32_t>().swap(s.prompt);
    return RIBN_B200_OK;
}

int ribn_b200_debug_inject(ribn_b200_executor* ex, int32_t kind, int32_t value) {
    if (ex == nullptr) return RIBN_B200_ERROR;
    switch (kind) {
        case RIBN_B200_INJECT_ALLOC_REFUSAL: ex->inject_alloc_failures = std::max(0, value); return RIBN_B200_OK;
        case RIBN_B200_INJECT_ERROR_WORD: ex->inject_error_word = value; return RIBN_B200_OK;
        case RIBN_B200_INJECT_BAD_ROW: ex->inject_bad_row = std::max(0, value); return RIBN_B200_OK;
        default: return fail(ex, "unknown injection kind %d", kind);
    }
}

int ribn_b200_debug_wait_expiry(ribn_b200_executor* ex, uint32_t spin_limit) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (!ex->finalized || ex->pending.active) return fail(ex, "wait_expiry: executor not idle");
    if (spin_limit == 0 || spin_limit > (1u << 20)) return fail(ex, "wait_expiry: the limit must be 1 .. 2^20 polls");
    cudaSetDevice(ex->cfg.device);
    // One thread waits on a barrier nothing completes; the wait gives up after `spin_limit` polls and leaves
    // code 99 in the executor's error word, where the next poll finds it.  The call itself returns once the
    // kernel has finished: the context stays usable.
    CU_TRY(ex, launch_wait_probe(ex->stream, ex->d_error, spin_limit, 99));
    CU_TRY(ex, cudaStreamSynchronize(ex->stream));
    return RIBN_B200_OK;
}

int ribn_b200_last_step_stats(ribn_b200_executor* ex, float* device_ms, uint32_t* kernel_launches) {
    if (ex == nullptr) return RIBN_B200_ERROR;
    if (device_ms) *device_ms = ex->last_ms;
    if (kernel_launches) *kernel_launches = ex->last_launches;
    return RIBN_B200_OK;
}

int ribn_b200_step_bytes(ribn_b200_executor* ex, uint64_t context_tokens_total, uint64_t* weight_bytes,
                         uint64_t* kv_bytes) {
    if (ex == nullptr) return RIBN_B200_ERROR;
    const ribn_b200_config& c = ex->cfg;
    uint64_t w = 0;
    for (const Tensor& t : ex->layer_tensors) w += t.bytes;
    w += ex->output_norm.bytes + ex->output.bytes;
    if (weight_bytes) *weight_bytes = w;
    if (kv_bytes) *kv_bytes = context_tokens_total * (uint64_t)c.layers * 2ull * c.kv_heads * c.head_dim * 2ull;
    return RIBN_B200_OK;
}

int ribn_b200_time_projection(ribn_b200_executor* ex, int32_t which, uint32_t repeats, float* average_us,
                              uint64_t* bytes_per_launch) {
    if (check_open(ex) != RIBN_B200_OK) return RIBN_B200_ERROR;
    if (!ex->finalized || ex->pending.active) return fail(ex, "time_projection: executor not idle");
    if (!packed_family_applies(ex) || repeats == 0 || average_us == nullptr) return fail(ex, "time_projection: unavailable");
    const ribn_b200_config& c = ex->cfg;
    cudaStream_t s = ex->stream;
    auto args_for = [&](int l) {
        switch (which) {
            case 0: return qkv_args(ex, l, 1);
            case 1: return o_args(ex, l, 1);
            case 2: return gate_up_args(ex, l, 1);
            case 3: return down_args(ex, l, 1);
            default: return head_args(ex, 1, ex->op_hidden);
        }
    };
    if (which < 0 || which > 4) return fail(ex, "time_projection: which must be 0..4");
    uint64_t bytes = 0;
    {
        const GemvArgs a = args_for(0);
        for (int i = 0; i < a.n_segments; ++i) {
            bytes += (uint64_t)a.seg[i].row_tiles * (uint64_t)(a.k / kTileCols) * (uint64_t)packed_tile_bytes(a.seg[i].type);
        }
    }
    if (bytes_per_launch) *bytes_per_launch = bytes;
    // Launch r takes layer r % layers, so consecutive launches read different weights from HBM.
    for (int warm = 0; warm < 3; ++warm) CU_TRY(ex, launch_gemv_mma(s, args_for(warm % c.layers), true));
    CU_TRY(ex, cudaEventRecord(ex->ev_start, s));
    for (uint32_t r = 0; r < repeats; ++r) CU_TRY(ex, launch_gemv_mma(s, args_for((int)(r % (uint32_t)c.layers)), true));
    CU_TRY(ex, cudaEventRecord(ex->ev_done, s));
    CU_TRY(ex, cudaEventSynchronize(ex->ev_done));
    float ms = 0.0f;
    CU_TRY(ex, cudaEventElapsedTime(&ms, ex->ev_start, ex->ev_done));
    *average_us = ms * 1000.0f / (float)repeats;
    int err = 0;
    CU_TRY(ex, cudaMemcpy(&err, ex->d_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (err != 0) return fail(ex, "time_projection: a bounded wait inside the kernel expired (code %d)", err);
    return RIBN_B200_OK;
}

}  // extern "C"
