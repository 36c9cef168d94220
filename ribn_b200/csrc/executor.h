// Host-side state of one executor: model plan, paged KV arena, per-sequence
// continuation, and the single in-flight submission.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ribn_b200.h"
#include "gemv.cuh"
#include "kernels.cuh"

namespace ribn {

struct Tensor {
    int type = -1;
    long long rows = 0, cols = 0;
    size_t bytes = 0;
    unsigned char* raw = nullptr;  // encoded GGUF bytes, verbatim
    PackedMatrix packed;           // tile-major repack for the fast kernels (matrices only)
    unsigned char* op_a = nullptr;     // K-quant matrices under RIBN_B200_FLAG_OPERAND_CACHE: tensor-core operand
    unsigned char* op_meta = nullptr;  // pieces and their per-k-tile records (launch_tc_cache)
    bool loaded() const { return raw != nullptr; }
};

enum LayerTensor {
    kAttnNorm, kAttnQ, kAttnK, kAttnV, kAttnQNorm, kAttnKNorm, kAttnOutput,
    kFfnNorm, kFfnGate, kFfnUp, kFfnDown, kLayerTensors
};

struct Sequence {
    uint64_t id = 0;
    int slot = -1;
    std::vector<uint32_t> prompt;
    uint32_t prompt_len = 0;
    uint32_t max_output = 0;
    uint32_t position = 0;      // committed prefix
    bool has_next = false;      // a sampled token is pending as the next decode input
    bool in_flight = false;
    bool released = false;      // release() arrived while in flight: retired when the submission completes
    std::vector<int32_t> pages;
};

struct Pending {
    bool active = false;
    uint64_t id = 0;
    std::vector<ribn_b200_batch_item> items;
    std::vector<int> sample_row;  // per item: index into the pinned result slots, or -1
    int n_sample = 0;
    int launches = 0;
};

}  // namespace ribn

// The handful of NCCL entry points tensor parallelism needs, resolved at run time from the libnccl the host
// process names (a single-GPU process never loads it).
struct NcclApi {
    void* handle = nullptr;
    int (*get_unique_id)(void*) = nullptr;
    int (*comm_init_rank)(void**, int, ribn_b200_nccl_id, int) = nullptr;
    int (*all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*comm_destroy)(void*) = nullptr;
    const char* (*get_error_string)(int) = nullptr;
};

struct ribn_b200_executor {
    ribn_b200_config cfg{};    // this rank's geometry: q_heads, kv_heads and ffn are the LOCAL shard's
    ribn_b200_config full{};   // the whole model's geometry (equal to cfg without tensor parallelism)
    int tp = 1, rank = 0;      // tensor-parallel group size and this executor's rank in it
    int ffn_first = 0;         // first ffn column of this rank's shard
    NcclApi nccl;
    void* comm = nullptr;      // ncclComm_t
    float* proj = nullptr;     // [max_batch_tokens][hidden]: this rank's partial o_proj / ffn_down sums before the all-reduce
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_start = nullptr, ev_done = nullptr;
    std::string error;
    bool faulted = false, finalized = false;

    std::vector<ribn::Tensor> layer_tensors;  // [layers][kLayerTensors]
    ribn::Tensor token_embd, output_norm, output;
    float* inv_freq = nullptr;  // [head_dim / 2]

    // paged KV arena: [layer][page * 16 + offset][kv_head][head_dim], F16
    __half* cache_k = nullptr;
    __half* cache_v = nullptr;
    long long layer_stride = 0;  // elements per layer
    int kv_pages = 0, pages_per_sequence = 0;
    std::vector<int32_t> free_pages;
    int32_t* d_page_tables = nullptr;  // [max_sequences][pages_per_sequence]
    uint32_t* d_next_token = nullptr;  // [max_sequences]

    std::unordered_map<uint64_t, ribn::Sequence> sequences;
    std::vector<int> free_slots;

    // one outstanding preparation, one outstanding submission
    bool prepared = false;
    std::vector<ribn_b200_batch_item> prepared_items;
    ribn::Pending pending;
    uint64_t next_submission = 1;
    float last_ms = 0.0f;
    uint32_t last_launches = 0;
    int last_n_sample = 0;

    // pinned staging + device step buffers
    ribn::RowDesc* h_rows = nullptr;
    uint32_t* h_tokens = nullptr;
    uint32_t* h_sampled = nullptr;
    ribn::RowDesc* d_rows = nullptr;
    uint32_t* d_tokens = nullptr;
    uint32_t* d_sampled = nullptr;
    ribn::StepMeta meta{};
    float *hidden = nullptr, *normed = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr,
          *gate = nullptr, *up = nullptr, *head_in = nullptr, *logits = nullptr;
    ribn::StepScratch scratch;
    // tensor-core operand forms of the activations (decode rows on the fast path)
    ribn::ActOperand op_hidden, op_attn, op_act, op_head;
    ribn::BatchOperand op_batch;  // batch form, refilled before every batched projection
    ribn::TcOperand op_tc;        // tensor-memory form (the same, for the tcgen05 kernel)
    float* tc_partial = nullptr;  // split-K sums of the tcgen05 kernel
    size_t tc_partial_floats = 0;
    // Captured decode steps, keyed by (tokens, sampling rows, attention span bucket).
    struct StepGraph { cudaGraphExec_t exec = nullptr; int launches = 0; };
    std::map<uint64_t, StepGraph> graphs;
    std::map<uint64_t, int> graph_seen;  // how often a batched decode shape has come up (hot shapes get a graph)
    int* d_error = nullptr;    // raised by a kernel whose bounded wait expired
    int* h_error = nullptr;    // pinned copy read at poll
    std::vector<void*> allocations;
    std::vector<uint64_t> deferred_releases;  // sequences released while referenced by the pending submission
    // Host-side fault injection (ribn_b200_debug_inject): how many of the next device allocations to refuse,
    // an error word to plant at the end of the next step, and a row record to corrupt at the next submit.
    int inject_alloc_failures = 0;
    int inject_error_word = 0;
    int inject_bad_row = 0;

    ribn::Tensor& lt(int layer, int which) { return layer_tensors[(size_t)layer * ribn::kLayerTensors + which]; }
};
