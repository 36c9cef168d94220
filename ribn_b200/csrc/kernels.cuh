// Launchers of every device kernel of the decode / chunked-prefill step.
// All pointers are device pointers; every launcher enqueues on `stream` and
// returns the CUDA error of the launch.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemv.cuh"

namespace ribn {

constexpr int kPageTokens = 16;  // KV_PAGE_TOKENS, crates/qwen/src/gguf.rs:16

// Per-row scheduling record uploaded by the host each step (16 bytes/row).
struct RowDesc {
    int32_t slot;          // executor sequence slot (page-table row, next-token row)
    int32_t prefix;        // tokens already in the cache
    int32_t tokens;        // tokens this step
    int32_t token_offset;  // >= 0: offset into the uploaded prompt-token array;
                           //  < 0: decode row, input is next_token[slot]
    int32_t sample_row;    // >= 0: index of this row in the sampling list; < 0: no output
    int32_t pad[3];
};

struct StepMeta {
    int32_t* cu_seqlens;    // [rows + 1]
    int32_t* token_row;     // [T]
    int32_t* token_pos;     // [T] absolute position in the sequence
    int32_t* token_slot;    // [T] physical KV token index (page * 16 + offset)
    uint32_t* token_id;     // [T] input token ids
    int32_t* token_seq;     // [T] executor sequence slot of the token's row
    int32_t* sample_token;  // [sampling rows] index into [T] of the row's last token
    int32_t* sample_slot;   // [sampling rows] sequence slot that receives the sampled token
};

cudaError_t launch_step_metadata(cudaStream_t stream, const RowDesc* rows, int n_rows, int n_tokens,
                                 const uint32_t* prompt_tokens, const uint32_t* next_token,
                                 const int32_t* page_tables, int pages_per_sequence, StepMeta meta);

// Plain metadata (the C-ABI operator): cu_seqlens / row / position / slot only.
cudaError_t launch_batch_metadata(cudaStream_t stream, const int32_t* row_slot, const int32_t* row_prefix,
                                  const int32_t* row_tokens, int n_rows, int n_tokens,
                                  const int32_t* page_tables, int pages_per_sequence, int page_tokens,
                                  int32_t* cu_seqlens, int32_t* token_row, int32_t* token_pos,
                                  int32_t* token_slot);

// hidden[t][:] = dequantised row token_id[t] of the raw-layout embedding table.
cudaError_t launch_embedding(cudaStream_t stream, int type, const unsigned char* table, int hidden,
                             int vocab, const uint32_t* token_id, int n_tokens, float* out);

// out[rows][cols] = decoded elements of raw-layout encoded rows.
cudaError_t launch_dequantize(cudaStream_t stream, int type, const unsigned char* bytes, long long rows,
                              long long cols, float* out);

cudaError_t launch_rms_norm(cudaStream_t stream, const float* x, const float* weight, int members,
                            int length, float eps, float* out);
// Gathers rows `index[m]` of x (index == nullptr: identity) before normalising.
cudaError_t launch_rms_norm_gather(cudaStream_t stream, const float* x, const int32_t* index,
                                   const float* weight, int members, int length, float eps, float* out);

// Reference GEMV: one warp per output row over raw GGUF blocks.
// y[m][n] (+)= sum_k deq(W[n][k]) * x[m][k]
cudaError_t launch_gemv_ref(cudaStream_t stream, int type, const unsigned char* w, long long n, long long k,
                            const float* x, int members, float* y, bool accumulate);

cudaError_t launch_silu_mul(cudaStream_t stream, const float* gate, const float* up, long long length,
                            float* out);
cudaError_t launch_residual_add(cudaStream_t stream, float* acc, const float* inc, long long length);
// out[m] = argmax of row m; when `slot` is given, next_token[slot[m]] gets it too.
cudaError_t launch_argmax(cudaStream_t stream, const float* logits, int members, long long length,
                          uint32_t* out, const int32_t* slot = nullptr, uint32_t* next_token = nullptr);
cudaError_t launch_f32_to_f16(cudaStream_t stream, const float* in, long long length, uint16_t* out);
cudaError_t launch_rope_neox(cudaStream_t stream, float* values, const long long* positions, int members,
                             int heads, int head_dim, int rot_dims, const float* inv_freq);

// Per-head Q/K RMSNorm, NeoX rotary, and the F16 append of K/V into the paged
// cache, for every token of the step.  q: [T][q_heads][hd] (in place),
// k, v: [T][kv_heads][hd] (k normalised and rotated in place).
cudaError_t launch_qk_norm_rope_append(cudaStream_t stream, float* q, float* k, const float* v,
                                       const float* q_norm, const float* k_norm, const float* inv_freq,
                                       const int32_t* token_pos, const int32_t* token_slot, int n_tokens,
                                       int q_heads, int kv_heads, int head_dim, float eps,
                                       __half* cache_k, __half* cache_v);

// Reference attention: one warp per (token, q head), online softmax over the
// sequence's pages.  Token t attends keys [max(0, pos - window + 1), pos]
// (window <= 0: from 0).
cudaError_t launch_attention_ref(cudaStream_t stream, const float* q, const __half* cache_k,
                                 const __half* cache_v, const int32_t* page_tables, int pages_per_sequence,
                                 const int32_t* token_seq, const int32_t* token_pos, int n_tokens,
                                 int q_heads, int kv_heads, int head_dim, int window, float* out);

// Split-KV attention: spans of one to eight tiles of kAttnSpanKeys keys, merged in
// span order.  `max_keys` bounds the longest key range of any token in the launch
// (with the token count it sizes the grid and sets how many 64-key tiles one
// span covers, so a token's low bits can differ between launches of different
// sizes, never inside one).  `partial` is scratch
// of `partial_bytes` for the per-span accumulators; tokens are processed in
// as many launches as that scratch requires.  `launches` (optional) is
// incremented per kernel launch.  `token_seq` may be null: every token then
// belongs to sequence 0 (one page-table row).  A GQA group has at most
// 16 query heads.  `run_first`, `run_count` (optional) tell where a run of
// consecutive tokens of ONE sequence lies in the launch (a prefill chunk):
// its whole groups of 4 x (16 / group size) tokens take a kernel that stages
// each key tile once for such a group and walks all its keys, no merge.
constexpr int kAttnSpanKeys = 64;
constexpr int kAttnMaxSpans = 1024;  // tiles per token: 65536 keys
cudaError_t launch_attention(cudaStream_t stream, const float* q, const __half* cache_k, const __half* cache_v,
                             const int32_t* page_tables, int pages_per_sequence, const int32_t* token_seq,
                             const int32_t* token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                             int window, int max_keys, float* partial, size_t partial_bytes, float* out,
                             int* launches, int run_first = -1, int run_count = 0);

// Decode form of the same attention for rows that add exactly one token: it
// also applies the per-head Q/K RMSNorm and rotary to the raw projections,
// appends the token's K/V row to the paged cache, and can emit the result in
// tensor-core operand form (K = q_heads * head_dim) for the output projection.
struct DecodeAttention {
    const float* q;   // [T][q_heads][hd] raw q projection
    const float* k;   // [T][kv_heads][hd] raw k projection
    const float* v;   // [T][kv_heads][hd]
    const float* q_norm;
    const float* k_norm;
    const float* inv_freq;
    float eps;
    __half* cache_k;
    __half* cache_v;
    const int32_t* page_tables;
    int pages_per_sequence;
    const int32_t* token_seq;
    const int32_t* token_pos;
    const int32_t* token_slot;
    int n_tokens, q_heads, kv_heads, head_dim, window, max_keys;
    float* partial;
    size_t partial_bytes;
    float* out;
    ActOperand operand;
    bool programmatic;  // launch as programmatic dependents of the previous kernel in the stream
};
cudaError_t launch_attention_decode(cudaStream_t stream, const DecodeAttention& d, int* launches);

// Decode steps of a Gated-DeltaNet recurrent layer behind its projections, for `members` sequences with their own
// states, `tokens` consecutive tokens each (1: a decode step; more: a prefill chunk, token by token inside the
// kernel with the state in registers, the same arithmetic as that many single steps)
// (crates/nvidia/src/qwen_reference.rs:202-278).  Device pointers; [m] = per member, rows = m * tokens + t.
struct GdnStep {
    int members, tokens, k_heads, v_heads, head_dim;
    int channels;            // q | k | v convolution channels: k_heads * hd | k_heads * hd | v_heads * hd
    int k_offset, v_offset;  // first k channel, first v channel
    const float* qkv;        // [rows][channels] mixed projection of the tokens
    const float* z;          // [rows][v_heads * hd] gate projection
    const float* beta_raw;   // [rows][v_heads]
    const float* alpha_raw;  // [rows][v_heads]
    const float* dt_bias;    // [v_heads]
    const float* a;          // [v_heads], -exp(A_log)
    const float* conv_weight;  // [channels][4], tap fastest
    const float* norm_weight;  // [hd], not +1'd
    float* const* conv_state;  // [m] -> [channels][3], oldest first; advanced in place
    float* const* state;       // [m] -> [v_heads][hd][hd], row major; updated in place
    float l2_eps, norm_eps;
    float* decay;            // [rows][v_heads] out
    float* beta;             // [rows][v_heads] out
    float* conv_act;         // [rows][channels] out: convolution + SiLU
    float* attn_out;         // [rows][v_heads * hd] out, optional: S^T q / sqrt(hd) before the gated norm
    float* out;              // [rows][v_heads * hd] out: what the output projection reads
};
cudaError_t launch_gdn_step(cudaStream_t stream, const GdnStep& step);
// out = attn * sigmoid(gate), the gate being the second half of each head's [q | gate] projection
// (crates/nvidia/src/qwen_reference.rs:386-392, 462-472).
cudaError_t launch_attention_gate(cudaStream_t stream, const float* attn, const float* q_gate, long long rows, int heads,
                                  int head_dim, float* out);

// Seeded F16 K/V for the first `tokens` logical positions of one sequence, every layer.
cudaError_t launch_synth_kv(cudaStream_t stream, __half* cache_k, __half* cache_v, long long layer_stride,
                            int layers, const int32_t* page_table, int tokens, int row_elems, uint64_t seed);
// out[token][row_elems] = cache rows of logical tokens [0, tokens) through the page table.
cudaError_t launch_gather_kv(cudaStream_t stream, const __half* cache, const int32_t* page_table, int tokens,
                             int row_elems, __half* out);

// Seeded synthetic tensors.
cudaError_t launch_fill_f32(cudaStream_t stream, float* out, long long n, float value);
cudaError_t launch_synth_quantized(cudaStream_t stream, int type, unsigned char* out, long long rows,
                                   long long cols, uint64_t seed, float stddev);
cudaError_t launch_synth_f16(cudaStream_t stream, __half* out, long long n, uint64_t seed, float stddev);

}  // namespace ribn
