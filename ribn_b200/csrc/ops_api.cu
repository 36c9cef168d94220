// Single-operator C-ABI entry points: host pointers in, host pointers out.
// Each stages its operands in device memory, runs the same kernels the
// executor's step uses, and copies the result back.  They exist so that
// per-primitive parity tests can be written the way the reference's device
// tests are (crates/nvidia/tests/cuda_reference.rs).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <string>
#include <vector>

#include "../../include/ribn_b200.h"
#include "blocks.cuh"
#include "gemv.cuh"
#include "kernels.cuh"

using namespace ribn;

namespace {

struct Scope {
    cudaStream_t stream = nullptr;
    std::vector<void*> owned;
    bool ok = false;
    explicit Scope(int device) {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return;
        if (cudaSetDevice(device) != cudaSuccess) return;
        ok = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess;
    }
    ~Scope() {
        if (stream) {
            cudaStreamSynchronize(stream);
            cudaStreamDestroy(stream);
        }
        for (void* p : owned) cudaFree(p);
    }
    template <typename T>
    T* alloc(size_t count) {
        void* p = nullptr;
        if (cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)) != cudaSuccess) return nullptr;
        owned.push_back(p);
        return (T*)p;
    }
    template <typename T>
    T* upload(const T* host, size_t count) {
        T* d = alloc<T>(count);
        if (d && count && cudaMemcpyAsync(d, host, count * sizeof(T), cudaMemcpyHostToDevice, stream) != cudaSuccess) {
            return nullptr;
        }
        return d;
    }
    template <typename T>
    bool download(T* host, const T* dev, size_t count) {
        if (count && cudaMemcpyAsync(host, dev, count * sizeof(T), cudaMemcpyDeviceToHost, stream) != cudaSuccess) {
            return false;
        }
        return cudaStreamSynchronize(stream) == cudaSuccess;
    }
};

// Why the calling thread's last operator call failed.
thread_local std::string g_op_error;

int op_fail(const char* what, cudaError_t e) {
    g_op_error = std::string(what) + ": " + (e == cudaSuccess ? "failed" : cudaGetErrorString(e));
    return RIBN_B200_ERROR;
}

#define OP_TRY(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) return op_fail(#expr, e_); } while (0)
#define OP_PTR(p) do { if ((p) == nullptr) return op_fail("device allocation or upload of " #p, cudaGetLastError()); } while (0)

size_t encoded_bytes(int type, long long rows, long long cols) {
    const int e = block_elems(type);
    if (e == 0 || cols % e != 0) return 0;
    return (size_t)rows * (size_t)(cols / e) * (size_t)block_bytes(type);
}

}  // namespace

extern "C" {

size_t ribn_b200_op_last_error(char* buffer, size_t capacity) {
    if (buffer != nullptr && capacity > 0) {
        const size_t n = std::min(capacity - 1, g_op_error.size());
        memcpy(buffer, g_op_error.data(), n);
        buffer[n] = 0;
    }
    return g_op_error.size();
}

int ribn_b200_debug_repack(int32_t type, const void* raw, int64_t rows, int64_t cols, void* out, size_t capacity,
                           size_t* byte_count) {
    if (!packable(type, rows, cols) || raw == nullptr) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    const size_t need = packed_bytes(type, rows, cols);
    if (byte_count) *byte_count = need;
    if (out == nullptr) return RIBN_B200_OK;
    if (capacity < need) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    repack_host(type, (const unsigned char*)raw, rows, cols, (unsigned char*)out, 1);
    return RIBN_B200_OK;
}

int ribn_b200_debug_unpack(int32_t device, int32_t type, const void* packed, int64_t rows, int64_t cols, float* out) {
    if (!packable(type, rows, cols) || packed == nullptr || out == nullptr) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    Scope s(device);
    if (!s.ok) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    unsigned char* d_in = s.upload((const unsigned char*)packed, packed_bytes(type, rows, cols));
    float* d_out = s.alloc<float>((size_t)rows * cols);
    OP_PTR(d_in); OP_PTR(d_out);
    OP_TRY(launch_unpack_packed(s.stream, type, d_in, rows, cols, d_out));
    return s.download(out, d_out, (size_t)rows * cols) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_embedding(int32_t device, int32_t type, const void* table, int32_t vocab, int32_t hidden,
                           const uint32_t* tokens, int32_t count, float* out) {
    const size_t n = encoded_bytes(type, vocab, hidden);
    if (n == 0 || table == nullptr || tokens == nullptr || out == nullptr || count <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    for (int i = 0; i < count; ++i) if (tokens[i] >= (uint32_t)vocab) return op_fail("token id out of range", cudaSuccess);
    Scope s(device);
    if (!s.ok) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    unsigned char* d_t = s.upload((const unsigned char*)table, n);
    uint32_t* d_ids = s.upload(tokens, (size_t)count);
    float* d_o = s.alloc<float>((size_t)count * hidden);
    OP_PTR(d_t); OP_PTR(d_ids); OP_PTR(d_o);
    OP_TRY(launch_embedding(s.stream, type, d_t, hidden, vocab, d_ids, count, d_o));
    return s.download(out, d_o, (size_t)count * hidden) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_qk_norm_rope_append(int32_t device, float* q, float* k, const float* v, const float* q_norm,
                                     const float* k_norm, const int32_t* positions, const int32_t* kv_slots,
                                     int32_t tokens, int32_t q_heads, int32_t kv_heads, int32_t head_dim, float rope_base,
                                     float eps, uint16_t* cache_k, uint16_t* cache_v, int32_t physical_tokens) {
    Scope s(device);
    if (!s.ok || tokens <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) || physical_tokens <= 0) {
        return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    }
    for (int i = 0; i < tokens; ++i) {
        if (kv_slots[i] < 0 || kv_slots[i] >= physical_tokens || positions[i] < 0) return op_fail("slot or position out of range", cudaSuccess);
    }
    const size_t qn = (size_t)tokens * q_heads * head_dim, kn = (size_t)tokens * kv_heads * head_dim;
    const size_t cache_elems = (size_t)physical_tokens * kv_heads * head_dim;
    std::vector<float> table((size_t)head_dim / 2);
    for (int p = 0; p < head_dim / 2; ++p) table[p] = powf(rope_base, -(2.0f * (float)p) / (float)head_dim);
    float* d_q = s.upload(q, qn);
    float* d_k = s.upload(k, kn);
    float* d_v = s.upload(v, kn);
    float* d_qn = s.upload(q_norm, (size_t)head_dim);
    float* d_kn = s.upload(k_norm, (size_t)head_dim);
    float* d_t = s.upload(table.data(), table.size());
    int32_t* d_pos = s.upload(positions, (size_t)tokens);
    int32_t* d_slot = s.upload(kv_slots, (size_t)tokens);
    uint16_t* d_ck = s.upload(cache_k, cache_elems);
    uint16_t* d_cv = s.upload(cache_v, cache_elems);
    OP_PTR(d_q); OP_PTR(d_k); OP_PTR(d_v); OP_PTR(d_qn); OP_PTR(d_kn); OP_PTR(d_t); OP_PTR(d_pos); OP_PTR(d_slot);
    OP_PTR(d_ck); OP_PTR(d_cv);
    OP_TRY(launch_qk_norm_rope_append(s.stream, d_q, d_k, d_v, d_qn, d_kn, d_t, d_pos, d_slot, tokens, q_heads, kv_heads,
                                      head_dim, eps, (__half*)d_ck, (__half*)d_cv));
    bool ok = s.download(q, d_q, qn) && s.download(k, d_k, kn);
    ok = ok && s.download(cache_k, d_ck, cache_elems) && s.download(cache_v, d_cv, cache_elems);
    return ok ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_attention_decode(int32_t device, const float* q, const float* k, const float* v, const float* q_norm,
                                  const float* k_norm, float rope_base, float eps, uint16_t* cache_k, uint16_t* cache_v,
                                  int32_t physical_tokens, const int32_t* page_tables, int32_t pages_per_sequence,
                                  const int32_t* positions, int32_t members, int32_t q_heads, int32_t kv_heads,
                                  int32_t head_dim, float* out) {
    Scope s(device);
    if (!s.ok || members <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || pages_per_sequence <= 0 ||
        (head_dim != 64 && head_dim != 128 && head_dim != 256) || physical_tokens <= 0) {
        return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    }
    std::vector<int32_t> seq(members), slot(members);
    int max_keys = 0;
    for (int m = 0; m < members; ++m) {
        const int pos = positions[m];
        if (pos < 0 || pos / kPageTokens >= pages_per_sequence) return op_fail("position outside the page table", cudaSuccess);
        const int page = page_tables[(size_t)m * pages_per_sequence + pos / kPageTokens];
        if (page < 0 || (page + 1) * kPageTokens > physical_tokens) return op_fail("page outside the cache", cudaSuccess);
        seq[m] = m;
        slot[m] = page * kPageTokens + pos % kPageTokens;
        max_keys = std::max(max_keys, pos + 1);
    }
    const size_t qn = (size_t)members * q_heads * head_dim, kn = (size_t)members * kv_heads * head_dim;
    const size_t cache_elems = (size_t)physical_tokens * kv_heads * head_dim;
    std::vector<float> table((size_t)head_dim / 2);
    for (int p = 0; p < head_dim / 2; ++p) table[p] = powf(rope_base, -(2.0f * (float)p) / (float)head_dim);
    DecodeAttention d{};
    d.q = s.upload(q, qn); d.k = s.upload(k, kn); d.v = s.upload(v, kn);
    d.q_norm = s.upload(q_norm, (size_t)head_dim); d.k_norm = s.upload(k_norm, (size_t)head_dim);
    d.inv_freq = s.upload(table.data(), table.size());
    d.eps = eps;
    d.cache_k = (__half*)s.upload(cache_k, cache_elems);
    d.cache_v = (__half*)s.upload(cache_v, cache_elems);
    d.page_tables = s.upload(page_tables, (size_t)members * pages_per_sequence);
    d.pages_per_sequence = pages_per_sequence;
    d.token_seq = s.upload(seq.data(), seq.size());
    d.token_pos = s.upload(positions, (size_t)members);
    d.token_slot = s.upload(slot.data(), slot.size());
    d.n_tokens = members; d.q_heads = q_heads; d.kv_heads = kv_heads; d.head_dim = head_dim;
    d.window = 0; d.max_keys = max_keys;
    const size_t spans = ((size_t)max_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
    d.partial_bytes = (size_t)members * q_heads * spans * (head_dim + 2) * sizeof(float);
    d.partial = s.alloc<float>(d.partial_bytes / sizeof(float));
    float* d_out = s.alloc<float>(qn);
    d.out = d_out;
    d.programmatic = false;
    OP_PTR(d.q); OP_PTR(d.k); OP_PTR(d.v); OP_PTR(d.q_norm); OP_PTR(d.k_norm); OP_PTR(d.inv_freq); OP_PTR(d.cache_k);
    OP_PTR(d.cache_v); OP_PTR(d.page_tables); OP_PTR(d.token_seq); OP_PTR(d.token_pos); OP_PTR(d.token_slot);
    OP_PTR(d.partial); OP_PTR(d_out);
    OP_TRY(launch_attention_decode(s.stream, d, nullptr));
    bool ok = s.download(out, d_out, qn);
    ok = ok && s.download(cache_k, (uint16_t*)d.cache_k, cache_elems) && s.download(cache_v, (uint16_t*)d.cache_v, cache_elems);
    return ok ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_dequantize(int32_t device, int32_t type, const void* bytes, int64_t rows, int64_t cols, float* out) {
    const size_t n = encoded_bytes(type, rows, cols);
    if (n == 0 || bytes == nullptr || out == nullptr) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    Scope s(device);
    if (!s.ok) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    unsigned char* d_in = s.upload((const unsigned char*)bytes, n);
    float* d_out = s.alloc<float>((size_t)rows * cols);
    OP_PTR(d_in); OP_PTR(d_out);
    OP_TRY(launch_dequantize(s.stream, type, d_in, rows, cols, d_out));
    return s.download(out, d_out, (size_t)rows * cols) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_gemv(int32_t device, int32_t type, const void* weights, int64_t rows, int64_t cols, const float* x,
                      int32_t members, float* y, int32_t variant) {
    const size_t n = encoded_bytes(type, rows, cols);
    if (n == 0 || weights == nullptr || x == nullptr || y == nullptr || members <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    Scope s(device);
    if (!s.ok) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    float* d_x = s.upload(x, (size_t)members * cols);
    float* d_y = s.alloc<float>((size_t)members * rows);
    OP_PTR(d_x); OP_PTR(d_y);
    if (variant == 1) {
        unsigned char* d_w = s.upload((const unsigned char*)weights, n);
        OP_PTR(d_w);
        OP_TRY(launch_gemv_ref(s.stream, type, d_w, rows, cols, d_x, members, d_y, false));
    } else {
        if (!packable(type, rows, cols)) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
        std::vector<unsigned char> packed(packed_bytes(type, rows, cols));
        repack_host(type, (const unsigned char*)weights, rows, cols, packed.data(),
                    (int)std::max(1u, std::min(16u, std::thread::hardware_concurrency())));
        unsigned char* d_w = s.upload(packed.data(), packed.size());
        OP_PTR(d_w);
        ActOperand op;
        op.dig = s.alloc<signed char>((size_t)members * 3 * cols);
        op.sx = s.alloc<float>((size_t)members * (cols / 32));
        op.sxs16 = s.alloc<float>((size_t)members * (cols / 16));
        op.ss32 = nullptr;
        int* d_err = s.alloc<int>(1);
        OP_PTR(op.dig); OP_PTR(op.sx); OP_PTR(op.sxs16); OP_PTR(d_err);
        OP_TRY(cudaMemsetAsync(d_err, 0, sizeof(int), s.stream));
        if (variant == 3 || variant == 4 || variant == 5) {
            // the tensor-memory kernels
            TcOperand top;
            const GemvSegment probe{d_w, type, (int)rows, (int)((rows + kTileRows - 1) / kTileRows), d_y};
            // variant 3: K-quant form where it applies (at most 64 members per launch); variant 4: always the generic form;
            // variant 5: the K-quant form over operands converted once (Q4_K and Q6_K only)
            const bool kquant = variant != 4 && gemm_tc_kquant(&probe, 1, 1);
            unsigned char *op_a = nullptr, *op_meta = nullptr;
            if (variant == 5) {
                if (!kquant) return op_fail("gemv: the operand cache holds Q4_K and Q6_K matrices only", cudaSuccess);
                op_a = s.alloc<unsigned char>(tc_cache_a_bytes(type, rows, cols));
                op_meta = s.alloc<unsigned char>(tc_cache_meta_bytes(rows, cols));
                OP_PTR(op_a); OP_PTR(op_meta);
                OP_TRY(launch_tc_cache(s.stream, type, d_w, rows, cols, op_a, op_meta));
            }
            const int per_launch = kquant ? 64 : kGemmTcMaxMembers;
            const int group = std::min(members, per_launch);
            top.chunks = (__half*)s.alloc<unsigned char>(tc_operand_bytes(group, (int)cols));
            top.scale_in = s.alloc<float>((size_t)group);
            top.member_scale = s.alloc<float>((size_t)group);
            OP_PTR(top.chunks); OP_PTR(top.scale_in); OP_PTR(top.member_scale);
            const size_t partial_floats = (size_t)8 * group * (size_t)rows;
            float* partial = kquant ? s.alloc<float>(partial_floats) : nullptr;
            if (kquant) OP_PTR(partial);
            int m_first = 0;
            if (kquant && members >= 2 * per_launch) {
                // whole groups of 64 rows in one launch, as a prefill step runs them (pairs of groups share
                // each converted weight stage)
                const int whole = members / per_launch;
                TcOperand all;
                all.chunks = (__half*)s.alloc<unsigned char>((size_t)whole * tc_operand_bytes(per_launch, (int)cols));
                all.scale_in = s.alloc<float>((size_t)whole * per_launch);
                all.member_scale = s.alloc<float>((size_t)whole * per_launch);
                OP_PTR(all.chunks); OP_PTR(all.scale_in); OP_PTR(all.member_scale);
                OP_TRY(launch_to_tc_operand_groups(s.stream, d_x, nullptr, nullptr, whole * per_launch, per_launch, (int)cols, 0.0f, all));
                GemmArgs a{};
                a.n_segments = 1;
                a.seg[0] = GemvSegment{d_w, type, (int)rows, (int)((rows + kTileRows - 1) / kTileRows), d_y, op_a, op_meta};
                a.k = (int)cols;
                a.members = per_launch;
                a.chunks = (const signed char*)all.chunks; a.member_scale = all.member_scale;
                a.epilogue = kStore;
                a.error_flag = d_err;
                a.kquant = 1;
                a.groups = whole;
                a.group_chunk_bytes = tc_operand_bytes(per_launch, (int)cols);
                OP_TRY(launch_gemm_tc(s.stream, a));
                m_first = whole * per_launch;
            }
            for (int m0 = m_first; m0 < members; m0 += per_launch) {
                const int m = std::min(per_launch, members - m0);
                OP_TRY(launch_to_tc_operand(s.stream, d_x + (size_t)m0 * cols, nullptr, nullptr, m, (int)cols, 0.0f, kquant, top));
                GemmArgs a{};
                a.n_segments = 1;
                a.seg[0] = GemvSegment{d_w, type, (int)rows, (int)((rows + kTileRows - 1) / kTileRows),
                                       d_y + (size_t)m0 * rows, op_a, op_meta};
                a.k = (int)cols;
                a.members = m;
                a.chunks = (const signed char*)top.chunks; a.member_scale = top.member_scale;
                a.epilogue = kStore;
                a.error_flag = d_err;
                a.kquant = kquant ? 1 : 0;
                a.partial = partial;
                a.partial_floats = partial_floats;
                OP_TRY(launch_gemm_tc(s.stream, a));
            }
        } else if (variant == 2) {
            // the batched kernel, in groups of up to kGemmMaxMembers members
            BatchOperand bop;
            const int group = std::min(members, kGemmMaxMembers);
            bop.chunks = s.alloc<signed char>(batch_operand_bytes(group, (int)cols));
            bop.member_scale = s.alloc<float>((size_t)group);
            bop.digit_inv = s.alloc<float>((size_t)group);
            OP_PTR(bop.chunks); OP_PTR(bop.member_scale); OP_PTR(bop.digit_inv);
            for (int m0 = 0; m0 < members; m0 += kGemmMaxMembers) {
                const int m = std::min(kGemmMaxMembers, members - m0);
                OP_TRY(launch_to_batch_operand(s.stream, d_x + (size_t)m0 * cols, nullptr, nullptr, m, (int)cols, 0.0f, bop));
                GemmArgs a{};
                a.n_segments = 1;
                a.seg[0] = GemvSegment{d_w, type, (int)rows, (int)((rows + kTileRows - 1) / kTileRows),
                                       d_y + (size_t)m0 * rows};
                a.k = (int)cols;
                a.members = m;
                a.chunks = bop.chunks; a.member_scale = bop.member_scale;
                a.epilogue = kStore;
                a.error_flag = d_err;
                OP_TRY(launch_gemm_imma(s.stream, a));
            }
        } else {
        OP_TRY(launch_to_operand(s.stream, d_x, nullptr, nullptr, members, (int)cols, op));
        for (int m0 = 0; m0 < members; m0 += kGemvMaxMembers) {
            GemvArgs a{};
            a.n_segments = 1;
            a.seg[0] = GemvSegment{d_w, type, (int)rows, (int)((rows + kTileRows - 1) / kTileRows),
                                   d_y + (size_t)m0 * rows};
            a.k = (int)cols;
            a.members = std::min(kGemvMaxMembers, members - m0);
            a.in.dig = op.dig + (size_t)m0 * 3 * cols;
            a.in.sx = op.sx + (size_t)m0 * (cols / 32);
            a.in.sxs16 = op.sxs16 + (size_t)m0 * (cols / 16);
            a.in_has_norm = 0;
            a.eps = 0.0f;
            a.epilogue = kStore;
            a.error_flag = d_err;
            OP_TRY(launch_gemv_mma(s.stream, a, false));
        }
        }
        int err = 0;
        if (!s.download(&err, d_err, 1)) return op_fail("gemv", cudaGetLastError());
        if (err != 0) return op_fail("gemv: a bounded wait inside the kernel expired", cudaSuccess);
    }
    return s.download(y, d_y, (size_t)members * rows) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_rms_norm(int32_t device, const float* x, const float* weight, int32_t members, int32_t length,
                          float eps, float* out) {
    Scope s(device);
    if (!s.ok || members <= 0 || length <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    float* d_x = s.upload(x, (size_t)members * length);
    float* d_w = s.upload(weight, (size_t)length);
    float* d_o = s.alloc<float>((size_t)members * length);
    OP_PTR(d_x); OP_PTR(d_w); OP_PTR(d_o);
    OP_TRY(launch_rms_norm(s.stream, d_x, d_w, members, length, eps, d_o));
    return s.download(out, d_o, (size_t)members * length) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_silu_mul(int32_t device, const float* gate, const float* up, int64_t length, float* out) {
    Scope s(device);
    if (!s.ok || length <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    float* d_g = s.upload(gate, (size_t)length);
    float* d_u = s.upload(up, (size_t)length);
    float* d_o = s.alloc<float>((size_t)length);
    OP_PTR(d_g); OP_PTR(d_u); OP_PTR(d_o);
    OP_TRY(launch_silu_mul(s.stream, d_g, d_u, length, d_o));
    return s.download(out, d_o, (size_t)length) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_gdn_step(int32_t device, int32_t members, int32_t tokens, int32_t k_heads, int32_t v_heads, int32_t head_dim,
                          const float* qkv, const float* z, const float* beta_raw, const float* alpha_raw,
                          const float* dt_bias, const float* a, const float* conv_weight, const float* norm_weight,
                          float* conv_state, float* state, float l2_eps, float norm_eps, float* decay, float* beta,
                          float* conv_act, float* attn_out, float* out) {
    Scope s(device);
    if (!s.ok || members <= 0 || tokens <= 0 || k_heads <= 0 || v_heads <= 0 || v_heads % k_heads != 0 || (head_dim != 64 && head_dim != 128)) {
        return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    }
    const size_t hd = (size_t)head_dim, channels = (size_t)(2 * k_heads + v_heads) * hd, inner = (size_t)v_heads * hd;
    const size_t conv_elems = channels * 3, state_elems = inner * hd;
    GdnStep g{};
    g.members = members; g.tokens = tokens; g.k_heads = k_heads; g.v_heads = v_heads; g.head_dim = head_dim;
    g.channels = (int)channels; g.k_offset = (int)(k_heads * hd); g.v_offset = (int)(2 * k_heads * hd);
    const size_t rows = (size_t)members * tokens;
    g.qkv = s.upload(qkv, rows * channels);
    g.z = s.upload(z, rows * inner);
    g.beta_raw = s.upload(beta_raw, rows * v_heads);
    g.alpha_raw = s.upload(alpha_raw, rows * v_heads);
    g.dt_bias = s.upload(dt_bias, (size_t)v_heads);
    g.a = s.upload(a, (size_t)v_heads);
    g.conv_weight = s.upload(conv_weight, channels * 4);
    g.norm_weight = s.upload(norm_weight, hd);
    float* d_conv = s.upload(conv_state, (size_t)members * conv_elems);
    float* d_state = s.upload(state, (size_t)members * state_elems);
    OP_PTR(g.qkv); OP_PTR(g.z); OP_PTR(g.beta_raw); OP_PTR(g.alpha_raw); OP_PTR(g.dt_bias); OP_PTR(g.a);
    OP_PTR(g.conv_weight); OP_PTR(g.norm_weight); OP_PTR(d_conv); OP_PTR(d_state);
    std::vector<float*> conv_ptrs((size_t)members), state_ptrs((size_t)members);
    for (int m = 0; m < members; ++m) { conv_ptrs[m] = d_conv + (size_t)m * conv_elems; state_ptrs[m] = d_state + (size_t)m * state_elems; }
    float** d_conv_ptrs = s.upload(conv_ptrs.data(), (size_t)members);
    float** d_state_ptrs = s.upload(state_ptrs.data(), (size_t)members);
    OP_PTR(d_conv_ptrs); OP_PTR(d_state_ptrs);
    g.conv_state = d_conv_ptrs; g.state = d_state_ptrs;
    g.l2_eps = l2_eps; g.norm_eps = norm_eps;
    g.decay = s.alloc<float>(rows * v_heads);
    g.beta = s.alloc<float>(rows * v_heads);
    g.conv_act = s.alloc<float>(rows * channels);
    g.attn_out = s.alloc<float>(rows * inner);
    g.out = s.alloc<float>(rows * inner);
    OP_PTR(g.decay); OP_PTR(g.beta); OP_PTR(g.conv_act); OP_PTR(g.attn_out); OP_PTR(g.out);
    OP_TRY(launch_gdn_step(s.stream, g));
    bool ok = s.download(conv_state, d_conv, (size_t)members * conv_elems) && s.download(state, d_state, (size_t)members * state_elems) &&
              s.download(out, g.out, rows * inner);
    if (ok && decay) ok = s.download(decay, g.decay, rows * v_heads);
    if (ok && beta) ok = s.download(beta, g.beta, rows * v_heads);
    if (ok && conv_act) ok = s.download(conv_act, g.conv_act, rows * channels);
    if (ok && attn_out) ok = s.download(attn_out, g.attn_out, rows * inner);
    return ok ? RIBN_B200_OK : op_fail("download of the step's results", cudaGetLastError());
}

int ribn_b200_op_attention_gate(int32_t device, const float* attn, const float* q_gate, int64_t rows, int32_t heads,
                                int32_t head_dim, float* out) {
    Scope s(device);
    if (!s.ok || rows <= 0 || heads <= 0 || head_dim <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    const size_t n = (size_t)rows * heads * head_dim;
    float* d_a = s.upload(attn, n);
    float* d_g = s.upload(q_gate, 2 * n);
    float* d_o = s.alloc<float>(n);
    OP_PTR(d_a); OP_PTR(d_g); OP_PTR(d_o);
    OP_TRY(launch_attention_gate(s.stream, d_a, d_g, rows, heads, head_dim, d_o));
    return s.download(out, d_o, n) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_argmax(int32_t device, const float* logits, int32_t members, int64_t length, uint32_t* out) {
    Scope s(device);
    if (!s.ok || members <= 0 || length <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    float* d_l = s.upload(logits, (size_t)members * length);
    uint32_t* d_o = s.alloc<uint32_t>((size_t)members);
    OP_PTR(d_l); OP_PTR(d_o);
    OP_TRY(launch_argmax(s.stream, d_l, members, length, d_o));
    return s.download(out, d_o, (size_t)members) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_rope_neox(int32_t device, float* values, const int64_t* positions, int32_t members, int32_t heads,
                           int32_t head_dim, int32_t rot_dims, float base) {
    Scope s(device);
    if (!s.ok || members <= 0 || rot_dims <= 0 || rot_dims > head_dim || (rot_dims & 1)) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    const size_t n = (size_t)members * heads * head_dim;
    std::vector<float> table((size_t)rot_dims / 2);
    for (int p = 0; p < rot_dims / 2; ++p) table[p] = powf(base, -(2.0f * (float)p) / (float)rot_dims);
    std::vector<long long> pos(positions, positions + members);
    float* d_v = s.upload(values, n);
    float* d_t = s.upload(table.data(), table.size());
    long long* d_p = s.upload(pos.data(), pos.size());
    OP_PTR(d_v); OP_PTR(d_t); OP_PTR(d_p);
    OP_TRY(launch_rope_neox(s.stream, d_v, d_p, members, heads, head_dim, rot_dims, d_t));
    return s.download(values, d_v, n) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_f32_to_f16(int32_t device, const float* in, int64_t length, uint16_t* out) {
    Scope s(device);
    if (!s.ok || length <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    float* d_i = s.upload(in, (size_t)length);
    uint16_t* d_o = s.alloc<uint16_t>((size_t)length);
    OP_PTR(d_i); OP_PTR(d_o);
    OP_TRY(launch_f32_to_f16(s.stream, d_i, length, d_o));
    return s.download(out, d_o, (size_t)length) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_attention(int32_t device, const float* q, const uint16_t* keys, const uint16_t* values,
                           const int32_t* page_table, int32_t page_tokens, int32_t physical_tokens, int32_t tokens,
                           int32_t rows, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t window,
                           float* out, int32_t variant) {
    Scope s(device);
    if (!s.ok || rows <= 0 || tokens < rows || page_tokens != kPageTokens || q_heads % kv_heads != 0) {
        return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    }
    const int pages = (tokens + page_tokens - 1) / page_tokens;
    const size_t kv_elems = (size_t)physical_tokens * kv_heads * head_dim;
    float* d_q = s.upload(q, (size_t)rows * q_heads * head_dim);
    __half* d_k = (__half*)s.upload(keys, kv_elems);
    __half* d_v = (__half*)s.upload(values, kv_elems);
    int32_t* d_table = s.upload(page_table, (size_t)pages);
    std::vector<int32_t> seq(rows, 0), pos(rows);
    for (int r = 0; r < rows; ++r) pos[r] = tokens - rows + r;  // row r attends tokens - rows + 1 + r keys
    int32_t* d_seq = s.upload(seq.data(), seq.size());
    int32_t* d_pos = s.upload(pos.data(), pos.size());
    float* d_o = s.alloc<float>((size_t)rows * q_heads * head_dim);
    OP_PTR(d_q); OP_PTR(d_k); OP_PTR(d_v); OP_PTR(d_table); OP_PTR(d_seq); OP_PTR(d_pos); OP_PTR(d_o);
    if (variant == 1) {
        OP_TRY(launch_attention_ref(s.stream, d_q, d_k, d_v, d_table, pages, d_seq, d_pos, rows, q_heads, kv_heads,
                                    head_dim, window, d_o));
    } else {
        const size_t spans = ((size_t)tokens + kAttnSpanKeys - 1) / kAttnSpanKeys;
        // span accumulators for every row when that is small, else 256 MiB (the rows then run in several launches)
        const size_t per_row = (size_t)q_heads * spans * (head_dim + 2) * sizeof(float);
        const size_t bytes = std::max(per_row, std::min(per_row * (size_t)rows, (size_t)256 << 20));
        float* d_partial = s.alloc<float>(bytes / sizeof(float));
        OP_PTR(d_partial);
        OP_TRY(launch_attention(s.stream, d_q, d_k, d_v, d_table, pages, d_seq, d_pos, rows, q_heads, kv_heads,
                                head_dim, window, tokens, d_partial, bytes, d_o, nullptr, 0, rows));
    }
    return s.download(out, d_o, (size_t)rows * q_heads * head_dim) ? RIBN_B200_OK : RIBN_B200_ERROR;
}

int ribn_b200_op_batch_metadata(int32_t device, const int32_t* row_slot, const int32_t* row_prefix,
                                const int32_t* row_tokens, int32_t rows, const int32_t* page_tables,
                                int32_t pages_per_sequence, int32_t page_tokens, int32_t* cu_seqlens,
                                int32_t* token_row, int32_t* token_position, int32_t* token_kv_slot) {
    Scope s(device);
    if (!s.ok || rows <= 0 || page_tokens <= 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
    int total = 0, max_slot = 0;
    for (int r = 0; r < rows; ++r) {
        if (row_tokens[r] < 0 || row_slot[r] < 0) return op_fail("invalid argument, or no usable CUDA device", cudaGetLastError());
        total += row_tokens[r];
        max_slot = std::max(max_slot, row_slot[r]);
    }
    int32_t* d_slot = s.upload(row_slot, (size_t)rows);
    int32_t* d_prefix = s.upload(row_prefix, (size_t)rows);
    int32_t* d_tokens = s.upload(row_tokens, (size_t)rows);
    int32_t* d_tables = s.upload(page_tables, (size_t)(max_slot + 1) * pages_per_sequence);
    int32_t* d_cu = s.alloc<int32_t>((size_t)rows + 1);
    int32_t* d_row = s.alloc<int32_t>((size_t)total);
    int32_t* d_pos = s.alloc<int32_t>((size_t)total);
    int32_t* d_kv = s.alloc<int32_t>((size_t)total);
    OP_PTR(d_slot); OP_PTR(d_prefix); OP_PTR(d_tokens); OP_PTR(d_tables); OP_PTR(d_cu); OP_PTR(d_row); OP_PTR(d_pos);
    OP_PTR(d_kv);
    OP_TRY(launch_batch_metadata(s.stream, d_slot, d_prefix, d_tokens, rows, total, d_tables, pages_per_sequence,
                                 page_tokens, d_cu, d_row, d_pos, d_kv));
    bool ok = s.download(cu_seqlens, d_cu, (size_t)rows + 1);
    ok = ok && s.download(token_row, d_row, (size_t)total);
    ok = ok && s.download(token_position, d_pos, (size_t)total);
    ok = ok && s.download(token_kv_slot, d_kv, (size_t)total);
    return ok ? RIBN_B200_OK : RIBN_B200_ERROR;
}

}  // extern "C"
