// Paged-KV ragged attention for decode rows and prefill chunks: split-KV
// ("flash-decoding") over spans of 64-key tiles with an online softmax, then a
// deterministic merge of the spans.
//
// Launches run the tensor-core span kernel below (the GQA group's query heads
// against 16-key slices as m16n8k16 MMAs, K / V staged in shared memory by
// asynchronous copies), then the merge kernel; the whole sixteen-token groups
// of a prefill chunk run the prefill kernel instead (a key tile staged once per
// group, every warp walks all the keys of its own tokens, no merge).  A token's
// result depends only on its own keys and on the launch's size class (tiles
// per span; chunk or not), never on where its pages live.
//
// The decode form (FUSED) also applies the per-head Q/K RMSNorm and the NeoX
// rotary and appends the new K/V row to the paged cache: the CTA that owns
// the span holding the token's own position computes that row, stores it, and
// serves it to its warps from shared memory.  Results leave in F32 and,
// optionally, in the tensor-core operand form the output projection consumes.
//
// The reference's two-pass form with a global scores buffer
// (crates/nvidia/src/model_ops.rs:441-545) is replaced, not translated.
#include <cuda_fp16.h>
#include <math.h>

#include <algorithm>

#include "gemv.cuh"
#include "kernels.cuh"
#include "operand.cuh"

namespace ribn {

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct AttnArgs {
    const float* q;            // [T][q_heads][HD]; raw projections when fused
    const float* k_new;        // [T][kv_heads][HD] raw (fused only)
    const float* v_new;        // [T][kv_heads][HD] (fused only)
    const float* q_norm;       // [HD] (fused only)
    const float* k_norm;       // [HD] (fused only)
    const float* inv_freq;     // [HD / 2] (fused only)
    float eps;
    __half* cache_k;
    __half* cache_v;
    const int32_t* page_tables;
    int pages_per_sequence;
    const int32_t* token_seq;
    const int32_t* token_pos;
    const int32_t* token_slot; // physical slot of the token's own position (fused only)
    int token_base;
    int q_heads, kv_heads, window, max_spans;
    int tiles;                 // 64-key tiles per span (tensor-core span kernel and its merge); 1 elsewhere
    int run_tokens;            // up to this many consecutive tokens of a sequence share one item (prefill launches); 1: none
    int run_first, run_count;  // host side: tokens [run_first, run_first + run_count) are consecutive tokens of one sequence; -1: unknown
    float* partial;
    float* out;                // [T][q_heads][HD]
    ActOperand operand;        // optional operand form of `out`, K = q_heads * HD
};

// RMSNorm + NeoX rotary of one head vector held lane-strided: element i of a
// lane is dimension lane + 32 i, so dimension d and its partner d + HD/2 sit
// in the same lane (i and i + DPL/2).
template <int HD>
__device__ __forceinline__ void norm_rope(float (&x)[HD / 32], const float* weight, const float* inv_freq, float eps,
                                          float pos, int lane) {
    constexpr int DPL = HD / 32;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int i = 0; i < DPL; ++i) x[i] = x[i] * inv * weight[lane + 32 * i];
#pragma unroll
    for (int i = 0; i < DPL / 2; ++i) {
        const float theta = pos * inv_freq[lane + 32 * i];
        const float s = sinf(theta), c = cosf(theta);
        const float x0 = x[i], x1 = x[i + DPL / 2];
        x[i] = x0 * c - x1 * s;
        x[i + DPL / 2] = x0 * s + x1 * c;
    }
}

// ---- tensor-core span kernel -----------------------------------------------------------------------
//
// A CTA of four warps walks (token, kv head, span) items; a span is `tiles` consecutive 64-key tiles and
// warp w takes keys [16 w, 16 w + 16) of every tile.  The 16 keys of a slice are the rows of an m16n8k16
// MMA and the query heads of the GQA group its (up to 8, or 2 x 8) columns, so the K / V rows are read
// from shared memory once for the whole group:
//   S^T = K Q^T   A = the K rows as they lie in the cache,
//                 B = Q as binary16 hi + lo (two MMAs: the F32 query loses nothing that matters), held
//                     in registers for the whole item;
//   O^T = V^T P^T A = the V rows through a transposing matrix load,
//                 B = the probabilities as binary16 hi + lo, moved from the S^T accumulator layout to
//                     the operand layout by an 8 x 8 matrix transpose across the warp.
// Products of binary16 values are exact in the F32 accumulators.  Each warp is a pipeline of its own: it
// copies its next 16-row slice into the second of two shared-memory slots while it multiplies the first
// (asynchronous copies it alone waits for; no CTA-wide barrier inside the loop) and keeps an online
// softmax over its slices; the first slice of the CTA's next item is requested under the last slice of
// the current one.  The four warps' results are folded in warp order and the spans in span order,
// so a token's result depends on its own keys and on `tiles`, never on its neighbours in the batch or on
// where its pages live.
constexpr int kMmaWarps = 4;
constexpr int kMmaKeys = kAttnSpanKeys / kMmaWarps;  // keys per warp and tile
static_assert(kMmaKeys == 16, "one k16 step of P.V per warp");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
// x = hi + lo with both binary16; returns the pair packed for two neighbouring values
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    const float2 back = __half22float2(h);
    const __half2 l = __floats2half2_rn(x0 - back.x, x1 - back.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

__device__ __forceinline__ int token_spans(const AttnArgs& a, int pos) {
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int span_keys = kAttnSpanKeys * a.tiles;
    return (pos + 1 - first + span_keys - 1) / span_keys;
}

// One warp merges the spans of one (token, q head) in span order:
// out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M).  Lane = dimension lane + 32 i.  The first
// group of spans' values is requested together with the maxima, so a short context costs one round trip.
template <int HD>
__device__ __forceinline__ void merge_head(const AttnArgs& a, int t, int qh, int spans, int lane) {
    constexpr int DPL = HD / 32;
    constexpr int REC = HD + 2;
    constexpr int GROUP = DPL <= 4 ? 16 : 8;  // spans whose values are in flight together
    const float* pp = a.partial + ((long long)(t - a.token_base) * a.q_heads + qh) * a.max_spans * REC;
    float v[GROUP][DPL];
#pragma unroll
    for (int u = 0; u < GROUP; ++u) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) v[u][i] = u < spans ? __ldcg(pp + u * REC + lane + 32 * i) : 0.0f;
    }
    float top = -INFINITY;
    float denom = 0.0f;  // per-lane partial sums in span order, folded in a fixed shuffle order
    for (int s = lane; s < spans; s += 32) top = fmaxf(top, __ldcg(pp + s * REC + HD));
    top = warp_max(top);
    for (int s = lane; s < spans; s += 32) denom = fmaf(__ldcg(pp + s * REC + HD + 1), __expf(__ldcg(pp + s * REC + HD) - top), denom);
    denom = warp_sum(denom);
    float sum[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) sum[i] = 0.0f;
    for (int s0 = 0; s0 < spans; s0 += GROUP) {
        const float mine = s0 + lane < spans ? __expf(__ldcg(pp + (s0 + lane) * REC + HD) - top) : 0.0f;
        if (s0 > 0) {
#pragma unroll
            for (int u = 0; u < GROUP; ++u) {
#pragma unroll
                for (int i = 0; i < DPL; ++i) v[u][i] = s0 + u < spans ? __ldcg(pp + (s0 + u) * REC + lane + 32 * i) : 0.0f;
            }
        }
#pragma unroll
        for (int u = 0; u < GROUP; ++u) {
            const float w = __shfl_sync(0xffffffffu, mine, u);
            if (s0 + u < spans) {
#pragma unroll
                for (int i = 0; i < DPL; ++i) sum[i] = fmaf(v[u][i], w, sum[i]);
            }
        }
    }
    ActOperand op = a.operand;
    op.ss32 = nullptr;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const float value = sum[i] / denom;
        a.out[((long long)t * a.q_heads + qh) * HD + lane + 32 * i] = value;
        if (op.dig != nullptr) operand_store_span(op, t - a.token_base, a.q_heads * HD, (qh * HD) / 32 + i, lane, value, 0.0f);
    }
}

template <int HD>
struct MmaLayout {
    static constexpr int RH = HD + 8;                    // halfs per staged row: 16 bytes of padding keep the matrix loads conflict-free
    static constexpr int STAGES = 2;                     // ring slots per warp: one slice multiplied, the next in flight
    static constexpr int SLOT = 2 * kMmaKeys * RH;       // halfs per slot: 16 K rows, then 16 V rows
    // [query rows: heads of the group x tokens of a run] hi, the same lo, the token's own K / V row, then the rings
    static size_t bytes(int q_rows) {
        return ((size_t)2 * q_rows * RH + 2 * RH + (size_t)kMmaWarps * STAGES * SLOT) * sizeof(__half);
    }
};

// One 16-key slice against the item's columns: S^T = K Q^T, the columns' online softmax, O^T += V^T P^T.
// `k_w`: the slice's 16 K rows followed by its 16 V rows in shared memory; `wbegin`: its first key; lim[nt][j]:
// the last key column 8 nt + 2 t4 + j may see (-1: no such column); `first`: nothing has been accumulated yet.
template <int HD, int NT>
__device__ __forceinline__ void slice_step(const __half* k_w, int wbegin, const int (&lim)[NT][2],
                                           const uint32_t (&qh)[NT][HD / 16][2], const uint32_t (&ql)[NT][HD / 16][2],
                                           float (&o)[NT][HD / 16][4], float (&run_m)[NT][2], float (&run_l)[NT][2],
                                           bool first, float scale, uint32_t k_off, uint32_t v_off, int g) {
    // S^T: keys g (values 0, 1) and g + 8 (values 2, 3) x columns 8 nt + 2 t4 + {0, 1}; the hi and lo
    // products accumulate apart (two shorter dependency chains) and meet at the end
    float sh[NT][4], sl[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { sh[nt][0] = sh[nt][1] = sh[nt][2] = sh[nt][3] = 0.0f; sl[nt][0] = sl[nt][1] = sl[nt][2] = sl[nt][3] = 0.0f; }
    {
        const uint32_t k_at = smem_u32(k_w) + k_off;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t ka[4];
            ldmatrix_x4(ka, k_at + ks * 32);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mma_f16(sh[nt], ka, qh[nt][ks][0], qh[nt][ks][1]);
                mma_f16(sl[nt], ka, ql[nt][ks][0], ql[nt][ks][1]);
            }
        }
    }
    const int key0 = wbegin + g, key1 = key0 + 8;
    uint32_t ph[NT][2], pl[NT][2];
    bool moved = false;
    float f[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float s0 = key0 <= lim[nt][0] ? (sh[nt][0] + sl[nt][0]) * scale : -INFINITY;
        const float s1 = key0 <= lim[nt][1] ? (sh[nt][1] + sl[nt][1]) * scale : -INFINITY;
        const float s2 = key1 <= lim[nt][0] ? (sh[nt][2] + sl[nt][2]) * scale : -INFINITY;
        const float s3 = key1 <= lim[nt][1] ? (sh[nt][3] + sl[nt][3]) * scale : -INFINITY;
        float ma = fmaxf(s0, s2), mb = fmaxf(s1, s3);  // heads 2 t4 and 2 t4 + 1 over this lane's keys
#pragma unroll
        for (int x = 4; x < 32; x <<= 1) {
            ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, x));
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, x));
        }
        ma = fmaxf(ma, run_m[nt][0]); mb = fmaxf(mb, run_m[nt][1]);
        moved = moved || ma != run_m[nt][0] || mb != run_m[nt][1];
        // a column that has seen no key yet (a token of the run whose keys start later) keeps -inf
        const float za = ma == -INFINITY ? 0.0f : ma, zb = mb == -INFINITY ? 0.0f : mb;
        f[nt][0] = __expf(run_m[nt][0] - za); f[nt][1] = __expf(run_m[nt][1] - zb);  // 0 on a column's first keys
        run_m[nt][0] = ma; run_m[nt][1] = mb;
        const float p0 = __expf(s0 - za), p1 = __expf(s1 - zb), p2 = __expf(s2 - za), p3 = __expf(s3 - zb);
        float la = p0 + p2, lb = p1 + p3;
#pragma unroll
        for (int x = 4; x < 32; x <<= 1) {
            la += __shfl_xor_sync(0xffffffffu, la, x);
            lb += __shfl_xor_sync(0xffffffffu, lb, x);
        }
        run_l[nt][0] = fmaf(run_l[nt][0], f[nt][0], la);
        run_l[nt][1] = fmaf(run_l[nt][1], f[nt][1], lb);
        // (key, head pair) -> (head, key pair): the operand layout of P^T
        uint32_t h0, l0, h1, l1;
        split_pair(p0, p1, h0, l0);
        split_pair(p2, p3, h1, l1);
        ph[nt][0] = movmatrix_trans(h0); ph[nt][1] = movmatrix_trans(h1);
        pl[nt][0] = movmatrix_trans(l0); pl[nt][1] = movmatrix_trans(l1);
    }
    if (!first && __any_sync(0xffffffffu, moved)) {  // a factor of exactly 1 changes nothing
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int mt = 0; mt < HD / 16; ++mt) {
                o[nt][mt][0] *= f[nt][0]; o[nt][mt][1] *= f[nt][1]; o[nt][mt][2] *= f[nt][0]; o[nt][mt][3] *= f[nt][1];
            }
        }
    }
    const uint32_t v_at = smem_u32(k_w) + v_off;
#pragma unroll
    for (int mt = 0; mt < HD / 16; ++mt) {
        uint32_t va[4];
        ldmatrix_x4_trans(va, v_at + mt * 32);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            mma_f16(o[nt][mt], va, ph[nt][0], ph[nt][1]);
            mma_f16(o[nt][mt], va, pl[nt][0], pl[nt][1]);
        }
    }
}

// One unit of work: a span of one (token, kv head).
struct SpanItem {
    int t, len, kvh, span, pos, spans, begin, end, n_tiles;   // tokens t .. t + len - 1 at positions pos ..; spans of the last
    const int32_t* table;
    bool owns_self;
};

template <int HD, bool FUSED, int NT>
__global__ void __launch_bounds__(kMmaWarps * 32, HD <= 128 && NT == 1 ? 3 : 1) attention_span_mma_kernel(const AttnArgs a, const int n_tokens) {
    using L = MmaLayout<HD>;
    constexpr int DPL = HD / 32;
    constexpr int RH = L::RH;
    constexpr int CPR = HD / 8;       // 16-byte pieces per row
    constexpr int REC = HD + 2;       // floats per head record: accumulators, maximum, sum
    constexpr int STAGES = L::STAGES;
    static_assert(STAGES == 2, "the slot arithmetic below alternates two slots");
    extern __shared__ __align__(16) unsigned char attn_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q_per_kv = a.q_heads / a.kv_heads;
    const int q_rows = q_per_kv * a.run_tokens;
    __half* q_hi = reinterpret_cast<__half*>(attn_smem);       // [q_rows][RH]: column = token of the run x head of the group
    __half* q_lo = q_hi + q_rows * RH;
    __half* k_self = q_lo + q_rows * RH;                       // [RH]
    __half* v_self = k_self + RH;                              // [RH]
    __half* ring = v_self + RH + warp * (STAGES * L::SLOT);    // this warp's slots
    const long long row_stride = (long long)a.kv_heads * HD;
    const int span_keys = kAttnSpanKeys * a.tiles;
    const int total_items = n_tokens * a.kv_heads * a.max_spans;

    // The CTA walks items blockIdx.x, blockIdx.x + gridDim.x, ...; spans past a token's last key are skipped.
    // Positions and page tables were written by kernels that completed before the projection ahead of
    // this one began, so they may be read before the programmatic dependency resolves.
    auto next_item = [&](int& id, SpanItem& it) -> bool {
        for (id += gridDim.x; id < total_items; id += gridDim.x) {
            it.span = id % a.max_spans;
            const int tk = id / a.max_spans;
            it.kvh = tk % a.kv_heads;
            const int local = tk / a.kv_heads;
            it.t = a.token_base + local;
            it.pos = a.token_pos[it.t];
            it.len = 1;
            const int seq = a.token_seq != nullptr ? a.token_seq[it.t] : 0;
            if (a.run_tokens > 1) {
                // Consecutive tokens of one sequence see the same keys up to the diagonal: the run that starts at an
                // aligned token, or at one that does not continue its predecessor, is served by its first token's
                // item; the run's other tokens have no item of their own.
                const int in_group = local % a.run_tokens;
                if (in_group != 0) {
                    const int seq_before = a.token_seq != nullptr ? a.token_seq[it.t - 1] : 0;
                    if (seq_before == seq && a.token_pos[it.t - 1] + 1 == it.pos) continue;
                }
                while (it.len < a.run_tokens - in_group && local + it.len < n_tokens &&
                       (a.token_seq != nullptr ? a.token_seq[it.t + it.len] : 0) == seq && a.token_pos[it.t + it.len] == it.pos + it.len) {
                    ++it.len;
                }
            }
            const int last = it.pos + it.len - 1;
            const int first = a.window > 0 ? max(0, it.pos - a.window + 1) : 0;   // runs only without a window
            it.spans = (last + 1 - first + span_keys - 1) / span_keys;
            if (it.span >= it.spans) continue;
            it.table = a.page_tables + (long long)seq * a.pages_per_sequence;
            it.begin = first + it.span * span_keys;
            it.end = min(last + 1, it.begin + span_keys);
            it.n_tiles = (it.end - it.begin + kAttnSpanKeys - 1) / kAttnSpanKeys;
            it.owns_self = FUSED && it.span == it.spans - 1;  // this span holds the token's own position
            return true;
        }
        return false;
    };
    // Slice i of this warp: keys [begin + 64 i + 16 warp, + 16).  Lane l looks up the cache row of key l & 15.
    auto slice_rows = [&](const SpanItem& it, int i) -> int {
        const int key = it.begin + i * kAttnSpanKeys + warp * kMmaKeys + (lane & 15);
        if (i >= it.n_tiles || key >= it.end) return 0;
        return it.table[key / kPageTokens] * kPageTokens + key % kPageTokens;
    };
    // Asynchronous 16-byte copies of the slice's K and V rows into slot `slot` (every piece in flight at
    // once): lane l takes piece l % CPR of rows l / CPR, l / CPR + 32 / CPR, ...  Rows past the token's last
    // key are zero, so that a zero probability meets no NaN.  One copy group per call, empty or not.
    const uint32_t ring_at = smem_u32(ring) + ((lane / CPR) * RH + (lane % CPR) * 8) * 2;
    constexpr int kRowsPerPass = 32 / CPR;
    auto issue = [&](const SpanItem& it, int i, int rows, int slot) {
        const __half* k_src = a.cache_k + (long long)it.kvh * HD + (lane % CPR) * 8;
        const __half* v_src = a.cache_v + (long long)it.kvh * HD + (lane % CPR) * 8;
        const int wbegin = it.begin + i * kAttnSpanKeys + warp * kMmaKeys;
        const int wcount = max(0, min(kMmaKeys, it.end - wbegin));
        const uint32_t k_at = ring_at + slot * (L::SLOT * 2);
        const uint32_t v_at = k_at + kMmaKeys * RH * 2;
        if (wcount == kMmaKeys && !(it.owns_self && it.pos < wbegin + kMmaKeys)) {
#pragma unroll
            for (int j = 0; j < kMmaKeys / kRowsPerPass; ++j) {
                const long long at = (long long)__shfl_sync(0xffffffffu, rows, j * kRowsPerPass + lane / CPR) * row_stride;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(k_at + j * (kRowsPerPass * RH * 2)), "l"(k_src + at) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(v_at + j * (kRowsPerPass * RH * 2)), "l"(v_src + at) : "memory");
            }
        } else {
#pragma unroll
            for (int j = 0; j < kMmaKeys / kRowsPerPass; ++j) {
                const int r = j * kRowsPerPass + lane / CPR;
                const long long at = (long long)__shfl_sync(0xffffffffu, rows, r) * row_stride;
                if (it.owns_self && wbegin + r == it.pos) continue;  // the token's own row arrives from k_self / v_self
                if (r < wcount) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(k_at + j * (kRowsPerPass * RH * 2)), "l"(k_src + at) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(v_at + j * (kRowsPerPass * RH * 2)), "l"(v_src + at) : "memory");
                } else {
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(k_at + j * (kRowsPerPass * RH * 2)), "r"(0) : "memory");
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_at + j * (kRowsPerPass * RH * 2)), "r"(0) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    SpanItem cur;
    int id = (int)blockIdx.x - (int)gridDim.x;
    bool valid = next_item(id, cur);
    // This warp's slices form one sequence across the CTA's items: slice c lives in slot c & 1, and while
    // slice c is multiplied slice c + 1 (the item's next, or the first of the next item) is in flight.
    int c = 0;
    int rows0 = 0, rows1 = 0;  // cache rows of the current item's slices 0 and 1
    if (valid) { rows0 = slice_rows(cur, 0); rows1 = slice_rows(cur, 1); }
    // Decode rows: every earlier key was written by an earlier step, so the first copies start while the
    // projection ahead of this kernel drains.  Otherwise the rows may come from the kernel just before.
    if (FUSED && valid) issue(cur, 0, rows0, 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!FUSED && valid) issue(cur, 0, rows0, 0);

    const int g = lane >> 2, t4 = lane & 3;
    const float scale = 1.0f / sqrtf((float)HD);
    // matrix-load offsets inside a slot: K rows as the A operand, V rows transposed as the A operand
    const uint32_t k_off = ((lane & 15) * RH + (lane >> 4) * 8) * 2;
    const uint32_t v_off = (kMmaKeys * RH + ((lane & 7) + (lane >> 4) * 8) * RH + ((lane >> 3) & 1) * 8) * 2;
    // Raw projections of an item, requested one item ahead: this warp's first two query heads, and the
    // token's new K / V row for the warp that produces it.
    constexpr int kAhead = 2;
    const int self_warp = q_per_kv & (kMmaWarps - 1);
    float qx[kAhead][DPL], kx[DPL], vx[DPL];
    auto fetch_raw = [&](const SpanItem& it) {
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int col = warp + u * kMmaWarps;
            if (col < it.len * q_per_kv) {
                const float* qp = a.q + ((long long)(it.t + col / q_per_kv) * a.q_heads + it.kvh * q_per_kv + col % q_per_kv) * HD;
#pragma unroll
                for (int i = 0; i < DPL; ++i) qx[u][i] = qp[lane + 32 * i];
            }
        }
        if (it.owns_self && warp == self_warp) {
            const float* kp = a.k_new + ((long long)it.t * a.kv_heads + it.kvh) * HD;
            const float* vp = a.v_new + ((long long)it.t * a.kv_heads + it.kvh) * HD;
#pragma unroll
            for (int i = 0; i < DPL; ++i) { kx[i] = kp[lane + 32 * i]; vx[i] = vp[lane + 32 * i]; }
        }
    };
    if (valid) fetch_raw(cur);

    while (valid) {
        // The item after this one: its first copies are issued under this item's last slice, so the stream of
        // copies does not pause for this item's fold or the next item's set-up.
        SpanItem nxt;
        int nid = id;
        const bool nvalid = next_item(nid, nxt);
        int nrows0 = 0, nrows1 = 0;
        if (nvalid) { nrows0 = slice_rows(nxt, 0); nrows1 = slice_rows(nxt, 1); }

        // The group's queries (normalised and rotated here for decode rows) as binary16 hi + lo rows.
        {
            int u = 0;
            for (int col = warp; col < cur.len * q_per_kv; col += kMmaWarps, ++u) {
                float x[DPL];
                if (u < kAhead) {
#pragma unroll
                    for (int i = 0; i < DPL; ++i) x[i] = u == 0 ? qx[0][i] : qx[1][i];
                } else {
                    const float* qp = a.q + ((long long)(cur.t + col / q_per_kv) * a.q_heads + cur.kvh * q_per_kv + col % q_per_kv) * HD;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) x[i] = qp[lane + 32 * i];
                }
                if (FUSED) norm_rope<HD>(x, a.q_norm, a.inv_freq, a.eps, (float)cur.pos, lane);
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const __half hi = __float2half_rn(x[i]);
                    q_hi[col * RH + lane + 32 * i] = hi;
                    q_lo[col * RH + lane + 32 * i] = __float2half_rn(x[i] - __half2float(hi));
                }
            }
        }
        if (cur.owns_self && warp == self_warp) {
            // The token's own K (normalised, rotated) and V, rounded to F16 exactly as the cache holds them.
            norm_rope<HD>(kx, a.k_norm, a.inv_freq, a.eps, (float)cur.pos, lane);
            __half* ck = a.cache_k + (long long)a.token_slot[cur.t] * row_stride + (long long)cur.kvh * HD;
            __half* cv = a.cache_v + (long long)a.token_slot[cur.t] * row_stride + (long long)cur.kvh * HD;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                const __half kh = __float2half_rn(kx[i]), vh = __float2half_rn(vx[i]);
                k_self[d] = kh; v_self[d] = vh;
                ck[d] = kh; cv[d] = vh;
            }
        }
        if (nvalid) fetch_raw(nxt);
        __syncthreads();  // queries and own row in place; every warp is done with the previous item's records
        // This lane's B fragments of Q^T: column 8 nt + g, dimensions 16 ks + 2 t4 + {0, 1} and + 8.
        const int cols = cur.len * q_per_kv;
        uint32_t qh[NT][HD / 16][2], ql[NT][HD / 16][2];
        int lim[NT][2];   // last key the tokens of columns 8 nt + 2 t4 and + 1 may see; -1 for a column past the run
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int col = nt * 8 + g;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int at = col * RH + ks * 16 + 2 * t4 + 8 * u;
                    qh[nt][ks][u] = col < cols ? *reinterpret_cast<const uint32_t*>(q_hi + at) : 0u;
                    ql[nt][ks][u] = col < cols ? *reinterpret_cast<const uint32_t*>(q_lo + at) : 0u;
                }
            }
            const int ca = nt * 8 + 2 * t4;
            lim[nt][0] = ca < cols ? cur.pos + ca / q_per_kv : -1;
            lim[nt][1] = ca + 1 < cols ? cur.pos + (ca + 1) / q_per_kv : -1;
        }
        // O^T accumulators: [dims 16 mt + g (values 0, 1) and + 8 (values 2, 3)] x [columns 8 nt + 2 t4 + {0, 1}]
        float o[NT][HD / 16][4];
        float run_m[NT][2], run_l[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int mt = 0; mt < HD / 16; ++mt) { o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.0f; }
            run_m[nt][0] = run_m[nt][1] = -INFINITY;
            run_l[nt][0] = run_l[nt][1] = 0.0f;
        }
        for (int i = 0; i < cur.n_tiles; ++i, ++c) {
            if (i + 1 < cur.n_tiles) {
                issue(cur, i + 1, rows1, (c + 1) & 1);
                rows1 = slice_rows(cur, i + 2);
            } else if (nvalid) {
                issue(nxt, 0, nrows0, (c + 1) & 1);
            } else {
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            asm volatile("cp.async.wait_group 1;" ::: "memory");
            const int wbegin = cur.begin + i * kAttnSpanKeys + warp * kMmaKeys;
            if (wbegin >= cur.end) continue;  // a short last tile: nothing for this warp
            __half* k_w = ring + (c & 1) * L::SLOT;
            if (cur.owns_self && cur.pos >= wbegin && cur.pos < wbegin + kMmaKeys) {
                // the token's own row takes its place in the slice (8 bytes per lane and row)
                for (int q4 = lane; q4 < HD / 4; q4 += 32) {
                    *reinterpret_cast<uint2*>(k_w + (cur.pos - wbegin) * RH + q4 * 4) = *reinterpret_cast<const uint2*>(k_self + q4 * 4);
                    *reinterpret_cast<uint2*>(k_w + (kMmaKeys + cur.pos - wbegin) * RH + q4 * 4) = *reinterpret_cast<const uint2*>(v_self + q4 * 4);
                }
            }
            __syncwarp();
            slice_step<HD, NT>(k_w, wbegin, lim, qh, ql, o, run_m, run_l, i == 0, scale, k_off, v_off, g);
            __syncwarp();  // every lane has read the slot before the next copies land in it
        }
        // This warp's result goes where its last slice was: that slot receives no copy before the next
        // item's first barrier, which every warp passes only after the fold below.
        const int rec_slot = (c - 1) & 1;
        float* rec = reinterpret_cast<float*>(ring + rec_slot * L::SLOT);
        if (cur.begin + warp * kMmaKeys < cur.end) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int h = nt * 8 + 2 * t4;   // this lane's first column
#pragma unroll
                for (int mt = 0; mt < HD / 16; ++mt) {
                    const int d = mt * 16 + g;
                    if (h < cols) { rec[h * REC + d] = o[nt][mt][0]; rec[h * REC + d + 8] = o[nt][mt][2]; }
                    if (h + 1 < cols) { rec[(h + 1) * REC + d] = o[nt][mt][1]; rec[(h + 1) * REC + d + 8] = o[nt][mt][3]; }
                }
                if (g == 0) {
                    if (h < cols) { rec[h * REC + HD] = run_m[nt][0]; rec[h * REC + HD + 1] = run_l[nt][0]; }
                    if (h + 1 < cols) { rec[(h + 1) * REC + HD] = run_m[nt][1]; rec[(h + 1) * REC + HD + 1] = run_l[nt][1]; }
                }
            }
        }
        __syncthreads();

        // Fold the warps' results in warp order: a warp per column, lane = dimension lane + 32 i.
        const int live_warps = min(kMmaWarps, (cur.end - cur.begin + kMmaKeys - 1) / kMmaKeys);
        const float* recs = reinterpret_cast<const float*>(v_self + RH + rec_slot * L::SLOT);
        constexpr int kWarpFloats = STAGES * L::SLOT / 2;  // floats between two warps' records
        for (int h = warp; h < cols; h += kMmaWarps) {
            const int token = cur.t + h / q_per_kv, qh_index = cur.kvh * q_per_kv + h % q_per_kv;
            // the column's own span count; a token of the run whose keys end before this span has nothing here
            const int col_spans = cur.len == 1 ? cur.spans : (cur.pos + h / q_per_kv + span_keys) / span_keys;
            if (cur.span >= col_spans) continue;
            float top = -INFINITY;
            for (int w = 0; w < live_warps; ++w) top = fmaxf(top, recs[w * kWarpFloats + h * REC + HD]);
            float acc[DPL], total = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
            for (int w = 0; w < live_warps; ++w) {
                const float fw = __expf(recs[w * kWarpFloats + h * REC + HD] - top);
                total = fmaf(recs[w * kWarpFloats + h * REC + HD + 1], fw, total);
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[i] = fmaf(recs[w * kWarpFloats + h * REC + lane + 32 * i], fw, acc[i]);
            }
            if (col_spans == 1) {
                ActOperand op = a.operand;
                op.ss32 = nullptr;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const float value = acc[i] / total;
                    a.out[((long long)token * a.q_heads + qh_index) * HD + lane + 32 * i] = value;
                    if (op.dig != nullptr) operand_store_span(op, token - a.token_base, a.q_heads * HD, (qh_index * HD) / 32 + i, lane, value, 0.0f);
                }
            } else {
                float* pp = a.partial + (((long long)(token - a.token_base) * a.q_heads + qh_index) * a.max_spans + cur.span) * REC;
#pragma unroll
                for (int i = 0; i < DPL; ++i) pp[lane + 32 * i] = acc[i];
                if (lane == 0) { pp[HD] = top; pp[HD + 1] = total; }
            }
        }
        cur = nxt; id = nid; valid = nvalid;
        rows0 = nrows0; rows1 = nrows1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- prefill kernel: a run of consecutive tokens of one sequence ---------------------------------------
//
// A CTA serves (4 x warp_tokens consecutive tokens, kv head); warp w owns warp_tokens of them (their query heads
// are its MMA columns) and walks ALL their keys, so there are no spans to merge and the result is final.  The
// four warps see the same keys up to their diagonals: a 64-key tile is staged in shared memory once per CTA
// (asynchronous copies, two buffers) and every warp multiplies its own columns against the tile's four
// 16-key slices with the slice arithmetic of the span kernel.  A token's bits depend only on its own keys.
template <int HD, int NT>
__global__ void __launch_bounds__(kMmaWarps * 32) attention_prefill_mma_kernel(const AttnArgs a, const int n_tokens, const int warp_tokens) {
    using L = MmaLayout<HD>;
    constexpr int DPL = HD / 32;
    constexpr int RH = L::RH;
    constexpr int CPR = HD / 8;
    extern __shared__ __align__(16) unsigned char attn_smem[];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t4 = lane & 3;
    const int q_per_kv = a.q_heads / a.kv_heads;
    const int cta_tokens = kMmaWarps * warp_tokens, cols = warp_tokens * q_per_kv;
    const int groups = n_tokens / cta_tokens;
    // the groups with the most keys first
    const int group = groups - 1 - (int)blockIdx.x / a.kv_heads, kvh = (int)blockIdx.x % a.kv_heads;
    const int t0 = a.token_base + group * cta_tokens;
    const int pos0 = a.token_pos[t0];
    const int32_t* table = a.page_tables + (long long)(a.token_seq != nullptr ? a.token_seq[t0] : 0) * a.pages_per_sequence;
    const int last = pos0 + cta_tokens - 1;                       // the CTA's last key
    const int warp_first = pos0 + warp * warp_tokens, warp_last = warp_first + warp_tokens - 1;
    const int n_tiles = last / kAttnSpanKeys + 1;
    const long long row_stride = (long long)a.kv_heads * HD;
    __half* q_hi = reinterpret_cast<__half*>(attn_smem) + (size_t)warp * 2 * 8 * NT * RH;   // this warp's [8 NT][RH]
    __half* q_lo = q_hi + 8 * NT * RH;
    __half* tiles = reinterpret_cast<__half*>(attn_smem) + (size_t)kMmaWarps * 2 * 8 * NT * RH;   // [2][4 slices][K 16 | V 16][RH]
    constexpr int kTileHalfs = kMmaWarps * L::SLOT;

    // thread -> (key row of the tile, half of the row's pieces): one page lookup per thread and tile
    const int srow = threadIdx.x >> 1, shalf = threadIdx.x & 1;
    auto stage = [&](int tile) {
        if (tile < n_tiles) {
            const int key = tile * kAttnSpanKeys + srow;
            __half* dk = tiles + (tile & 1) * kTileHalfs + (srow >> 4) * L::SLOT + (srow & 15) * RH + shalf * (HD / 2);
            __half* dv = dk + kMmaKeys * RH;
            if (key <= last) {
                const long long phys = (long long)table[key / kPageTokens] * kPageTokens + key % kPageTokens;
                const __half* sk = a.cache_k + phys * row_stride + (long long)kvh * HD + shalf * (HD / 2);
                const __half* sv = a.cache_v + phys * row_stride + (long long)kvh * HD + shalf * (HD / 2);
#pragma unroll
                for (int j = 0; j < CPR / 2; ++j) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dk + j * 8)), "l"(sk + j * 8) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dv + j * 8)), "l"(sv + j * 8) : "memory");
                }
            } else {
#pragma unroll
                for (int j = 0; j < CPR / 2; ++j) {
                    *reinterpret_cast<uint4*>(dk + j * 8) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(dv + j * 8) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0);

    // this warp's queries as binary16 hi + lo rows, then its B fragments
    for (int col = 0; col < cols; ++col) {
        const float* qp = a.q + ((long long)(t0 + warp * warp_tokens + col / q_per_kv) * a.q_heads + kvh * q_per_kv + col % q_per_kv) * HD;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const float x = qp[lane + 32 * i];
            const __half hi = __float2half_rn(x);
            q_hi[col * RH + lane + 32 * i] = hi;
            q_lo[col * RH + lane + 32 * i] = __float2half_rn(x - __half2float(hi));
        }
    }
    __syncwarp();
    uint32_t qh[NT][HD / 16][2], ql[NT][HD / 16][2];
    int lim[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int col = nt * 8 + g;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int at = col * RH + ks * 16 + 2 * t4 + 8 * u;
                qh[nt][ks][u] = col < cols ? *reinterpret_cast<const uint32_t*>(q_hi + at) : 0u;
                ql[nt][ks][u] = col < cols ? *reinterpret_cast<const uint32_t*>(q_lo + at) : 0u;
            }
        }
        const int ca = nt * 8 + 2 * t4;
        lim[nt][0] = ca < cols ? warp_first + ca / q_per_kv : -1;
        lim[nt][1] = ca + 1 < cols ? warp_first + (ca + 1) / q_per_kv : -1;
    }
    float o[NT][HD / 16][4], run_m[NT][2], run_l[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int mt = 0; mt < HD / 16; ++mt) { o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.0f; }
        run_m[nt][0] = run_m[nt][1] = -INFINITY;
        run_l[nt][0] = run_l[nt][1] = 0.0f;
    }
    const float scale = 1.0f / sqrtf((float)HD);
    const uint32_t k_off = ((lane & 15) * RH + (lane >> 4) * 8) * 2;
    const uint32_t v_off = (kMmaKeys * RH + ((lane & 7) + (lane >> 4) * 8) * RH + ((lane >> 3) & 1) * 8) * 2;
    bool first = true;
    for (int tile = 0; tile < n_tiles; ++tile) {
        stage(tile + 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();   // the tile is in place for every warp
        const __half* buf = tiles + (tile & 1) * kTileHalfs;
#pragma unroll 1
        for (int sl = 0; sl < kMmaWarps; ++sl) {
            const int wbegin = tile * kAttnSpanKeys + sl * kMmaKeys;
            if (wbegin > warp_last) break;   // past this warp's diagonal
            slice_step<HD, NT>(buf + sl * L::SLOT, wbegin, lim, qh, ql, o, run_m, run_l, first, scale, k_off, v_off, g);
            first = false;
        }
        __syncthreads();   // every warp has read the buffer before the copies of tile + 2 land in it
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // out[token][head][d] = o / l: dims 16 mt + g (values 0, 1) and + 8 (values 2, 3) of columns 8 nt + 2 t4 + {0, 1}
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int col = nt * 8 + 2 * t4 + j;
            if (col < cols) {
                const int token = t0 + warp * warp_tokens + col / q_per_kv, head = kvh * q_per_kv + col % q_per_kv;
                float* dst = a.out + ((long long)token * a.q_heads + head) * HD;
                const float total = run_l[nt][j];
#pragma unroll
                for (int mt = 0; mt < HD / 16; ++mt) {
                    dst[mt * 16 + g] = o[nt][mt][j] / total;
                    dst[mt * 16 + g + 8] = o[nt][mt][2 + j] / total;
                }
            }
        }
    }
}

// The merge: one warp per (token, q head).  A launch of its own, so that the span CTAs retire as soon as their
// sums are stored and the next projection's weight stream can start under the merge.
template <int HD>
__global__ void __launch_bounds__(kMmaWarps * 32) attention_merge_kernel(const AttnArgs a, const int n_tokens) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int pair = blockIdx.x * kMmaWarps + (threadIdx.x >> 5);
    if (pair >= n_tokens * a.q_heads) return;
    const int t = a.token_base + pair / a.q_heads, qh = pair % a.q_heads;
    const int spans = token_spans(a, a.token_pos[t]);
    if (spans <= 1) return;  // written directly by the span kernel
    merge_head<HD>(a, t, qh, spans, threadIdx.x & 31);
}

int attn_sm_count() {
    static int counts[kMaxDevices] = {0};  // per device ordinal
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (counts[dev] == 0) {
        if (cudaDeviceGetAttribute(&counts[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || counts[dev] <= 0) counts[dev] = 148;
    }
    return counts[dev];
}

template <typename Kernel>
cudaError_t launch_pdl(cudaStream_t stream, Kernel kernel, dim3 grid, int threads, size_t smem, const AttnArgs& a,
                       bool programmatic) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned int)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <typename Kernel>
cudaError_t launch_pdl(cudaStream_t stream, Kernel kernel, dim3 grid, int threads, size_t smem, const AttnArgs& a,
                       bool programmatic, int extra, int extra2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned int)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a, extra, extra2);
}

template <typename Kernel>
cudaError_t launch_pdl(cudaStream_t stream, Kernel kernel, dim3 grid, int threads, size_t smem, const AttnArgs& a,
                       bool programmatic, int extra) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned int)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a, extra);
}

// The span kernel and its merge over tokens [first_token, first_token + n_tokens) of the launch.
template <int HD>
cudaError_t launch_spans_hd(cudaStream_t stream, AttnArgs a, bool fused, int first_token, int n_tokens, int max_keys,
                            size_t partial_bytes, int* launches, bool programmatic) {
    const int q_per_kv = a.q_heads / a.kv_heads;
    const int max_tiles = (max_keys + kAttnSpanKeys - 1) / kAttnSpanKeys;
    if (max_tiles > kAttnMaxSpans) return cudaErrorInvalidValue;
    // Tiles per span: as many as leave sixteen CTAs per SM's worth of spans (the per-item set-up and the
    // merge are paid once per span); a launch that cannot fill the GPU keeps one tile per span.
    // Prefill-sized launches: up to 16 / group-size consecutive tokens of a sequence are the columns of one item
    // and share its staged K / V rows (a token's bits do not depend on the grouping).
    a.run_tokens = (!fused && a.window <= 0 && a.operand.dig == nullptr && n_tokens >= 16) ? std::max(1, 16 / q_per_kv) : 1;
    const long long item_tokens = (n_tokens + a.run_tokens - 1) / a.run_tokens;
    a.tiles = 1;
    while (a.tiles < 8 && item_tokens * a.kv_heads * ((max_tiles + 2 * a.tiles - 1) / (2 * a.tiles)) >= 16 * 148) a.tiles *= 2;
    a.max_spans = (max_tiles + a.tiles - 1) / a.tiles;
    const size_t per_token = (size_t)a.q_heads * a.max_spans * (HD + 2) * sizeof(float);
    int chunk = n_tokens;
    if (a.max_spans > 1) {
        if (a.partial == nullptr || partial_bytes < per_token) return cudaErrorInvalidValue;
        chunk = (int)std::min<size_t>((size_t)n_tokens, partial_bytes / per_token);
    }
    if (a.operand.dig != nullptr && chunk < n_tokens) return cudaErrorInvalidValue;  // operand rows are launch-relative
    const size_t mma_smem = MmaLayout<HD>::bytes(q_per_kv * a.run_tokens);
    {
        // above the default shared-memory limit: opt in once per instantiation and device
        static bool configured_on[kMaxDevices] = {false};  // function attributes are per device
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
        bool& configured = configured_on[dev];
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(attention_span_mma_kernel<HD, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_span_mma_kernel<HD, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_span_mma_kernel<HD, true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_span_mma_kernel<HD, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            configured = true;
        }
    }
    for (int base = 0; base < n_tokens; base += chunk) {
        const int n = std::min(chunk, n_tokens - base);
        a.token_base = first_token + base;
        cudaError_t e;
        {
            // persistent CTAs, as many as can be resident, walk the launch's (token, kv head, span) items
            const bool wide = q_per_kv * a.run_tokens > 8;
            int resident = 0;
            cudaError_t q = wide ? (fused ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, attention_span_mma_kernel<HD, true, 2>, kMmaWarps * 32, mma_smem)
                                          : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, attention_span_mma_kernel<HD, false, 2>, kMmaWarps * 32, mma_smem))
                                 : (fused ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, attention_span_mma_kernel<HD, true, 1>, kMmaWarps * 32, mma_smem)
                                          : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, attention_span_mma_kernel<HD, false, 1>, kMmaWarps * 32, mma_smem));
            if (q != cudaSuccess) return q;
            resident = std::max(1, resident);
            const dim3 grid((unsigned)std::min<long long>((long long)n * a.kv_heads * a.max_spans, (long long)attn_sm_count() * resident));
            if (!wide) {
                e = fused ? launch_pdl(stream, attention_span_mma_kernel<HD, true, 1>, grid, kMmaWarps * 32, mma_smem, a, programmatic, n)
                          : launch_pdl(stream, attention_span_mma_kernel<HD, false, 1>, grid, kMmaWarps * 32, mma_smem, a, programmatic, n);
            } else {
                e = fused ? launch_pdl(stream, attention_span_mma_kernel<HD, true, 2>, grid, kMmaWarps * 32, mma_smem, a, programmatic, n)
                          : launch_pdl(stream, attention_span_mma_kernel<HD, false, 2>, grid, kMmaWarps * 32, mma_smem, a, programmatic, n);
            }
        }
        if (e != cudaSuccess) return e;
        if (launches) ++*launches;
        if (a.max_spans > 1) {
            e = launch_pdl(stream, attention_merge_kernel<HD>, dim3((n * a.q_heads + kMmaWarps - 1) / kMmaWarps), kMmaWarps * 32, 0, a,
                           programmatic, n);
            if (e != cudaSuccess) return e;
            if (launches) ++*launches;
        }
    }
    return cudaSuccess;
}

template <int HD>
cudaError_t launch_hd(cudaStream_t stream, AttnArgs a, bool fused, int n_tokens, int max_keys, size_t partial_bytes,
                      int* launches, bool programmatic = false) {
    const int q_per_kv = a.q_heads / a.kv_heads;
    if (q_per_kv > 16) return cudaErrorInvalidValue;  // the group is the 16 columns of two MMA tiles
    // A long run of consecutive tokens of one sequence (a prefill chunk; the caller says where it lies) takes the
    // prefill kernel for as many whole CTA groups as it holds; what lies before, behind and beyond takes the spans.
    const int warp_tokens = std::max(1, 16 / q_per_kv), cta_tokens = kMmaWarps * warp_tokens;
    if (!fused && a.window <= 0 && a.operand.dig == nullptr && a.run_first >= 0 && a.run_count >= 64 &&
        a.run_first + a.run_count <= n_tokens) {
        const int aligned = a.run_count / cta_tokens * cta_tokens;
        const bool wide = warp_tokens * q_per_kv > 8;
        const size_t smem = (size_t)(kMmaWarps * 2 * 8 * (wide ? 2 : 1) + 2 * kMmaWarps * 2 * kMmaKeys) * (HD + 8) * sizeof(__half);
        static bool configured_on[kMaxDevices] = {false};  // function attributes are per device
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
        if (!configured_on[dev]) {
            cudaError_t e = cudaFuncSetAttribute(attention_prefill_mma_kernel<HD, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_prefill_mma_kernel<HD, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            configured_on[dev] = true;
        }
        AttnArgs p = a;
        p.token_base = a.run_first;
        const dim3 grid((unsigned)(aligned / cta_tokens * a.kv_heads));
        cudaError_t e = wide ? launch_pdl(stream, attention_prefill_mma_kernel<HD, 2>, grid, kMmaWarps * 32, smem, p, programmatic, aligned, warp_tokens)
                             : launch_pdl(stream, attention_prefill_mma_kernel<HD, 1>, grid, kMmaWarps * 32, smem, p, programmatic, aligned, warp_tokens);
        if (e != cudaSuccess) return e;
        if (launches) ++*launches;
        if (a.run_first > 0) {
            e = launch_spans_hd<HD>(stream, a, fused, 0, a.run_first, max_keys, partial_bytes, launches, programmatic);
            if (e != cudaSuccess) return e;
        }
        const int behind = a.run_first + aligned;
        if (behind < n_tokens) e = launch_spans_hd<HD>(stream, a, fused, behind, n_tokens - behind, max_keys, partial_bytes, launches, programmatic);
        return e;
    }
    return launch_spans_hd<HD>(stream, a, fused, 0, n_tokens, max_keys, partial_bytes, launches, programmatic);
}

cudaError_t dispatch(cudaStream_t stream, const AttnArgs& a, bool fused, int head_dim, int n_tokens, int max_keys,
                     size_t partial_bytes, int* launches, bool programmatic = false) {
    switch (head_dim) {
        case 64: return launch_hd<64>(stream, a, fused, n_tokens, max_keys, partial_bytes, launches, programmatic);
        case 128: return launch_hd<128>(stream, a, fused, n_tokens, max_keys, partial_bytes, launches, programmatic);
        case 256: return launch_hd<256>(stream, a, fused, n_tokens, max_keys, partial_bytes, launches, programmatic);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_attention(cudaStream_t stream, const float* q, const __half* cache_k, const __half* cache_v,
                             const int32_t* page_tables, int pages_per_sequence, const int32_t* token_seq,
                             const int32_t* token_pos, int n_tokens, int q_heads, int kv_heads, int head_dim,
                             int window, int max_keys, float* partial, size_t partial_bytes, float* out,
                             int* launches, int run_first, int run_count) {
    if (n_tokens <= 0) return cudaSuccess;
    if (q_heads % kv_heads != 0 || q_heads / kv_heads > 16 || max_keys <= 0) return cudaErrorInvalidValue;
    if (head_dim == 32) {
        // Below 64 dims the span kernel's lane layout does not apply: the plain kernel serves.
        cudaError_t e = launch_attention_ref(stream, q, cache_k, cache_v, page_tables, pages_per_sequence, token_seq,
                                             token_pos, n_tokens, q_heads, kv_heads, head_dim, window, out);
        if (e == cudaSuccess && launches) ++*launches;
        return e;
    }
    if (window > 0) max_keys = std::min(max_keys, window);
    AttnArgs a{};
    a.q = q;
    a.cache_k = const_cast<__half*>(cache_k);
    a.cache_v = const_cast<__half*>(cache_v);
    a.page_tables = page_tables;
    a.pages_per_sequence = pages_per_sequence;
    a.token_seq = token_seq;
    a.token_pos = token_pos;
    a.q_heads = q_heads;
    a.kv_heads = kv_heads;
    a.window = window;
    a.partial = partial;
    a.out = out;
    a.run_first = run_first; a.run_count = run_count;
    return dispatch(stream, a, false, head_dim, n_tokens, max_keys, partial_bytes, launches);
}

cudaError_t launch_attention_decode(cudaStream_t stream, const DecodeAttention& d, int* launches) {
    if (d.n_tokens <= 0) return cudaSuccess;
    if (d.q_heads % d.kv_heads != 0 || d.q_heads / d.kv_heads > 16 || d.max_keys <= 0) return cudaErrorInvalidValue;
    AttnArgs a{};
    a.q = d.q; a.k_new = d.k; a.v_new = d.v;
    a.q_norm = d.q_norm; a.k_norm = d.k_norm; a.inv_freq = d.inv_freq; a.eps = d.eps;
    a.cache_k = d.cache_k; a.cache_v = d.cache_v;
    a.page_tables = d.page_tables; a.pages_per_sequence = d.pages_per_sequence;
    a.token_seq = d.token_seq; a.token_pos = d.token_pos; a.token_slot = d.token_slot;
    a.q_heads = d.q_heads; a.kv_heads = d.kv_heads; a.window = d.window;
    a.partial = d.partial; a.out = d.out; a.operand = d.operand;
    a.run_first = -1; a.run_count = 0;
    const int max_keys = d.window > 0 ? std::min(d.max_keys, d.window) : d.max_keys;
    return dispatch(stream, a, true, d.head_dim, d.n_tokens, max_keys, d.partial_bytes, launches, d.programmatic);
}

}  // namespace ribn
