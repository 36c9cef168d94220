"""GPU parity of the single operators, called through the C ABI, against the
CPU oracle on the reference's own fixtures and on seeded random inputs.
Bit-exact for decode, F16 rounding, metadata and token selection; the
reference's own tolerances elsewhere (crates/nvidia/tests/cuda_reference.rs)."""
import struct

import numpy as np
import pytest

from oracle import binding as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_library):
    from ribn_b200 import ops as o
    return o


# ---- dequant: bit-exact (crates/gguf/src/lib.rs:1479-1565 and random blocks) ---------------
def test_known_answer_blocks(ops):
    q8 = bytearray(34); q8[0:2] = struct.pack("<H", 0x3C00); q8[2], q8[3] = 0x80, 0x7F
    out = ops.dequantize(H.Q8_0, bytes(q8), 1, 32)[0]
    assert out[0] == -128.0 and out[1] == 127.0
    q4 = bytearray(144); q4[0:2] = struct.pack("<H", 0x3C00); q4[4:8] = b"\x01" * 4; q4[16] = 0x10
    out = ops.dequantize(H.Q4_K, bytes(q4), 1, 256)[0]
    assert out[0] == 0.0 and out[32] == 1.0
    q6 = bytearray(210); q6[192:208] = b"\x01" * 16; q6[208:210] = struct.pack("<H", 0x3C00)
    assert np.all(ops.dequantize(H.Q6_K, bytes(q6), 1, 256) == -32.0)


@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
def test_dequant_bit_exact_on_fixtures_and_random_blocks(ops, kind):
    elems, size = H.BLOCK[kind]
    fx = H.fixture(kind)
    n = fx.size // size
    assert np.array_equal(ops.dequantize(kind, fx, 1, n * elems).view(np.uint32),
                          orc.dequantize_rows(kind, fx, 1, n * elems).view(np.uint32))
    rng = np.random.default_rng(100 + kind)
    blocks = rng.integers(0, 256, size=(512, size), dtype=np.uint8)
    for off in ([0] if kind == H.Q8_0 else [0, 2] if kind == H.Q4_K else [208]):
        blocks[:, off + 1] &= 0x7B  # finite f16 scales, both signs
    rows, cols = 64, 8 * elems
    got = ops.dequantize(kind, blocks, rows, cols)
    want = orc.dequantize_rows(kind, blocks, rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_of_quantised_normal_weights_is_bit_exact(ops):
    rng = np.random.default_rng(5)
    for kind in (H.Q8_0, H.Q4_K, H.Q6_K):
        enc = H.quantize(kind, rng.normal(0, 0.02, size=(33, 768)).astype(np.float32))
        assert np.array_equal(ops.dequantize(kind, enc, 33, 768).view(np.uint32),
                              orc.dequantize_rows(kind, enc, 33, 768).view(np.uint32))


# ---- elementwise (cuda_reference.rs:902-963) ---------------------------------------------------
def test_rms_norm(ops):
    x = np.array([1.0, -2.0, 3.0, -4.0], dtype=np.float32)
    w = np.array([1.0, 0.5, 2.0, -1.0], dtype=np.float32)
    assert np.max(np.abs(ops.rms_norm(x, w, 1e-5) - orc.rms_norm(x, w, 1e-5))) < 1e-5
    rng = np.random.default_rng(0)
    xs = rng.normal(0, 3, size=(5, 4096)).astype(np.float32)
    ws = rng.normal(1, 0.2, size=4096).astype(np.float32)
    got = ops.rms_norm(xs, ws, 1e-6)
    for m in range(5):
        assert np.max(np.abs(got[m] - orc.rms_norm(xs[m], ws, 1e-6))) < 1e-5


def test_silu_mul(ops):
    i = np.arange(513, dtype=np.float32)
    gate, up = i * np.float32(0.01) - np.float32(2.5), np.float32(1.0) - i * np.float32(0.002)
    assert np.max(np.abs(ops.silu_mul(gate, up) - orc.silu_mul(gate, up))) < 1e-5


def test_argmax_matches_first_max_rule(ops):
    logits = np.full(513, -10.0, dtype=np.float32)
    logits[401] = logits[402] = 7.0
    assert ops.argmax(logits) == 401
    logits[3] = np.nan
    assert ops.argmax(logits) == 401
    assert ops.argmax(np.full(9, np.nan, dtype=np.float32)) == 0
    rng = np.random.default_rng(1)
    big = rng.normal(0, 1, size=(7, 151936)).astype(np.float32)
    big[2, 77] = big[2, 150000] = 9.0       # tie across distant positions
    big[4, :] = -np.inf
    big[5, 1000:] = np.nan
    got = ops.argmax(big)
    want = [orc.argmax(big[m]) for m in range(7)]
    assert list(got) == want and got[2] == 77


def test_f32_to_f16_bit_exact(ops):
    rng = np.random.default_rng(2)
    vals = np.concatenate([rng.normal(0, 1, 5000), rng.normal(0, 1e-6, 2000), rng.normal(0, 4e4, 1000),
                           np.array([0.0, -0.0, 65504.0, 65520.0, 1e9, -1e9, 5.9e-8, 2.98e-8, np.inf])]).astype(np.float32)
    assert np.array_equal(ops.f32_to_f16_bits(vals), orc.f32_to_f16_bits(vals))


def test_rope_neox(ops):
    # cuda_reference.rs:1929-1972 geometry, then dense-Qwen3 geometry with far positions
    heads, hd, rot, base = 4, 256, 64, 1.0e7
    host = ((np.arange(heads * hd) % 97).astype(np.float32) * np.float32(0.03) - np.float32(1.4)).astype(np.float32)
    got = ops.rope_neox(host.reshape(1, -1), [3], heads, hd, rot, base)[0]
    assert np.max(np.abs(got - orc.rope_neox(host, heads, hd, rot, base, 3))) < 1e-5
    rng = np.random.default_rng(3)
    vals = rng.normal(0, 1, size=(3, 8 * 128)).astype(np.float32)
    positions = [0, 4097, 16383]
    got = ops.rope_neox(vals, positions, 8, 128, 128, 1.0e6)
    for m, p in enumerate(positions):
        assert np.max(np.abs(got[m] - orc.rope_neox(vals[m], 8, 128, 128, 1.0e6, p))) < 1e-5


# ---- attention (cuda_reference.rs:1995-2093, paged_attention.rs:57-152) ---------------------------
def _attention_case(tokens, rows, table, seed, QH=6, KVH=2, HD=32):
    q, state = H.lcg_f16_values(seed, rows * QH * HD)
    k, state = H.lcg_f16_values(state, tokens * KVH * HD)
    v, state = H.lcg_f16_values(state, tokens * KVH * HD)
    kb, vb = k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16)
    pages = len(table)
    phys_k = np.zeros((pages * 16, KVH * HD), dtype=np.uint16)
    phys_v = np.zeros_like(phys_k)
    for t in range(tokens):
        phys = table[t // 16] * 16 + t % 16
        phys_k[phys] = kb.reshape(tokens, -1)[t]
        phys_v[phys] = vb.reshape(tokens, -1)[t]
    return q, kb, vb, phys_k, phys_v


@pytest.mark.parametrize("variant", [0, 1], ids=["split-kv", "reference-kernel"])
@pytest.mark.parametrize("tokens,rows", [(1, 1), (4, 1), (5, 1), (8, 1), (7, 3), (10, 10), (40, 1), (37, 9),
                                         (200, 1), (150, 70)])
def test_attention_against_oracle_and_paged_equals_contiguous(ops, tokens, rows, variant):
    QH, KVH, HD = 6, 2, 32
    pages = (tokens + 15) // 16
    identity = list(range(pages))
    shuffled = list(reversed(range(pages))) if pages > 1 else [0]
    q, kb, vb, pk, pv = _attention_case(tokens, rows, identity, 12345 + tokens)
    got = ops.attention(q, pk, pv, identity, tokens, rows, QH, KVH, HD, variant=variant)
    for r in range(rows):
        seen = tokens - rows + 1 + r
        want = orc.attention(q.reshape(rows, -1)[r], kb[: seen * KVH * HD], vb[: seen * KVH * HD], seen, QH, KVH, HD)
        assert np.max(np.abs(got[r] - want)) < 1e-3
    _, _, _, pk2, pv2 = _attention_case(tokens, rows, shuffled, 12345 + tokens)
    again = ops.attention(q, pk2, pv2, shuffled, tokens, rows, QH, KVH, HD, variant=variant)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))  # paged == contiguous, bit for bit


def test_attention_dense_qwen3_geometry_long_context(ops):
    QH, KVH, HD, tokens = 32, 8, 128, 1000
    rng = np.random.default_rng(9)
    q = rng.normal(0, 1, QH * HD).astype(np.float32)
    k = rng.normal(0, 1, tokens * KVH * HD).astype(np.float16).view(np.uint16)
    v = rng.normal(0, 1, tokens * KVH * HD).astype(np.float16).view(np.uint16)
    pages = (tokens + 15) // 16
    table = list(rng.permutation(pages))
    pk = np.zeros((pages * 16, KVH * HD), dtype=np.uint16); pv = np.zeros_like(pk)
    for t in range(tokens):
        pk[table[t // 16] * 16 + t % 16] = k.reshape(tokens, -1)[t]
        pv[table[t // 16] * 16 + t % 16] = v.reshape(tokens, -1)[t]
    want = orc.attention(q, k, v, tokens, QH, KVH, HD)
    tail = orc.attention(q, k[(tokens - 128) * KVH * HD:], v[(tokens - 128) * KVH * HD:], 128, QH, KVH, HD)
    for variant in (0, 1):
        got = ops.attention(q, pk, pv, table, tokens, 1, QH, KVH, HD, variant=variant)[0]
        assert np.max(np.abs(got - want)) < 1e-3
        # sliding window: the last 128 keys only
        win = ops.attention(q, pk, pv, table, tokens, 1, QH, KVH, HD, window=128, variant=variant)[0]
        assert np.max(np.abs(win - tail)) < 1e-3


# ---- ragged batch metadata: exact -------------------------------------------------------------------
def test_batch_metadata_exact(ops):
    rng = np.random.default_rng(4)
    rows, pps = 37, 40
    slot = rng.permutation(64)[:rows].astype(np.int32)
    tokens = rng.integers(1, 30, size=rows).astype(np.int32)
    tokens[::3] = 1
    prefix = rng.integers(0, pps * 16 - 30, size=rows).astype(np.int32)
    tables = rng.permutation(64 * pps).astype(np.int32).reshape(64, pps)
    cu, row, pos, kv = ops.batch_metadata(slot, prefix, tokens, tables)
    want_cu = np.concatenate([[0], np.cumsum(tokens)]).astype(np.int32)
    assert np.array_equal(cu, want_cu)
    want_row = np.repeat(np.arange(rows), tokens)
    want_pos = np.concatenate([prefix[r] + np.arange(tokens[r]) for r in range(rows)])
    want_kv = tables[slot[want_row], want_pos // 16] * 16 + want_pos % 16
    assert np.array_equal(row, want_row) and np.array_equal(pos, want_pos) and np.array_equal(kv, want_kv)
    # empty-ish and maximum cases
    cu, row, pos, kv = ops.batch_metadata([0], [0], [1], tables)
    assert list(cu) == [0, 1] and list(pos) == [0] and kv[0] == tables[0, 0] * 16
    big = np.ones(1000, dtype=np.int32)
    cu, row, pos, kv = ops.batch_metadata(np.arange(1000) % 64, np.zeros(1000), big, tables)
    assert cu[-1] == 1000 and np.array_equal(row, np.arange(1000))


@pytest.mark.parametrize("QH,KVH,HD,tokens,rows", [(32, 8, 128, 300, 64), (16, 8, 128, 200, 96), (8, 2, 64, 777, 150),
                                                   (16, 1, 128, 64, 64)])
def test_attention_large_launches_take_the_staged_span_kernel(ops, QH, KVH, HD, tokens, rows):
    # rows x kv heads x spans >= 1024: K / V rows staged in shared memory once per query-head group;
    # compared with the oracle per row, and paged == contiguous bit for bit.
    rng = np.random.default_rng(QH + tokens)
    q = rng.normal(0, 1, size=(rows, QH * HD)).astype(np.float32)
    k = rng.normal(0, 1, tokens * KVH * HD).astype(np.float16).view(np.uint16)
    v = rng.normal(0, 1, tokens * KVH * HD).astype(np.float16).view(np.uint16)
    pages = (tokens + 15) // 16
    results = []
    for table in (list(range(pages)), list(rng.permutation(pages))):
        pk = np.zeros((pages * 16, KVH * HD), dtype=np.uint16); pv = np.zeros_like(pk)
        for t in range(tokens):
            pk[table[t // 16] * 16 + t % 16] = k.reshape(tokens, -1)[t]
            pv[table[t // 16] * 16 + t % 16] = v.reshape(tokens, -1)[t]
        results.append(ops.attention(q, pk, pv, table, tokens, rows, QH, KVH, HD, variant=0))
    assert np.array_equal(results[0].view(np.uint32), results[1].view(np.uint32))
    for r in range(0, rows, 7):
        seen = tokens - rows + 1 + r
        want = orc.attention(q[r], k[: seen * KVH * HD], v[: seen * KVH * HD], seen, QH, KVH, HD)
        assert np.max(np.abs(results[0][r] - want)) < 1e-4, r


# ---- the packed layout decodes to the reference's values, bit for bit ------------------------------
@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
@pytest.mark.parametrize("rows,cols", [(16, 256), (37, 768), (1, 512), (130, 1024)])
def test_decode_from_packed_tiles_is_bit_exact(ops, kind, rows, cols):
    """The tile-major repack keeps every bit: decoding FROM the packed tiles on the device (the weight
    decoder of the decode-and-split tensor-memory kernel) equals dequantize_block on the raw blocks,
    ragged row counts (padding rows of the last tile) included."""
    elems, size = H.BLOCK[kind]
    rng = np.random.default_rng(31 * kind + rows)
    raw = rng.integers(0, 256, size=(rows * (cols // elems), size), dtype=np.uint8)
    for off in ([0] if kind == H.Q8_0 else [0, 2] if kind == H.Q4_K else [208]):
        raw[:, off + 1] &= 0x7B  # finite f16 scales, both signs
    packed = ops.repack(kind, raw, rows, cols)
    got = ops.unpack(kind, packed, rows, cols)
    want = orc.dequantize_rows(kind, raw, rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    enc = H.quantize(kind, rng.normal(0, 0.02, size=(rows, cols)).astype(np.float32))
    got = ops.unpack(kind, ops.repack(kind, enc, rows, cols), rows, cols)
    assert np.array_equal(got.view(np.uint32), orc.dequantize_rows(kind, enc, rows, cols).view(np.uint32))


# ---- embedding rows: bit-exact (q4_k_embedding, crates/nvidia/src/kernels/quantized/q4_k.cu:1-60) ------
@pytest.mark.parametrize("kind", [H.Q4_K, H.Q8_0, H.Q6_K])
def test_embedding_rows_bit_exact(ops, kind):
    vocab, hidden = 300, 512
    rng = np.random.default_rng(40 + kind)
    table = H.quantize(kind, rng.normal(0, 0.02, size=(vocab, hidden)).astype(np.float32))
    tokens = np.array([0, 299, 17, 17, 128, 1, 254], dtype=np.uint32)
    got = ops.embedding(kind, table, vocab, hidden, tokens)
    want = orc.dequantize_rows(kind, table, vocab, hidden)[tokens]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


# ---- per-head Q/K RMSNorm + rotary + F16 cache append (cuda_reference.rs:902-963, 1929-1972, 3368-3436) ------
def _qk_reference(q, k, v, qn, kn, positions, QH, KVH, HD, base, eps):
    """Oracle composition: per-head rms_norm with the shared weight, NeoX rotary, F16 bits of k and v."""
    T = len(positions)
    q2, k2 = np.empty_like(q), np.empty_like(k)
    for t in range(T):
        qh = np.concatenate([orc.rms_norm(q[t].reshape(QH, HD)[h], qn, eps) for h in range(QH)])
        kh = np.concatenate([orc.rms_norm(k[t].reshape(KVH, HD)[h], kn, eps) for h in range(KVH)])
        q2[t] = orc.rope_neox(qh, QH, HD, HD, base, int(positions[t]))
        k2[t] = orc.rope_neox(kh, KVH, HD, HD, base, int(positions[t]))
    return q2, k2, orc.f32_to_f16_bits(k2), orc.f32_to_f16_bits(v)


def test_qk_norm_rope_append_against_oracle(ops):
    QH, KVH, HD, T, base, eps = 8, 2, 128, 5, 1.0e6, 1.0e-6
    rng = np.random.default_rng(61)
    q = rng.normal(0, 1.5, size=(T, QH * HD)).astype(np.float32)
    k = rng.normal(0, 1.5, size=(T, KVH * HD)).astype(np.float32)
    v = rng.normal(0, 1.0, size=(T, KVH * HD)).astype(np.float32)
    qn = (1.0 + rng.normal(0, 0.2, HD)).astype(np.float32)
    kn = (1.0 + rng.normal(0, 0.2, HD)).astype(np.float32)
    positions = np.array([0, 1, 77, 4097, 16383], dtype=np.int32)
    slots = np.array([5, 0, 31, 18, 9], dtype=np.int32)
    cache_k = rng.integers(0, 65536, size=(32, KVH * HD)).astype(np.uint16)
    cache_v = rng.integers(0, 65536, size=(32, KVH * HD)).astype(np.uint16)
    gq, gk, ck, cv = ops.qk_norm_rope_append(q, k, v, qn, kn, positions, slots, QH, KVH, HD, base, eps, cache_k, cache_v)
    wq, wk, wkb, wvb = _qk_reference(q, k, v, qn, kn, positions, QH, KVH, HD, base, eps)
    assert np.max(np.abs(gq - wq)) < 1e-5 and np.max(np.abs(gk - wk)) < 1e-5
    assert np.array_equal(cv[slots], wvb)                               # v is rounded once: bit-exact
    assert np.array_equal(ck[slots], orc.f32_to_f16_bits(gk))           # the rounding of the device's own k is exact
    assert np.max(np.abs(ck[slots].view(np.float16).astype(np.float32) - wkb.view(np.float16).astype(np.float32))) < 4e-3
    untouched = np.setdiff1d(np.arange(32), slots)
    assert np.array_equal(ck[untouched], cache_k[untouched]) and np.array_equal(cv[untouched], cache_v[untouched])


@pytest.mark.parametrize("members,context", [(1, 1000), (2, 333), (16, 600)], ids=["direct-1", "direct-2", "staged-16"])
def test_fused_decode_attention_against_oracle(ops, members, context):
    """The decode step's fused kernels (Q/K norm, rotary, cache append, split-KV attention) on their own:
    one new token per sequence onto a cached context; appended rows and outputs against the oracle's."""
    QH, KVH, HD, base, eps = 32, 8, 128, 1.0e6, 1.0e-6
    rng = np.random.default_rng(70 + members)
    pages_per = (context + 16) // 16 + 1
    positions = np.array([context - 3 * m for m in range(members)], dtype=np.int32)
    tables = rng.permutation(members * pages_per).astype(np.int32).reshape(members, pages_per)
    physical = members * pages_per * 16
    cache_k = np.zeros((physical, KVH * HD), dtype=np.uint16)
    cache_v = np.zeros_like(cache_k)
    hist_k = rng.normal(0, 1, size=(members, context, KVH * HD)).astype(np.float16)
    hist_v = rng.normal(0, 1, size=(members, context, KVH * HD)).astype(np.float16)
    for m in range(members):
        for t in range(positions[m]):
            row = tables[m, t // 16] * 16 + t % 16
            cache_k[row] = hist_k[m, t].view(np.uint16)
            cache_v[row] = hist_v[m, t].view(np.uint16)
    q = rng.normal(0, 1.5, size=(members, QH * HD)).astype(np.float32)
    k = rng.normal(0, 1.5, size=(members, KVH * HD)).astype(np.float32)
    v = rng.normal(0, 1.0, size=(members, KVH * HD)).astype(np.float32)
    qn = (1.0 + rng.normal(0, 0.2, HD)).astype(np.float32)
    kn = (1.0 + rng.normal(0, 0.2, HD)).astype(np.float32)
    out, ck, cv = ops.attention_decode(q, k, v, qn, kn, base, eps, cache_k, cache_v, tables, positions, QH, KVH, HD)
    wq, wk, wkb, wvb = _qk_reference(q, k, v, qn, kn, positions, QH, KVH, HD, base, eps)
    for m in range(members):
        p = int(positions[m])
        row = tables[m, p // 16] * 16 + p % 16
        assert np.array_equal(cv[row], wvb[m])
        got_k = ck[row].view(np.float16).astype(np.float32)
        assert np.max(np.abs(got_k - wkb[m].view(np.float16).astype(np.float32))) < 4e-3   # one F16 step of |k| < 8
        keys = np.concatenate([hist_k[m, :p].reshape(-1).view(np.uint16), ck[row]])
        vals = np.concatenate([hist_v[m, :p].reshape(-1).view(np.uint16), cv[row]])
        want = orc.attention(wq[m], keys, vals, p + 1, QH, KVH, HD)
        assert np.max(np.abs(out[m] - want)) < 1e-3, m


def test_prefill_chunk_attention_at_16k_context(ops):
    """The chunked-prefill mix's largest shape: a 2048-token chunk onto a 14,336-token cached prefix
    (Qwen3-8B head geometry); sampled rows against the oracle, first and last rows included."""
    QH, KVH, HD, tokens, rows = 32, 8, 128, 16384, 2048
    rng = np.random.default_rng(16384)
    q = rng.normal(0, 1, size=(rows, QH * HD)).astype(np.float32)
    k = rng.normal(0, 1, size=(tokens, KVH * HD)).astype(np.float16)
    v = rng.normal(0, 1, size=(tokens, KVH * HD)).astype(np.float16)
    pages = tokens // 16
    table = rng.permutation(pages).astype(np.int32)
    pk = np.empty((tokens, KVH * HD), dtype=np.uint16)
    pv = np.empty_like(pk)
    order = (table[np.arange(tokens) // 16] * 16 + np.arange(tokens) % 16)
    pk[order] = k.view(np.uint16)
    pv[order] = v.view(np.uint16)
    got = ops.attention(q, pk, pv, table, tokens, rows, QH, KVH, HD, variant=0)
    kb, vb = k.view(np.uint16).reshape(-1), v.view(np.uint16).reshape(-1)
    for r in (0, 1, 511, 1024, 2046, 2047):
        seen = tokens - rows + 1 + r
        want = orc.attention(q[r], kb[: seen * KVH * HD], vb[: seen * KVH * HD], seen, QH, KVH, HD)
        assert np.max(np.abs(got[r] - want)) < 1e-3, r


@pytest.mark.parametrize("QH,KVH,HD,tokens", [(32, 8, 128, 40000), (16, 1, 64, 9000), (8, 2, 256, 3000)],
                         ids=["qwen3-8b-40k", "sixteen-heads-per-kv", "width-256"])
def test_decode_attention_at_long_contexts(ops, QH, KVH, HD, tokens):
    """One decode row over a long context: hundreds of spans through the merge (its span groups and shuffles),
    a group of sixteen query heads (two MMA column tiles) and head width 256; against the oracle, and paged ==
    contiguous bit for bit."""
    rng = np.random.default_rng(tokens + QH)
    q = rng.normal(0, 1, QH * HD).astype(np.float32)
    k = rng.normal(0, 1, size=(tokens, KVH * HD)).astype(np.float16)
    v = rng.normal(0, 1, size=(tokens, KVH * HD)).astype(np.float16)
    pages = (tokens + 15) // 16
    results = []
    for table in (np.arange(pages), rng.permutation(pages)):
        pk = np.zeros((pages * 16, KVH * HD), dtype=np.uint16); pv = np.zeros_like(pk)
        order = table[np.arange(tokens) // 16] * 16 + np.arange(tokens) % 16
        pk[order] = k.view(np.uint16); pv[order] = v.view(np.uint16)
        results.append(ops.attention(q, pk, pv, [int(t) for t in table], tokens, 1, QH, KVH, HD, variant=0)[0])
    assert np.array_equal(results[0].view(np.uint32), results[1].view(np.uint32))
    want = orc.attention(q, k.view(np.uint16).reshape(-1), v.view(np.uint16).reshape(-1), tokens, QH, KVH, HD)
    assert np.max(np.abs(results[0] - want)) < 1e-4
