"""Pins the CPU oracle against the reference's own known answers.

Every expectation here is a value the reference's tests state
(crates/gguf/src/lib.rs:1479-1582; crates/nvidia/tests/cuda_reference.rs) or a
closed-form property of its equations; the oracle is only trusted by the GPU
parity tests because these pass."""
import struct

import numpy as np
import pytest

from oracle import binding as orc
from tests import helpers as H


def bits(x) -> int:
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


# --- crates/gguf/src/lib.rs:1479-1565 -----------------------------------------------------
def test_scalar_blocks_known_answers():
    assert bits(orc.dequantize_block(orc.F32, struct.pack("<f", 1.5))[0]) == bits(1.5)
    assert bits(orc.dequantize_block(orc.F16, struct.pack("<H", 0x3C00))[0]) == bits(1.0)


def test_q8_0_known_answer():
    q8 = bytearray(34)
    q8[0:2] = struct.pack("<H", 0x3C00)
    q8[2], q8[3] = 0x80, 0x7F
    out = orc.dequantize_block(orc.Q8_0, bytes(q8))
    assert len(out) == 32 and bits(out[0]) == bits(-128.0) and bits(out[1]) == bits(127.0)


def test_q4_k_known_answer():
    q4 = bytearray(144)
    q4[0:2] = struct.pack("<H", 0x3C00)
    q4[4:8] = b"\x01" * 4
    q4[16] = 0x10
    out = orc.dequantize_block(orc.Q4_K, bytes(q4))
    assert len(out) == 256 and bits(out[0]) == bits(0.0) and bits(out[32]) == bits(1.0)


def test_q6_k_known_answer():
    q6 = bytearray(210)
    q6[192:208] = b"\x01" * 16
    q6[208:210] = struct.pack("<H", 0x3C00)
    out = orc.dequantize_block(orc.Q6_K, bytes(q6))
    assert len(out) == 256 and all(bits(v) == bits(-32.0) for v in out)


def test_rejects_invalid_blocks():
    # lib.rs:1567-1582: short Q4_K block; unsupported type 22
    with pytest.raises(ValueError, match="expected 144 actual 143"):
        orc.dequantize_block(orc.Q4_K, bytes(143))
    with pytest.raises(ValueError, match="unsupported"):
        orc.dequantize_block(22, bytes(82))


# --- f16 conversions --------------------------------------------------------------------
def test_f16_to_f32_is_exact_for_every_pattern():
    patterns = np.arange(0x10000, dtype=np.uint16)
    want = patterns.view(np.float16).astype(np.float32)
    L = orc.lib()
    got = np.array([L.orc_f16_to_f32(int(p)) for p in patterns], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.all(np.isnan(got[~finite]))


def test_f32_to_f16_rounds_to_nearest_even():
    # cuda_reference.rs:3368-3436 checks kv_append_f16's rounding; numpy's float16 cast is IEEE RNE.
    rng = np.random.default_rng(7)
    vals = np.concatenate([
        rng.normal(0, 1, 4000), rng.normal(0, 1e-5, 2000), rng.normal(0, 3e4, 2000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e6, -1e6, 6e-8, 2.98e-8, 2.99e-8, 1.0009765625,
                  1.00048828125, 1.00146484375, np.inf, -np.inf]),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = orc.f32_to_f16_bits(vals)
    assert np.array_equal(got, want)


# --- decoder vs an independent numpy decoder, random blocks ---------------------------------
@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
def test_decoder_matches_independent_numpy_decoder(kind):
    rng = np.random.default_rng(kind)
    elems, size = H.BLOCK[kind]
    blocks = rng.integers(0, 256, size=(200, size), dtype=np.uint8)
    # keep the f16 scale fields finite
    for off in ([0] if kind == H.Q8_0 else [0, 2] if kind == H.Q4_K else [208]):
        blocks[:, off + 1] &= 0x3B
    want = H.np_dequant(kind, blocks.reshape(-1)).reshape(200, elems)
    got = orc.dequantize_rows(kind, blocks, 200, elems)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("kind", [H.Q8_0, H.Q4_K, H.Q6_K])
def test_quantiser_round_trip_is_close(kind):
    # the test-only quantisers produce valid blocks whose decode is near the source values
    rng = np.random.default_rng(3)
    x = rng.normal(0, 0.02, size=(4, 512)).astype(np.float32)
    enc = H.quantize(kind, x)
    back = orc.dequantize_rows(kind, enc, 4, 512)
    tol = {H.Q8_0: 4e-4, H.Q4_K: 8e-3, H.Q6_K: 2e-3}[kind]
    assert np.max(np.abs(back - x)) < tol


# --- GEMV fixtures: cuda_reference.rs:690-846 -------------------------------------------------
@pytest.mark.parametrize("kind,rows,cols", [(H.Q4_K, 2, 512), (H.Q6_K, 2, 512), (H.Q8_0, 2, 96)])
def test_gemv_fixture_against_sequential_sum(kind, rows, cols):
    enc = H.fixture(kind)
    x = H.fixture_input(cols)
    w = H.np_dequant(kind, enc).reshape(rows, cols)
    want = np.zeros(rows, dtype=np.float32)
    for r in range(rows):
        acc = np.float32(0.0)
        for k in range(cols):
            acc = np.float32(acc + np.float32(w[r, k] * x[k]))
        want[r] = acc
    got = orc.gemv(kind, enc, cols, rows, x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_gemv_threads_do_not_change_bits():
    rng = np.random.default_rng(11)
    enc = H.quantize(H.Q4_K, rng.normal(0, 0.02, size=(64, 512)).astype(np.float32))
    x = rng.normal(0, 1, 512).astype(np.float32)
    orc.set_threads(1)
    a = orc.gemv(H.Q4_K, enc, 512, 64, x)
    orc.set_threads(4)
    b = orc.gemv(H.Q4_K, enc, 512, 64, x)
    orc.set_threads(1)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


# --- elementwise: cuda_reference.rs:902-963 ---------------------------------------------------
def test_rms_norm_known_values():
    x = np.array([1.0, -2.0, 3.0, -4.0], dtype=np.float32)
    w = np.array([1.0, 0.5, 2.0, -1.0], dtype=np.float32)
    inv = np.float32(1.0) / np.sqrt(np.float32(np.float32(30.0) / np.float32(4.0) + np.float32(1e-5)))
    want = (x * inv * w).astype(np.float32)
    got = orc.rms_norm(x, w, 1e-5)
    assert np.allclose(got, want, atol=1e-6)
    assert abs(got[0] - 0.36514813) < 1e-6 and abs(got[3] - 1.4605925) < 1e-6


def test_silu_ramp():
    i = np.arange(513, dtype=np.float32)
    gate, up = i * np.float32(0.01) - np.float32(2.5), np.float32(1.0) - i * np.float32(0.002)
    want = gate.astype(np.float64) / (1.0 + np.exp(-gate.astype(np.float64))) * up
    assert np.max(np.abs(orc.silu_mul(gate, up) - want)) < 1e-5


def test_argmax_tie_takes_lowest_index_and_skips_nan():
    logits = np.full(513, -10.0, dtype=np.float32)
    logits[401] = logits[402] = 7.0
    assert orc.argmax(logits) == 401
    logits[5] = np.nan
    assert orc.argmax(logits) == 401
    assert orc.argmax(np.full(8, np.nan, dtype=np.float32)) == 0
    assert orc.argmax(np.array([-np.inf, -np.inf], dtype=np.float32)) == 0


# --- rope: cuda_reference.rs:1929-1972 ----------------------------------------------------------
def test_rope_neox_reference_geometry():
    heads, hd, rot, base, pos = 4, 256, 64, 1.0e7, 3
    host = ((np.arange(heads * hd) % 97).astype(np.float32) * np.float32(0.03) - np.float32(1.4)).astype(np.float32)
    got = orc.rope_neox(host, heads, hd, rot, base, pos)
    want = host.astype(np.float64).copy()
    for h in range(heads):
        for p in range(rot // 2):
            theta = pos * base ** (-(2.0 * p) / rot)
            x0, x1 = host[h * hd + p], host[h * hd + rot // 2 + p]
            want[h * hd + p] = x0 * np.cos(theta) - x1 * np.sin(theta)
            want[h * hd + rot // 2 + p] = x0 * np.sin(theta) + x1 * np.cos(theta)
    assert np.max(np.abs(got - want)) < 1e-5
    assert np.array_equal(got.reshape(heads, hd)[:, rot:], host.reshape(heads, hd)[:, rot:])  # pass-through dims


# --- attention: cuda_reference.rs:1995-2093 (without the Qwen3.5 output gate) ---------------------
def test_attention_lcg_fixture_against_float64_softmax():
    QH, KVH, HD, T = 6, 2, 32, 3
    state = 12345
    q, state = H.lcg_f16_values(state, QH * HD)
    _gate, state = H.lcg_f16_values(state, QH * 2 * HD)
    k, state = H.lcg_f16_values(state, T * KVH * HD)
    v, state = H.lcg_f16_values(state, T * KVH * HD)
    kb, vb = k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16)
    assert np.array_equal(kb, orc.f32_to_f16_bits(k))  # the fixture is exact in F16
    got = orc.attention(q, kb, vb, T, QH, KVH, HD).reshape(QH, HD)
    k3, v3 = k.reshape(T, KVH, HD).astype(np.float64), v.reshape(T, KVH, HD).astype(np.float64)
    for qh in range(QH):
        kvh = qh // (QH // KVH)
        s = (k3[:, kvh, :] @ q.reshape(QH, HD)[qh].astype(np.float64)) / np.sqrt(HD)
        p = np.exp(s - s.max())
        p /= p.sum()
        assert np.max(np.abs(got[qh] - p @ v3[:, kvh, :])) < 1e-3


# --- the composed model --------------------------------------------------------------------------
def test_tiny_model_steps_are_deterministic_and_causal():
    cfg = H.TINY
    tensors = H.make_model(cfg, seed=5)
    model = orc.Qwen3Oracle(H.oracle_config(cfg, 64), tensors)
    a, b = model.new_sequence(), model.new_sequence()
    toks = [3, 77, 200, 9]
    la = [a.step(t) for t in toks]
    lb = [b.step(t) for t in toks[:3]] + [b.step(10)]
    for i in range(3):
        assert np.array_equal(la[i], lb[i])
    assert not np.array_equal(la[3], lb[3])
    assert a.position == 4 and np.all(np.isfinite(la[3]))
    a.close(); b.close(); model.close()
