"""Pins the Gemma-4 CPU oracle (oracle/gemma.c) to the reference's own known answers, read from its
test sources: crates/gemma4/tests/cpu_ops.rs:21-135 (linear, RMS, rotary, factors),
crates/gemma4/tests/cpu_attention.rs:23-123 (masks, grouping, softmax, invalid spans) and
crates/gemma4/tests/rotary.rs:9-68 with tests/fixtures/rotary.json (inverse frequencies)."""
import json
import math
import os

import numpy as np
import pytest

from oracle import gemma_binding as G

HERE = os.path.dirname(os.path.abspath(__file__))


def b(*values):
    return G.bf16(np.array(values, dtype=np.float32))


def f(bits):
    return G.to_f32(np.array(bits, dtype=np.uint16))


def test_bf16_rounds_to_nearest_even_and_keeps_nan_canonical():
    assert list(b(1.0, -2.0, 0.0)) == [0x3F80, 0xC000, 0x0000]
    # 1 + 2^-8 is a tie between 0x3f80 and 0x3f81: even wins; 1 + 3 * 2^-8 ties upward to 0x3f82
    assert list(b(1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8)) == [0x3F80, 0x3F82]
    assert int(G.lib().orc_gm_bf16(float("nan"))) == 0x7FC0
    rng = np.random.default_rng(3)
    x = rng.standard_normal(4096).astype(np.float32) * 37.0
    assert np.array_equal(G.bf16(x), G.bf16_fast(x))


def test_linear_rounds_once_after_fp32_accumulation():
    w = b(1.0, 2.0, 4.0, 0.5, -1.0, 2.0)
    assert list(G.project(b(1.0, 1.0, 1.0), 1, w, 2, 3)) == list(b(7.0, 1.5))
    w = b(0.1, 0.2, 0.3)
    v = f(w)
    expected = np.float32(np.float32(v[0] + v[1]) + v[2])
    assert list(G.project(b(1.0, 1.0, 1.0), 1, w, 1, 3)) == list(b(expected))


def test_rms_normalizes_with_fp32_statistics_and_direct_scale():
    out = G.rms_norm(b(3.0, 4.0), 1, 2, 1e-6, b(1.0, 1.0))
    inverse = np.float32(np.float32(12.5) + np.float32(1e-6)) ** np.float32(-0.5)
    assert list(out) == list(b(np.float32(3.0) * inverse, np.float32(4.0) * inverse))
    # scale-free form (value normalisation)
    assert list(G.rms_norm(b(3.0, 4.0), 1, 2, 1e-6, None)) == list(out)


def test_rotary_rounds_each_product_and_reads_both_factor_halves():
    out = G.apply_rotary(np.array([0x8000, b(-2.0)[0]], np.uint16), 1, 1, 2, b(1.0, 1.0), b(0.0, 0.0))
    assert list(out) == [0x0000, b(-2.0)[0]]
    out = G.apply_rotary(b(2.0, 4.0), 1, 1, 2, b(1.0, 0.5), b(0.0, 0.25))
    assert list(out) == list(b(2.0 * 1.0 + (-4.0) * 0.0, 4.0 * 0.5 + 2.0 * 0.25))
    out = G.apply_rotary(b(3.0, -4.0), 1, 1, 2, b(0.0, 0.0), b(1.0, 1.0))
    assert list(out) == list(b(4.0, 3.0))


def test_factors_duplicate_halves_and_keep_padded_frequencies_identity():
    width = 512  # the pinned checkpoint's global head width, proportional rotary with theta 1e6
    cos, sin = G.factors(width, 1.0e6, True, [0, 5])
    cos, sin = cos.reshape(2, width), sin.reshape(2, width)
    assert np.array_equal(cos[:, : width // 2], cos[:, width // 2:])
    assert np.array_equal(sin[:, : width // 2], sin[:, width // 2:])
    assert np.all(cos[0] == 0x3F80) and np.all(sin[0] == 0x0000)
    active = width // 4
    assert np.all(cos[1, active: width // 2] == 0x3F80) and np.all(sin[1, active: width // 2] == 0x0000)
    # the rotated quarter is not the identity at a non-zero position
    assert np.any(sin[1, : width // 8] != 0)


def test_inverse_frequencies_match_the_reference_fixture():
    doc = json.load(open(os.path.join(HERE, "golden", "gemma_rotary.json")))
    checked = 0
    for case in doc["cases"]:
        for kind in case["kinds"].values():
            hd, theta, prop = kind["head_dim"], kind["theta"], kind["proportional"]
            bits = kind["inverse_frequency_bits"]
            assert len(bits) == hd // 2
            for pair, want in enumerate(bits):
                got = np.float32(G.inverse_frequency(hd, theta, prop, pair)).view(np.uint32)
                if want == 0:
                    assert got == 0 and prop and pair >= hd // 8
                    continue
                assert abs(int(got) - int(want)) <= 4, (case["name"], hd, pair)
                exponent = np.float32(2 * pair) / np.float32(hd)
                exact = float(np.float32(theta)) ** (-float(exponent))
                assert abs(float(np.uint32(got).view(np.float32)) - exact) / exact <= 3 * 2.0 ** -23
                checked += 1
            assert np.float32(G.inverse_frequency(hd, theta, prop, 0)).view(np.uint32) == np.float32(1).view(np.uint32)
    assert checked == 128 + 64 + 5 + 2


def test_causal_and_sliding_masks_expose_only_visible_keys():
    q, k, v = b(1, 1, 1, 1), b(0, 0, 0, 0), b(1, 2, 3, 4)
    assert list(G.attention(q, k, v, 1, 1, 1, None, 0, 0)) == list(b(1.0, 1.5, 2.0, 2.5))
    assert list(G.attention(q, k, v, 1, 1, 1, 2, 0, 0)) == list(b(1.0, 1.5, 2.5, 3.5))


def test_grouped_heads_share_key_value_heads_and_softmax_normalizes():
    out = G.attention(b(1, 1, 1, 1), b(0, 0), b(10, 20), 4, 2, 1, None, 0, 0)
    assert list(out) == list(b(10, 10, 20, 20))
    out = G.attention(b(1.0), b(1.0, 0.0), b(1.0, 2.0), 1, 1, 1, None, 1, 0)
    e1, e0 = np.exp(np.float32(1.0)), np.float32(1.0)
    total = np.float32(e1 + e0)
    # weights are rounded to BF16 before they meet the values
    w1, w0 = f(b(e1 / total))[0], f(b(e0 / total))[0]
    assert list(out) == list(b(np.float32(w1 * np.float32(1.0)) + np.float32(w0 * np.float32(2.0))))


def test_invalid_attention_spans_reject():
    z = b(0.0, 0.0)
    with pytest.raises(ValueError):
        G.attention(z, z, z, 1, 1, 1, None, 1, 0)   # a query beyond the key span
    with pytest.raises(ValueError):
        G.attention(z, z, z, 1, 1, 1, None, 0, 1)   # queries before the key span
    with pytest.raises(ValueError):
        G.attention(b(0, 0, 0), z, z, 3, 2, 1, None, 0, 0)  # non-whole head groups


def test_elementwise_rounding_boundaries():
    x = b(0.5, -1.25, 3.0)
    xs = f(x)
    alpha, cubic = np.float32(0.7978846), np.float32(0.044715)
    inner = alpha * xs * (np.float32(1.0) + cubic * xs * xs)
    want = b(*(np.float32(0.5) * xs * (np.float32(1.0) + np.tanh(inner.astype(np.float32)))))
    got = G.gelu_tanh(x)
    assert np.max(np.abs(got.astype(np.int32) - want.astype(np.int32))) <= 1
    # soft cap: three roundings
    logits = b(12.0, -45.0, 0.25)
    d = G.bf16(f(logits) / np.float32(30.0))
    h = G.bf16(np.tanh(f(d)).astype(np.float32))
    assert np.max(np.abs(G.softcap(logits, 30.0).astype(np.int32) - G.bf16(f(h) * np.float32(30.0)).astype(np.int32))) <= 1
    # per-layer combine: (a + b) rounded, then * 2^-1/2 rounded
    s = G.bf16(f(b(1.0, 2.0)) + f(b(0.5, 0.125)))
    assert list(G.ple_combine(b(1.0, 2.0), b(0.5, 0.125))) == list(G.bf16(f(s) * np.float32(math.sqrt(0.5))))
    assert G.argmax(b(1.0, 3.0, 3.0, 2.0)) == 1
    assert G.argmax(np.array([0x7FC0, b(5.0)[0]], np.uint16)) == 0  # NaN incumbent is never replaced
