"""The committed golden vectors (tests/golden/fixtures.json, made by tests/golden/make_golden.py from
the reference's fixture definitions with an independent float64 evaluation) against the CPU oracle
(not gpu) and against the CUDA library through the C ABI (gpu)."""
import json
import os

import numpy as np
import pytest

from oracle import binding as orc
from tests import helpers as H

with open(os.path.join(os.path.dirname(__file__), "golden", "fixtures.json")) as f:
    G = json.load(f)


def _bits(values):
    return np.asarray(values, dtype=np.uint32)


def _cases(impl):
    """impl: namespace with dequantize/gemv/rms_norm/silu_mul/argmax/rope/attention taking numpy arrays."""
    for case in G["dequant"]:
        enc = np.frombuffer(bytes.fromhex(case["bytes_hex"]), dtype=np.uint8)
        elems, size = H.BLOCK[case["type"]]
        got = impl.dequantize(case["type"], enc, enc.size // size * elems)
        assert np.array_equal(got.view(np.uint32).ravel(), _bits(case["f32_bits"])), case["type"]
    for case in G["gemv"]:
        enc = H.fixture(case["type"])
        x = H.fixture_input(case["cols"], case["member"])
        got = impl.gemv(case["type"], enc, case["rows"], case["cols"], x)
        assert np.max(np.abs(got.astype(np.float64) - np.array(case["y"]))) < case["tolerance"]
    c = G["rms_norm"]
    assert np.max(np.abs(impl.rms_norm(c["x"], c["weight"], c["eps"]) - np.array(c["y"]))) < c["tolerance"]
    c = G["silu_mul"]
    assert np.max(np.abs(impl.silu_mul(c["gate"], c["up"]) - np.array(c["y"]))) < c["tolerance"]
    c = G["argmax"]
    logits = np.zeros(c["length"], np.float32)
    for k, v in c["set"].items():
        logits[int(k)] = np.nan if v == "nan" else v
    assert impl.argmax(logits) == c["pick"]
    c = G["rope_neox"]
    got = impl.rope(np.array(c["x"], np.float32), c["heads"], c["head_dim"], c["rot"], c["base"], c["position"])
    assert np.max(np.abs(got.astype(np.float64) - np.array(c["y"]))) < c["tolerance"]
    c = G["attention"]
    got = impl.attention(np.array(c["q"], np.float32), np.array(c["k"], np.float32), np.array(c["v"], np.float32),
                         c["tokens"], c["q_heads"], c["kv_heads"], c["head_dim"])
    assert np.max(np.abs(got.astype(np.float64).ravel() - np.array(c["y"]))) < c["tolerance"]


class _Oracle:
    dequantize = staticmethod(lambda t, enc, count: orc.dequantize_rows(t, enc, 1, count))
    gemv = staticmethod(lambda t, enc, rows, cols, x: orc.gemv(t, enc, cols, rows, x))
    rms_norm = staticmethod(lambda x, w, eps: orc.rms_norm(x, w, eps))
    silu_mul = staticmethod(lambda g, u: orc.silu_mul(g, u))
    argmax = staticmethod(lambda l: orc.argmax(l))
    rope = staticmethod(lambda v, heads, hd, rot, base, pos: orc.rope_neox(v, heads, hd, rot, base, pos))

    @staticmethod
    def attention(q, k, v, tokens, qh, kvh, hd):
        return orc.attention(q, k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16), tokens, qh, kvh, hd)


def test_oracle_reproduces_the_golden_vectors():
    _cases(_Oracle)


@pytest.mark.gpu
def test_cuda_library_reproduces_the_golden_vectors(built_library):
    from ribn_b200 import ops

    class Cuda:
        dequantize = staticmethod(lambda t, enc, count: ops.dequantize(t, enc, 1, count))
        gemv = staticmethod(lambda t, enc, rows, cols, x: ops.gemv(t, enc, rows, cols, x, variant=1 if cols % 256 else 0))
        rms_norm = staticmethod(lambda x, w, eps: ops.rms_norm(np.array(x, np.float32), w, eps))
        silu_mul = staticmethod(lambda g, u: ops.silu_mul(g, u))
        argmax = staticmethod(lambda l: ops.argmax(l))
        rope = staticmethod(lambda v, heads, hd, rot, base, pos: ops.rope_neox(v, [pos], heads, hd, rot, base))

        @staticmethod
        def attention(q, k, v, tokens, qh, kvh, hd):
            pages = (tokens + 15) // 16
            keys = np.zeros((pages * 16, kvh * hd), np.float16); keys[:tokens] = k.reshape(tokens, kvh * hd)
            vals = np.zeros((pages * 16, kvh * hd), np.float16); vals[:tokens] = v.reshape(tokens, kvh * hd)
            return ops.attention(q, keys.view(np.uint16), vals.view(np.uint16), np.arange(pages), tokens, 1, qh, kvh, hd)

    _cases(Cuda)
