"""ctypes loader for ``liboracle.so`` — the CPU restatement of the reference's
host equations.  TEST INFRASTRUCTURE ONLY: the shipped library never imports
this module, and a missing CUDA extension is never papered over with it."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

F32, F16, Q8_0, Q4_K, Q6_K = 0, 1, 8, 12, 14


class Qwen3Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn", "vocab", "context")] + \
               [("rope_base", C.c_float), ("eps", C.c_float)]


def build(force: bool = False) -> str:
    path = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith(".c")]
    stale = (not os.path.exists(path)) or any(os.path.getmtime(s) > os.path.getmtime(path) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return path


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        L = _LIB
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_dequantize_block.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_dequantize_row.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_gemv.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        L.orc_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_void_p]
        L.orc_rope_neox.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int64]
        L.orc_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        V = C.c_void_p
        L.orc_gdn_scalar_gate.argtypes = [V, V, V, V, C.c_int, V, V]
        L.orc_gdn_conv_silu.argtypes = [V, V, V, C.c_int, V, V]
        L.orc_l2_norm_heads.argtypes = [V, C.c_int, C.c_int, C.c_float]
        L.orc_gdn_state_update.argtypes = [V, V, V, V, V, V, C.c_int, C.c_int, C.c_int, C.c_int, V]
        L.orc_gdn_gated_norm.argtypes = [V, V, V, C.c_int, C.c_int, C.c_float, V]
        L.orc_gdn_step.argtypes = [C.c_int, C.c_int, C.c_int, V, V, V, V, V, V, V, V, V, V, C.c_float, C.c_float, V, V, V, V, V]
        L.orc_attention_gate.argtypes = [V, V, C.c_int, C.c_int, C.c_int, V]
        L.orc_argmax.restype = C.c_uint32
        L.orc_argmax.argtypes = [C.c_void_p, C.c_int64]
        L.orc_attention.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.orc_qwen3_create.restype = C.c_void_p
        L.orc_qwen3_create.argtypes = [C.POINTER(Qwen3Config)]
        L.orc_qwen3_destroy.argtypes = [C.c_void_p]
        L.orc_qwen3_set_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int]
        L.orc_qwen3_seq_create.restype = C.c_void_p
        L.orc_qwen3_seq_create.argtypes = [C.c_void_p]
        L.orc_qwen3_seq_destroy.argtypes = [C.c_void_p]
        L.orc_qwen3_seq_position.argtypes = [C.c_void_p]
        L.orc_qwen3_seq_fill.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_qwen3_step.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.orc_qwen3_seq_cache.restype = C.c_void_p
        L.orc_qwen3_seq_cache.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_set_threads.argtypes = [C.c_int]
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def block_elems(t: int) -> int:
    return lib().orc_block_elems(t)


def block_bytes(t: int) -> int:
    return lib().orc_block_bytes(t)


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


def dequantize_block(t: int, encoded: bytes) -> np.ndarray:
    """engine_gguf::dequantize_block: raises ValueError like the reference's
    UnsupportedTensorType / InvalidTensorBlockLength errors."""
    n = block_elems(t)
    if n == 0:
        raise ValueError(f"unsupported tensor type {t}")
    buf = np.frombuffer(bytes(encoded), dtype=np.uint8).copy()
    out = np.empty(n, dtype=np.float32)
    rc = lib().orc_dequantize_block(t, _p(buf), len(buf), _p(out))
    if rc == -2:
        raise ValueError(f"invalid block length: type {t} expected {block_bytes(t)} actual {len(buf)}")
    if rc != 0:
        raise ValueError(f"unsupported tensor type {t}")
    return out


def dequantize_rows(t: int, encoded: np.ndarray, n: int, k: int) -> np.ndarray:
    enc = np.ascontiguousarray(encoded, dtype=np.uint8).reshape(-1)
    out = np.empty((n, k), dtype=np.float32)
    assert lib().orc_dequantize_row(t, _p(enc), n * k, _p(out)) == 0
    return out


def gemv(t: int, w: np.ndarray, k: int, n: int, x: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(n, dtype=np.float32)
    assert lib().orc_gemv(t, _p(w), k, n, _p(x), _p(y)) == 0
    return y


def rms_norm(x, w, eps) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x), _p(w), x.size, eps, _p(out))
    return out


def rope_neox(v, heads, head_dim, rot, base, pos) -> np.ndarray:
    v = np.ascontiguousarray(v, dtype=np.float32).copy()
    lib().orc_rope_neox(_p(v), heads, head_dim, rot, base, pos)
    return v


def silu_mul(g, u) -> np.ndarray:
    g = np.ascontiguousarray(g, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float32)
    out = np.empty_like(g)
    lib().orc_silu_mul(_p(g), _p(u), g.size, _p(out))
    return out


# ---- Gated-DeltaNet recurrent layer step and the attention output gate (oracle/gdn.c) ----------------
def _f(v):
    return np.ascontiguousarray(v, dtype=np.float32)


def gdn_scalar_gate(alpha, beta_raw, dt_bias, a):
    alpha, beta_raw, dt_bias, a = _f(alpha), _f(beta_raw), _f(dt_bias), _f(a)
    decay, beta = np.empty_like(alpha), np.empty_like(alpha)
    lib().orc_gdn_scalar_gate(_p(alpha), _p(beta_raw), _p(dt_bias), _p(a), alpha.size, _p(decay), _p(beta))
    return decay, beta


def gdn_conv_silu(x, weight, history):
    """Returns (raw, activated, advanced history); history [channels][3] oldest first, weight [channels][4]."""
    x, weight, history = _f(x), _f(weight), _f(history).copy()
    raw, act = np.empty_like(x), np.empty_like(x)
    lib().orc_gdn_conv_silu(_p(x), _p(weight), _p(history), x.size, _p(raw), _p(act))
    return raw, act, history


def l2_norm_heads(values, heads: int, head_dim: int, eps: float) -> np.ndarray:
    v = _f(values).copy()
    lib().orc_l2_norm_heads(_p(v), heads, head_dim, eps)
    return v


def gdn_state_update(matrix, q, k, conv, decay, beta, v_heads: int, k_heads: int, head_dim: int, v_offset: int):
    """Returns (out [v_heads * head_dim], updated matrix)."""
    m = _f(matrix).copy()
    q, k, conv, decay, beta = _f(q), _f(k), _f(conv), _f(decay), _f(beta)
    out = np.empty(v_heads * head_dim, dtype=np.float32)
    lib().orc_gdn_state_update(_p(m), _p(q), _p(k), _p(conv), _p(decay), _p(beta), v_heads, k_heads, head_dim, v_offset, _p(out))
    return out, m


def gdn_gated_norm(o, z, norm, heads: int, head_dim: int, eps: float) -> np.ndarray:
    o, z, norm = _f(o), _f(z), _f(norm)
    out = np.empty_like(o)
    lib().orc_gdn_gated_norm(_p(o), _p(z), _p(norm), heads, head_dim, eps, _p(out))
    return out


def gdn_step(qkv, z, beta_raw, alpha_raw, dt_bias, a, conv_weight, norm_weight, conv_state, state, k_heads: int,
             v_heads: int, head_dim: int, l2_eps: float, norm_eps: float):
    """One sequence's step behind the projections; returns the same dict as ribn_b200.ops.gdn_step (one member)."""
    channels, inner = (2 * k_heads + v_heads) * head_dim, v_heads * head_dim
    qkv, z, br, ar = _f(qkv), _f(z), _f(beta_raw), _f(alpha_raw)
    conv, st = _f(conv_state).copy(), _f(state).copy()
    decay, beta = np.empty(v_heads, np.float32), np.empty(v_heads, np.float32)
    act, attn, out = np.empty(channels, np.float32), np.empty(inner, np.float32), np.empty(inner, np.float32)
    dt, aa, cw, nw = _f(dt_bias), _f(a), _f(conv_weight), _f(norm_weight)
    lib().orc_gdn_step(k_heads, v_heads, head_dim, _p(qkv), _p(z), _p(br), _p(ar), _p(dt), _p(aa), _p(cw), _p(nw), _p(conv),
                       _p(st), l2_eps, norm_eps, _p(decay), _p(beta), _p(act), _p(attn), _p(out))
    return dict(out=out, decay=decay, beta=beta, conv_act=act, attn_out=attn, conv_state=conv, state=st)


def attention_gate(attn, q_gate, rows: int, heads: int, head_dim: int) -> np.ndarray:
    attn, q_gate = _f(attn), _f(q_gate)
    out = np.empty_like(attn)
    lib().orc_attention_gate(_p(attn), _p(q_gate), rows, heads, head_dim, _p(out))
    return out


def argmax(logits) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().orc_argmax(_p(logits), logits.size))


def f32_to_f16_bits(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    L = lib()
    return np.array([L.orc_f32_to_f16(float(v)) for v in a.reshape(-1)], dtype=np.uint16).reshape(a.shape)


def attention(q, keys_f16, values_f16, tokens, q_heads, kv_heads, head_dim) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(keys_f16, dtype=np.uint16)
    v = np.ascontiguousarray(values_f16, dtype=np.uint16)
    out = np.empty(q_heads * head_dim, dtype=np.float32)
    lib().orc_attention(_p(q), _p(k), _p(v), tokens, q_heads, kv_heads, head_dim, _p(out))
    return out


class Qwen3Oracle:
    """Dense Qwen3 decoder on the CPU, one token at a time per sequence."""

    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = Qwen3Config(**{k: cfg[k] for k, _ in Qwen3Config._fields_})
        self._h = lib().orc_qwen3_create(C.byref(self.cfg))
        self._keep = []
        for name, (t, n, k, data) in tensors.items():
            arr = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
            self._keep.append(arr)
            rc = lib().orc_qwen3_set_tensor(self._h, name.encode(), t, n, k, _p(arr), 0)
            if rc != 0:
                raise ValueError(f"oracle rejected tensor {name}")

    def new_sequence(self):
        return Qwen3OracleSeq(self)

    def close(self):
        if self._h:
            lib().orc_qwen3_destroy(self._h)
            self._h = None


class Qwen3OracleSeq:
    def __init__(self, model: Qwen3Oracle):
        self.model = model
        self._h = lib().orc_qwen3_seq_create(model._h)

    @property
    def position(self) -> int:
        return lib().orc_qwen3_seq_position(self._h)

    def fill(self, keys: np.ndarray, values: np.ndarray, tokens: int):
        keys = np.ascontiguousarray(keys, dtype=np.uint16)
        values = np.ascontiguousarray(values, dtype=np.uint16)
        assert lib().orc_qwen3_seq_fill(self._h, tokens, _p(keys), _p(values)) == 0

    def step(self, token: int, want_logits: bool = True, want_hidden: bool = False):
        cfg = self.model.cfg
        logits = np.empty(cfg.vocab, dtype=np.float32) if want_logits else None
        hidden = np.empty(cfg.hidden, dtype=np.float32) if want_hidden else None
        rc = lib().orc_qwen3_step(self._h, int(token),
                                  _p(logits) if logits is not None else None,
                                  _p(hidden) if hidden is not None else None)
        if rc != 0:
            raise RuntimeError("oracle step failed")
        if want_hidden:
            return logits, hidden
        return logits

    def cache(self, layer: int, which: int, tokens: int) -> np.ndarray:
        cfg = self.model.cfg
        ptr = lib().orc_qwen3_seq_cache(self._h, layer, which)
        n = tokens * cfg.kv_heads * cfg.head_dim
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint16)), shape=(n,)).copy()

    def close(self):
        if self._h:
            lib().orc_qwen3_seq_destroy(self._h)
            self._h = None
