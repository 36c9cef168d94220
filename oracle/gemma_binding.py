"""ctypes view of the Gemma-4 half of ``liboracle.so`` (``oracle/gemma.c``).  TEST INFRASTRUCTURE
ONLY: the shipped library never imports this module.  BF16 tensors travel as ``numpy.uint16``."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import binding

MAX_LAYERS = 64


class GemmaConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "layers", "hidden", "heads", "kv_heads", "head_dim", "global_head_dim", "ffn", "vocab", "ple", "ple_vocab",
        "window", "context", "kv_shared")] + \
        [(n, C.c_float) for n in ("eps", "softcap", "theta_local", "theta_global")] + \
        [("full", C.c_int32 * MAX_LAYERS)]


def make_config(cfg: dict) -> GemmaConfig:
    """cfg: the integer / float fields above plus ``layer_types`` (list of 'sliding' / 'full')."""
    c = GemmaConfig()
    for name, _ in GemmaConfig._fields_:
        if name != "full":
            setattr(c, name, cfg[name])
    for i, kind in enumerate(cfg["layer_types"]):
        c.full[i] = 1 if kind == "full" else 0
    return c


_READY = False


def lib() -> C.CDLL:
    global _READY
    L = binding.lib()
    if not _READY:
        P = C.c_void_p
        L.orc_gm_bf16.restype = C.c_uint16
        L.orc_gm_bf16.argtypes = [C.c_float]
        L.orc_gm_project.argtypes = [P, C.c_int, P, C.c_int64, C.c_int64, P]
        L.orc_gm_rms_norm.argtypes = [P, C.c_int, C.c_int, C.c_float, P, P]
        L.orc_gm_inverse_frequency.restype = C.c_float
        L.orc_gm_inverse_frequency.argtypes = [C.c_int, C.c_float, C.c_int, C.c_int]
        L.orc_gm_factors.argtypes = [C.c_int, C.c_float, C.c_int, P, C.c_int, P, P]
        L.orc_gm_apply_rotary.argtypes = [P, C.c_int, C.c_int, C.c_int, P, P, P]
        L.orc_gm_attention.argtypes = [P, C.c_int, P, P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, P]
        for name in ("orc_gm_add", "orc_gm_multiply"):
            getattr(L, name).argtypes = [P, P, C.c_int64, P]
        L.orc_gm_scale.argtypes = [P, C.c_float, C.c_int64, P]
        L.orc_gm_gelu_tanh.argtypes = [P, C.c_int64, P]
        L.orc_gm_softcap.argtypes = [P, C.c_float, C.c_int64, P]
        L.orc_gm_ple_combine.argtypes = [P, P, C.c_int64, P]
        L.orc_gm_argmax.restype = C.c_uint32
        L.orc_gm_argmax.argtypes = [P, C.c_int64]
        L.orc_gemma_create.restype = P
        L.orc_gemma_create.argtypes = [C.POINTER(GemmaConfig)]
        L.orc_gemma_destroy.argtypes = [P]
        L.orc_gemma_set_tensor.argtypes = [P, C.c_char_p, P, C.c_int64]
        L.orc_gemma_ready.argtypes = [P]
        L.orc_gemma_seq_create.restype = P
        L.orc_gemma_seq_create.argtypes = [P]
        L.orc_gemma_seq_destroy.argtypes = [P]
        L.orc_gemma_seq_position.argtypes = [P]
        L.orc_gemma_seq_reset.argtypes = [P]
        L.orc_gemma_step.argtypes = [P, P, C.c_int, P, P]
        _READY = True
    return L


def _u16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def bf16(values) -> np.ndarray:
    """FP32 -> BF16 bits, round to nearest even (the oracle's own rounding, element by element)."""
    a = np.ascontiguousarray(values, dtype=np.float32)
    L = lib()
    return np.array([L.orc_gm_bf16(float(v)) for v in a.reshape(-1)], dtype=np.uint16).reshape(a.shape)


def bf16_fast(values) -> np.ndarray:
    """The same rounding vectorised in numpy (checked against ``bf16`` by the tests)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    out = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    out[nan] = 0x7FC0
    return out


def to_f32(bits) -> np.ndarray:
    return (_u16(bits).astype(np.uint32) << 16).view(np.float32)


def project(x, rows, w, n, k) -> np.ndarray:
    x, w = _u16(x), _u16(w)
    out = np.empty(rows * n, dtype=np.uint16)
    lib().orc_gm_project(_p(x), rows, _p(w), n, k, _p(out))
    return out


def rms_norm(x, rows, width, eps, scale=None) -> np.ndarray:
    x = _u16(x)
    s = None if scale is None else _u16(scale)
    out = np.empty(rows * width, dtype=np.uint16)
    lib().orc_gm_rms_norm(_p(x), rows, width, eps, _p(s), _p(out))
    return out


def inverse_frequency(head_dim, theta, proportional, pair) -> float:
    return float(lib().orc_gm_inverse_frequency(head_dim, theta, int(proportional), pair))


def factors(head_dim, theta, proportional, positions):
    pos = np.ascontiguousarray(positions, dtype=np.uint32)
    cos = np.empty(pos.size * head_dim, dtype=np.uint16)
    sin = np.empty_like(cos)
    lib().orc_gm_factors(head_dim, theta, int(proportional), _p(pos), pos.size, _p(cos), _p(sin))
    return cos, sin


def apply_rotary(x, rows, heads, width, cos, sin) -> np.ndarray:
    x, cos, sin = _u16(x), _u16(cos), _u16(sin)
    out = np.empty_like(x)
    lib().orc_gm_apply_rotary(_p(x), rows, heads, width, _p(cos), _p(sin), _p(out))
    return out


def attention(q, keys, values, heads, kv_heads, width, window, query_start, key_start) -> np.ndarray:
    q, keys, values = _u16(q), _u16(keys), _u16(values)
    seq, kv_seq = q.size // (heads * width), keys.size // (kv_heads * width)
    out = np.empty_like(q)
    rc = lib().orc_gm_attention(_p(q), seq, _p(keys), _p(values), kv_seq, heads, kv_heads, width, window or 0,
                                query_start, key_start, _p(out))
    if rc != 0:
        raise ValueError("invalid attention span")
    return out


def _binary(name, a, b):
    a, b = _u16(a), _u16(b)
    out = np.empty_like(a)
    getattr(lib(), name)(_p(a), _p(b), a.size, _p(out))
    return out


def add(a, b): return _binary("orc_gm_add", a, b)
def multiply(a, b): return _binary("orc_gm_multiply", a, b)
def ple_combine(a, b): return _binary("orc_gm_ple_combine", a, b)


def scale(a, factor) -> np.ndarray:
    a = _u16(a); out = np.empty_like(a)
    lib().orc_gm_scale(_p(a), factor, a.size, _p(out))
    return out


def gelu_tanh(a) -> np.ndarray:
    a = _u16(a); out = np.empty_like(a)
    lib().orc_gm_gelu_tanh(_p(a), a.size, _p(out))
    return out


def softcap(a, cap) -> np.ndarray:
    a = _u16(a); out = np.empty_like(a)
    lib().orc_gm_softcap(_p(a), cap, a.size, _p(out))
    return out


def argmax(logits) -> int:
    a = _u16(logits)
    return int(lib().orc_gm_argmax(_p(a), a.size))


class GemmaOracle:
    """The reference's host decoder restated: one model, any number of independent sequences."""

    def __init__(self, cfg: dict, tensors: dict):
        self.cfg = cfg
        self._c = make_config(cfg)
        self._h = lib().orc_gemma_create(C.byref(self._c))
        if not self._h:
            raise ValueError("oracle rejected the Gemma configuration")
        for name, data in tensors.items():
            a = _u16(data).reshape(-1)
            if lib().orc_gemma_set_tensor(self._h, name.encode(), _p(a), a.size) != 0:
                raise ValueError(f"oracle rejected tensor {name} ({a.size} elements)")
        if not lib().orc_gemma_ready(self._h):
            raise ValueError("oracle is missing tensors")

    def new_sequence(self):
        return GemmaOracleSeq(self)

    def close(self):
        if self._h:
            lib().orc_gemma_destroy(self._h)
            self._h = None


class GemmaOracleSeq:
    def __init__(self, model: GemmaOracle):
        self.model = model
        self._h = lib().orc_gemma_seq_create(model._h)
        if not self._h:
            raise ValueError("oracle model is incomplete")

    @property
    def position(self) -> int:
        return lib().orc_gemma_seq_position(self._h)

    def _step(self, tokens, want_logits):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty(self.model.cfg["vocab"], dtype=np.uint16) if want_logits else None
        if lib().orc_gemma_step(self._h, _p(t), t.size, _p(logits), None) != 0:
            raise ValueError("empty, overlong or out-of-range token chunk")
        return logits

    def advance_prefill(self, tokens):
        self._step(tokens, False)

    def prefill(self, tokens) -> np.ndarray:
        return self._step(tokens, True)

    def decode(self, token: int) -> np.ndarray:
        return self._step([token], True)

    def close(self):
        if self._h:
            lib().orc_gemma_seq_destroy(self._h)
            self._h = None
