"""Single operators through the C ABI (host arrays in, host arrays out).
Mirrors the operator wrappers of the reference's ``CudaQuantizedGemv`` /
``CudaQwen35Ops`` (crates/nvidia/src/quantized.rs, crates/nvidia/src/model_ops.rs)
so per-primitive parity tests read like the reference's device tests."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import OK, lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _check(rc: int, what: str):
    if rc != OK:
        buf = C.create_string_buffer(1024)
        lib().ribn_b200_op_last_error(buf, len(buf))
        why = buf.value.decode(errors="replace") or "is a B200 visible? there is no CPU path"
        raise RuntimeError(f"ribn_b200 {what} failed: {why}")


def dequantize(ggml_type: int, encoded, rows: int, cols: int, device: int = 0) -> np.ndarray:
    enc = np.ascontiguousarray(np.frombuffer(bytes(encoded), dtype=np.uint8) if not isinstance(encoded, np.ndarray)
                               else encoded.view(np.uint8).reshape(-1))
    out = np.empty((rows, cols), dtype=np.float32)
    _check(lib().ribn_b200_op_dequantize(device, ggml_type, _p(enc), rows, cols, _p(out)), "dequantize")
    return out


def unpack(ggml_type: int, packed, rows: int, cols: int, device: int = 0) -> np.ndarray:
    """Decode FROM the tile-major packed form (output of :func:`repack`) on the device."""
    pk = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
    out = np.empty((rows, cols), dtype=np.float32)
    _check(lib().ribn_b200_debug_unpack(device, ggml_type, _p(pk), rows, cols, _p(out)), "unpack")
    return out


def embedding(ggml_type: int, table, vocab: int, hidden: int, tokens, device: int = 0) -> np.ndarray:
    t = np.ascontiguousarray(table).view(np.uint8).reshape(-1)
    ids = np.ascontiguousarray(tokens, dtype=np.uint32)
    out = np.empty((ids.size, hidden), dtype=np.float32)
    _check(lib().ribn_b200_op_embedding(device, ggml_type, _p(t), vocab, hidden, _p(ids), ids.size, _p(out)), "embedding")
    return out


def qk_norm_rope_append(q, k, v, q_norm, k_norm, positions, kv_slots, q_heads: int, kv_heads: int, head_dim: int,
                        rope_base: float, eps: float, cache_k, cache_v, device: int = 0):
    """Returns (q, k, cache_k, cache_v) after per-head RMSNorm, NeoX rotary and the F16 cache append."""
    q = np.ascontiguousarray(q, dtype=np.float32).copy()
    k = np.ascontiguousarray(k, dtype=np.float32).copy()
    v = np.ascontiguousarray(v, dtype=np.float32)
    qn = np.ascontiguousarray(q_norm, dtype=np.float32)
    kn = np.ascontiguousarray(k_norm, dtype=np.float32)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    slots = np.ascontiguousarray(kv_slots, dtype=np.int32)
    ck = np.ascontiguousarray(cache_k, dtype=np.uint16).copy()
    cv = np.ascontiguousarray(cache_v, dtype=np.uint16).copy()
    physical = ck.size // (kv_heads * head_dim)
    _check(lib().ribn_b200_op_qk_norm_rope_append(device, _p(q), _p(k), _p(v), _p(qn), _p(kn), _p(pos), _p(slots),
                                                  pos.size, q_heads, kv_heads, head_dim, rope_base, eps, _p(ck), _p(cv),
                                                  physical), "qk_norm_rope_append")
    return q, k, ck, cv


def attention_decode(q, k, v, q_norm, k_norm, rope_base: float, eps: float, cache_k, cache_v, page_tables, positions,
                     q_heads: int, kv_heads: int, head_dim: int, device: int = 0):
    """The decode step's fused norm + rotary + append + attention, one new token per sequence.
    Returns (out [members][q_heads * head_dim], cache_k, cache_v)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    qn = np.ascontiguousarray(q_norm, dtype=np.float32)
    kn = np.ascontiguousarray(k_norm, dtype=np.float32)
    ck = np.ascontiguousarray(cache_k, dtype=np.uint16).copy()
    cv = np.ascontiguousarray(cache_v, dtype=np.uint16).copy()
    tables = np.ascontiguousarray(page_tables, dtype=np.int32)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    members = pos.size
    physical = ck.size // (kv_heads * head_dim)
    out = np.empty((members, q_heads * head_dim), dtype=np.float32)
    _check(lib().ribn_b200_op_attention_decode(device, _p(q), _p(k), _p(v), _p(qn), _p(kn), rope_base, eps, _p(ck), _p(cv),
                                               physical, _p(tables), tables.shape[1], _p(pos), members, q_heads, kv_heads,
                                               head_dim, _p(out)), "attention_decode")
    return out, ck, cv


def gemv(ggml_type: int, weights, rows: int, cols: int, x, variant: int = 0, device: int = 0) -> np.ndarray:
    w = np.ascontiguousarray(weights).view(np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    members = 1 if x.ndim == 1 else x.shape[0]
    y = np.empty((members, rows), dtype=np.float32)
    _check(lib().ribn_b200_op_gemv(device, ggml_type, _p(w), rows, cols, _p(x), members, _p(y), variant), "gemv")
    return y[0] if x.ndim == 1 else y


def rms_norm(x, weight, eps: float, device: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    members = 1 if x.ndim == 1 else x.shape[0]
    out = np.empty_like(x)
    _check(lib().ribn_b200_op_rms_norm(device, _p(x), _p(w), members, x.shape[-1], eps, _p(out)), "rms_norm")
    return out


def silu_mul(gate, up, device: int = 0) -> np.ndarray:
    g = np.ascontiguousarray(gate, dtype=np.float32)
    u = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(g)
    _check(lib().ribn_b200_op_silu_mul(device, _p(g), _p(u), g.size, _p(out)), "silu_mul")
    return out


def gdn_step(qkv, z, beta_raw, alpha_raw, dt_bias, a, conv_weight, norm_weight, conv_state, state, k_heads: int,
             v_heads: int, head_dim: int, l2_eps: float, norm_eps: float, tokens: int = 1, device: int = 0):
    """Gated-DeltaNet decode steps behind the projections for `members` sequences of `tokens` consecutive tokens each
    (ribn_b200_op_gdn_step; rows are member-major).  Returns a dict: out, decay, beta, conv_act, attn_out (one row
    per token), and the advanced conv_state and state (one per member)."""
    channels, inner = (2 * k_heads + v_heads) * head_dim, v_heads * head_dim
    x = np.ascontiguousarray(qkv, dtype=np.float32).reshape(-1, channels)
    rows = x.shape[0]
    members = rows // tokens
    if members * tokens != rows:
        raise ValueError("rows must be members * tokens")
    f = lambda v, shape: np.ascontiguousarray(v, dtype=np.float32).reshape(shape)
    zz, br, ar = f(z, (rows, inner)), f(beta_raw, (rows, v_heads)), f(alpha_raw, (rows, v_heads))
    dt, aa, cw, nw = f(dt_bias, (v_heads,)), f(a, (v_heads,)), f(conv_weight, (channels, 4)), f(norm_weight, (head_dim,))
    conv = f(conv_state, (members, channels, 3)).copy()
    st = f(state, (members, v_heads, head_dim, head_dim)).copy()
    decay, beta = np.empty((rows, v_heads), np.float32), np.empty((rows, v_heads), np.float32)
    act, attn, out = np.empty((rows, channels), np.float32), np.empty((rows, inner), np.float32), np.empty((rows, inner), np.float32)
    _check(lib().ribn_b200_op_gdn_step(device, members, tokens, k_heads, v_heads, head_dim, _p(x), _p(zz), _p(br), _p(ar), _p(dt),
                                       _p(aa), _p(cw), _p(nw), _p(conv), _p(st), l2_eps, norm_eps, _p(decay), _p(beta), _p(act),
                                       _p(attn), _p(out)), "gdn_step")
    return dict(out=out, decay=decay, beta=beta, conv_act=act, attn_out=attn, conv_state=conv, state=st)


def attention_gate(attn, q_gate, heads: int, head_dim: int, device: int = 0) -> np.ndarray:
    """out = attn * sigmoid(gate half of the [q | gate] projection) (ribn_b200_op_attention_gate)."""
    at = np.ascontiguousarray(attn, dtype=np.float32).reshape(-1, heads * head_dim)
    qg = np.ascontiguousarray(q_gate, dtype=np.float32).reshape(at.shape[0], heads * 2 * head_dim)
    out = np.empty_like(at)
    _check(lib().ribn_b200_op_attention_gate(device, _p(at), _p(qg), at.shape[0], heads, head_dim, _p(out)), "attention_gate")
    return out


def argmax(logits, device: int = 0):
    l = np.ascontiguousarray(logits, dtype=np.float32)
    members = 1 if l.ndim == 1 else l.shape[0]
    out = np.empty(members, dtype=np.uint32)
    _check(lib().ribn_b200_op_argmax(device, _p(l), members, l.shape[-1], _p(out)), "argmax")
    return int(out[0]) if l.ndim == 1 else out


def rope_neox(values, positions, heads: int, head_dim: int, rot_dims: int, base: float, device: int = 0) -> np.ndarray:
    v = np.ascontiguousarray(values, dtype=np.float32).copy()
    pos = np.ascontiguousarray(np.atleast_1d(positions), dtype=np.int64)
    _check(lib().ribn_b200_op_rope_neox(device, _p(v), _p(pos), pos.size, heads, head_dim, rot_dims, base), "rope")
    return v


def f32_to_f16_bits(values, device: int = 0) -> np.ndarray:
    v = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(v.shape, dtype=np.uint16)
    _check(lib().ribn_b200_op_f32_to_f16(device, _p(v), v.size, _p(out)), "f32_to_f16")
    return out


def attention(q, keys_f16, values_f16, page_table, tokens: int, rows: int, q_heads: int, kv_heads: int,
              head_dim: int, window: int = 0, variant: int = 0, device: int = 0) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(keys_f16, dtype=np.uint16)
    v = np.ascontiguousarray(values_f16, dtype=np.uint16)
    table = np.ascontiguousarray(page_table, dtype=np.int32)
    physical = k.size // (kv_heads * head_dim)
    out = np.empty((rows, q_heads * head_dim), dtype=np.float32)
    _check(lib().ribn_b200_op_attention(device, _p(q), _p(k), _p(v), _p(table), 16, physical, tokens, rows, q_heads,
                                        kv_heads, head_dim, window, _p(out), variant), "attention")
    return out


def batch_metadata(row_slot, row_prefix, row_tokens, page_tables, page_tokens: int = 16, device: int = 0):
    slot = np.ascontiguousarray(row_slot, dtype=np.int32)
    prefix = np.ascontiguousarray(row_prefix, dtype=np.int32)
    tokens = np.ascontiguousarray(row_tokens, dtype=np.int32)
    tables = np.ascontiguousarray(page_tables, dtype=np.int32)
    total = int(tokens.sum())
    cu = np.empty(slot.size + 1, dtype=np.int32)
    row = np.empty(total, dtype=np.int32)
    pos = np.empty(total, dtype=np.int32)
    kv = np.empty(total, dtype=np.int32)
    _check(lib().ribn_b200_op_batch_metadata(device, _p(slot), _p(prefix), _p(tokens), slot.size, _p(tables),
                                             tables.shape[1], page_tokens, _p(cu), _p(row), _p(pos), _p(kv)),
           "batch_metadata")
    return cu, row, pos, kv


def repack(ggml_type: int, raw, rows: int, cols: int) -> np.ndarray:
    """Host-side tile-major repack (no device needed)."""
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    need = C.c_size_t(0)
    _check(lib().ribn_b200_debug_repack(ggml_type, _p(raw), rows, cols, None, 0, C.byref(need)), "repack size")
    out = np.empty(need.value, dtype=np.uint8)
    _check(lib().ribn_b200_debug_repack(ggml_type, _p(raw), rows, cols, _p(out), out.size, C.byref(need)), "repack")
    return out
