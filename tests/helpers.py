"""Test-only helpers: the reference's fixture-block definitions restated,
an independent numpy decoder for cross-checking the C oracle, numpy
quantisers for building small valid checkpoints, and tiny model builders."""
from __future__ import annotations

import numpy as np

F32, F16, Q8_0, Q4_K, Q6_K = 0, 1, 8, 12, 14
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210), F32: (1, 4), F16: (1, 2)}


# --- fixture blocks: crates/nvidia/tests/cuda_reference.rs:251-273, 327-364 ---------------
def q4_k_fixture_block(seed: int) -> np.ndarray:
    b = np.zeros(144, dtype=np.uint8)
    b[0:2] = np.frombuffer(np.uint16(0x3C00).tobytes(), dtype=np.uint8)
    b[2:4] = np.frombuffer(np.uint16(0x3800).tobytes(), dtype=np.uint8)
    for i in range(4):
        b[4 + i] = ((1 + seed + i) | ((i & 3) << 6)) & 0xFF
        b[8 + i] = ((1 + i) | (((i + 1) & 3) << 6)) & 0xFF
        b[12 + i] = ((5 + seed + i) | ((2 + i) << 4)) & 0xFF
    for i in range(128):
        pattern = (i + seed * 5) % 16
        low = (pattern * 3) & 0x0F
        high = (15 - pattern * 3) & 0x0F
        b[16 + i] = low | (high << 4)
    return b


def q6_k_fixture_block(seed: int) -> np.ndarray:
    b = np.zeros(210, dtype=np.uint8)
    for i in range(128):
        b[i] = (i * 7 + seed * 11) % 256
    for i in range(64):
        b[128 + i] = (i * 13 + seed * 5) % 256
    for i in range(16):
        b[192 + i] = np.int8(((i + seed * 3) % 17) - 8).view(np.uint8)
    b[208:210] = np.frombuffer(np.uint16(0x3C00).tobytes(), dtype=np.uint8)
    return b


def q8_0_fixture_block(seed: int) -> np.ndarray:
    b = np.zeros(34, dtype=np.uint8)
    b[0:2] = np.frombuffer(np.uint16(0x3C00).tobytes(), dtype=np.uint8)
    for i in range(32):
        b[2 + i] = np.int8(((i + seed * 3) % 31) - 15).view(np.uint8)
    return b


def fixture(kind: int) -> np.ndarray:
    if kind == Q4_K:
        return np.concatenate([q4_k_fixture_block(s) for s in range(4)])
    if kind == Q6_K:
        return np.concatenate([q6_k_fixture_block(s) for s in range(4)])
    return np.concatenate([q8_0_fixture_block(s) for s in range(6)])


def fixture_input(n: int, member: int = 0) -> np.ndarray:
    """x[i] = ((i + 7 m) % 17) * 0.125 - 1 (cuda_reference.rs:709-714, 5172-5278)."""
    i = np.arange(n)
    return (((i + 7 * member) % 17).astype(np.float32) * np.float32(0.125) - np.float32(1.0)).astype(np.float32)


def lcg_f16_values(state: int, count: int):
    """fixture_quantized_f32: 0.125 steps in [-4, 4), exact in F16 (cuda_reference.rs:1603-1610)."""
    out = np.empty(count, dtype=np.float32)
    for i in range(count):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(((state >> 16) & 0x3F)) * np.float32(0.125) - np.float32(4.0)
    return out, state


# --- independent numpy decoder --------------------------------------------------------------
def _f16(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def np_dequant(kind: int, data: np.ndarray) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    elems, size = BLOCK[kind]
    blocks = data.reshape(-1, size)
    n = blocks.shape[0]
    if kind == Q8_0:
        d = _f16(blocks[:, 0:2].copy()).reshape(n, 1)
        return (d * blocks[:, 2:].view(np.int8).astype(np.float32)).astype(np.float32).reshape(-1)
    if kind == Q4_K:
        d = _f16(blocks[:, 0:2].copy()).reshape(n, 1)
        dmin = _f16(blocks[:, 2:4].copy()).reshape(n, 1)
        p = blocks[:, 4:16].astype(np.uint8)
        sc = np.zeros((n, 8), dtype=np.uint8)
        mn = np.zeros((n, 8), dtype=np.uint8)
        sc[:, :4] = p[:, 0:4] & 0x3F
        sc[:, 4:] = (p[:, 8:12] & 0x0F) | ((p[:, 0:4] >> 2) & 0x30)
        mn[:, :4] = p[:, 4:8] & 0x3F
        mn[:, 4:] = (p[:, 8:12] >> 4) | ((p[:, 4:8] >> 2) & 0x30)
        qs = blocks[:, 16:].reshape(n, 4, 32)
        q = np.empty((n, 8, 32), dtype=np.float32)
        q[:, 0::2] = (qs & 0x0F).astype(np.float32)
        q[:, 1::2] = (qs >> 4).astype(np.float32)
        gs = (d * sc.astype(np.float32)).astype(np.float32)[:, :, None]
        gm = (dmin * mn.astype(np.float32)).astype(np.float32)[:, :, None]
        return ((gs * q).astype(np.float32) - gm).astype(np.float32).reshape(-1)
    if kind == Q6_K:
        ql = blocks[:, :128].reshape(n, 2, 2, 32)      # [chunk][variant & 1][l]
        qh = blocks[:, 128:192].reshape(n, 2, 32)      # [chunk][l]
        sc = blocks[:, 192:208].view(np.int8).astype(np.float32).reshape(n, 8, 2)
        d = _f16(blocks[:, 208:210].copy()).reshape(n, 1, 1)
        q = np.empty((n, 2, 4, 32), dtype=np.int32)
        for v in range(4):
            low = (ql[:, :, v & 1, :] >> (0 if v < 2 else 4)) & 0x0F
            high = (qh >> (2 * v)) & 0x03
            q[:, :, v, :] = (low | (high << 4)).astype(np.int32) - 32
        q = q.reshape(n, 8, 2, 16).astype(np.float32)
        gs = (d * sc).astype(np.float32)[:, :, :, None]
        return (gs * q).astype(np.float32).reshape(-1)
    if kind == F32:
        return data.view(np.float32).copy()
    if kind == F16:
        return _f16(data)
    raise ValueError(kind)


# --- numpy quantisers (test checkpoints only) ------------------------------------------------
def quantize(kind: int, values: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    if kind == F32:
        return v.view(np.uint8).copy()
    if kind == Q8_0:
        x = v.reshape(-1, 32)
        d = (np.abs(x).max(axis=1) / 127.0).astype(np.float16)
        df = d.astype(np.float32)
        inv = np.where(df > 0, 1.0 / np.maximum(df, 1e-30), 0.0)
        q = np.clip(np.rint(x * inv[:, None]), -127, 127).astype(np.int8)
        out = np.zeros((x.shape[0], 34), dtype=np.uint8)
        out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        out[:, 2:] = q.view(np.uint8)
        return out.reshape(-1)
    if kind == Q4_K:
        x = v.reshape(-1, 8, 32)
        n = x.shape[0]
        lo = np.minimum(x.min(axis=2), 0.0)
        hi = np.maximum(x.max(axis=2), 0.0)
        scale = (hi - lo) / 15.0
        minimum = -lo
        d = (scale.max(axis=1) / 63.0).astype(np.float16)
        dmin = (minimum.max(axis=1) / 63.0).astype(np.float16)
        df, dmf = d.astype(np.float32)[:, None], dmin.astype(np.float32)[:, None]
        sc = np.where(df > 0, np.clip(np.rint(scale / np.maximum(df, 1e-30)), 0, 63), 0).astype(np.uint8)
        mn = np.where(dmf > 0, np.clip(np.rint(minimum / np.maximum(dmf, 1e-30)), 0, 63), 0).astype(np.uint8)
        gs = df * sc
        gm = dmf * mn
        inv = np.where(gs > 0, 1.0 / np.maximum(gs, 1e-30), 0.0)
        q = np.clip(np.rint((x + gm[:, :, None]) * inv[:, :, None]), 0, 15).astype(np.uint8)
        out = np.zeros((n, 144), dtype=np.uint8)
        out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
        out[:, 4:8] = sc[:, :4] | ((sc[:, 4:] >> 4) << 6)
        out[:, 8:12] = mn[:, :4] | ((mn[:, 4:] >> 4) << 6)
        out[:, 12:16] = (sc[:, 4:] & 0x0F) | ((mn[:, 4:] & 0x0F) << 4)
        out[:, 16:] = (q[:, 0::2] | (q[:, 1::2] << 4)).reshape(n, 128)
        return out.reshape(-1)
    if kind == Q6_K:
        x = v.reshape(-1, 16, 16)
        n = x.shape[0]
        scale = np.abs(x).max(axis=2) / 31.0
        d = (scale.max(axis=1) / 127.0).astype(np.float16)
        df = d.astype(np.float32)[:, None]
        sc = np.where(df > 0, np.clip(np.rint(scale / np.maximum(df, 1e-30)), 1, 127), 0).astype(np.int8)
        gs = df * sc.astype(np.float32)
        inv = np.where(gs > 0, 1.0 / np.maximum(gs, 1e-30), 0.0)
        q = (np.clip(np.rint(x * inv[:, :, None]), -32, 31) + 32).astype(np.uint8).reshape(n, 2, 4, 32)
        out = np.zeros((n, 210), dtype=np.uint8)
        ql = np.zeros((n, 2, 2, 32), dtype=np.uint8)
        qh = np.zeros((n, 2, 32), dtype=np.uint8)
        for var in range(4):
            ql[:, :, var & 1, :] |= (q[:, :, var, :] & 0x0F) << (0 if var < 2 else 4)
            qh |= (q[:, :, var, :] >> 4) << (2 * var)
        out[:, :128] = ql.reshape(n, 128)
        out[:, 128:192] = qh.reshape(n, 64)
        out[:, 192:208] = sc.view(np.uint8)
        out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
        return out.reshape(-1)
    raise ValueError(kind)


TINY = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=512,
            rope_base=1.0e6, rms_eps=1.0e-6)


def make_model(cfg: dict, seed: int, scheme: str = "q4_k_m", norm_jitter: bool = True) -> dict:
    """name -> (type, rows, cols, encoded bytes) for a dense Qwen3-shaped checkpoint."""
    rng = np.random.default_rng(seed)
    base, wide = (Q8_0, Q8_0) if scheme == "q8_0" else (Q4_K, Q6_K)
    H, QD, KD, F, V = (cfg["hidden"], cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"],
                       cfg["ffn"], cfg["vocab"])
    t = {}

    def mat(name, kind, rows, cols, std=0.02):
        t[name] = (kind, rows, cols, quantize(kind, rng.normal(0.0, std, size=(rows, cols)).astype(np.float32)))

    def norm(name, n):
        w = np.ones(n, dtype=np.float32)
        if norm_jitter:
            w = (w + rng.normal(0.0, 0.1, size=n)).astype(np.float32)
        t[name] = (F32, 1, n, w.view(np.uint8).copy())

    for l in range(cfg["layers"]):
        p = f"blk.{l}."
        norm(p + "attn_norm.weight", H)
        mat(p + "attn_q.weight", base, QD, H)
        mat(p + "attn_k.weight", base, KD, H)
        mat(p + "attn_v.weight", wide, KD, H)
        norm(p + "attn_q_norm.weight", cfg["head_dim"])
        norm(p + "attn_k_norm.weight", cfg["head_dim"])
        mat(p + "attn_output.weight", base, H, QD)
        norm(p + "ffn_norm.weight", H)
        mat(p + "ffn_gate.weight", base, F, H)
        mat(p + "ffn_up.weight", base, F, H)
        mat(p + "ffn_down.weight", wide, H, F)
    mat("token_embd.weight", base, V, H)
    norm("output_norm.weight", H)
    mat("output.weight", wide, V, H)
    return t


def oracle_config(cfg: dict, context: int) -> dict:
    return dict(layers=cfg["layers"], hidden=cfg["hidden"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], context=context,
                rope_base=cfg["rope_base"], eps=cfg["rms_eps"])
