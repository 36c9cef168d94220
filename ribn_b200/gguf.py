"""GGUF container reader (and a small writer for tests) and the dense-Qwen3 load path.

The reference reads the container in ``crates/gguf/src/lib.rs:183-300`` (magic, version 3, metadata
key/values, tensor directory, data aligned to ``general.alignment``) and stages the encoded tensor
bytes verbatim (``crates/nvidia/src/staging.rs:263-315``); its model config comes from
``<arch>.*`` metadata keys (``crates/qwen/src/gguf/config.rs:17-32``).  This module restates the
public container layout and maps a ``general.architecture = "qwen3"`` file onto the executor:
every tensor goes through ``QwenB200.load_tensor`` under its GGUF name, untouched.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

MAGIC = 0x46554747  # "GGUF", little endian
VERSION = 3
DEFAULT_ALIGNMENT = 32

# metadata value types of the container
U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q",
           F64: "<d"}

# ggml tensor types the executor stores: (elements per block, bytes per block)
BLOCKS = {0: (1, 4), 1: (1, 2), 8: (32, 34), 12: (256, 144), 14: (256, 210)}


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    dims: Tuple[int, ...]     # innermost first, as stored: (cols, rows) for a matrix
    ggml_type: int
    offset: int               # relative to the start of the aligned data section

    @property
    def rows(self) -> int:
        n = 1
        for d in self.dims[1:]:
            n *= d
        return n

    @property
    def cols(self) -> int:
        return self.dims[0]

    def byte_count(self) -> int:
        if self.ggml_type not in BLOCKS:
            raise GgufError(f"tensor {self.name!r} has ggml type {self.ggml_type}, which this executor does not store")
        elems, size = BLOCKS[self.ggml_type]
        if self.cols % elems:
            raise GgufError(f"tensor {self.name!r}: {self.cols} columns are not whole blocks of {elems}")
        return self.rows * (self.cols // elems) * size


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("truncated GGUF value")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if n > (1 << 24) or self.pos + n > len(self.buf):
            raise GgufError("GGUF string length exceeds the parser bound")
        s = bytes(self.buf[self.pos:self.pos + n])
        self.pos += n
        try:
            return s.decode("utf-8")
        except UnicodeDecodeError as e:
            raise GgufError("GGUF string is not valid UTF-8") from e

    def value(self, kind: int, depth: int = 0):
        if kind in _SCALAR:
            v = self.take(_SCALAR[kind])
            if kind == BOOL:
                if v not in (0, 1):
                    raise GgufError(f"invalid GGUF boolean value {v}")
                return bool(v)
            return v
        if kind == STRING:
            return self.string()
        if kind == ARRAY:
            if depth >= 2:
                raise GgufError("GGUF metadata array nesting is too deep")
            inner, count = self.take("<I"), self.take("<Q")
            if count > (1 << 26):
                raise GgufError("GGUF array length exceeds the parser bound")
            if inner in _SCALAR and inner != BOOL:
                fmt = _SCALAR[inner]
                size = struct.calcsize(fmt) * count
                if self.pos + size > len(self.buf):
                    raise GgufError("truncated GGUF value")
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=count, offset=self.pos).copy()
                self.pos += size
                return arr
            return [self.value(inner, depth + 1) for _ in range(count)]
        raise GgufError(f"invalid GGUF metadata value type {kind}")


class GgufFile:
    """Parsed header of one GGUF file; tensor bytes are served from a read-only memory map."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        r = _Reader(self._map)
        magic = r.take("<I")
        if magic != MAGIC:
            raise GgufError(f"invalid GGUF magic 0x{magic:08x}")
        version = r.take("<I")
        if version != VERSION:
            raise GgufError(f"unsupported GGUF version {version}")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        if n_tensors > (1 << 20) or n_kv > (1 << 20):
            raise GgufError("GGUF counts exceed the parser bound")
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = r.string()
            if key in self.metadata:
                raise GgufError(f"duplicate GGUF metadata key {key!r}")
            self.metadata[key] = r.value(r.take("<I"))
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = r.string()
            n_dims = r.take("<I")
            if not 1 <= n_dims <= 4:
                raise GgufError(f"invalid GGUF tensor dimension count {n_dims}")
            dims = tuple(r.take("<Q") for _ in range(n_dims))
            self.tensors[name] = TensorInfo(name, dims, r.take("<I"), r.take("<Q"))
        alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        if alignment <= 0 or alignment & (alignment - 1):
            raise GgufError(f"invalid GGUF tensor-data alignment {alignment}")
        self.data_offset = (r.pos + alignment - 1) // alignment * alignment
        for t in self.tensors.values():
            if t.ggml_type in BLOCKS and self.data_offset + t.offset + t.byte_count() > len(self._map):
                raise GgufError(f"GGUF tensor {t.name!r} has out-of-bounds offset {t.offset}")

    def tensor_bytes(self, name: str) -> np.ndarray:
        t = self.tensors.get(name)
        if t is None:
            raise GgufError(f"GGUF tensor {name!r} was not found")
        return np.frombuffer(self._map, dtype=np.uint8, count=t.byte_count(), offset=self.data_offset + t.offset)

    def require(self, key: str):
        if key not in self.metadata:
            raise GgufError(f"missing GGUF metadata key {key!r}")
        return self.metadata[key]

    def close(self):
        # numpy views of the map may still be alive; dropping the references is enough
        self._map = None
        self._f.close()


def qwen3_config(f: GgufFile) -> dict:
    """Model dimensions of a dense-Qwen3 file, in the executor's config vocabulary."""
    arch = f.require("general.architecture")
    if arch != "qwen3":
        raise GgufError(f"unsupported GGUF architecture {arch!r}")
    hidden = int(f.require("qwen3.embedding_length"))
    q_heads = int(f.require("qwen3.attention.head_count"))
    head_dim = int(f.metadata.get("qwen3.attention.key_length", hidden // q_heads))
    embd = f.tensors.get("token_embd.weight")
    if embd is None:
        raise GgufError("GGUF tensor 'token_embd.weight' was not found")
    return dict(layers=int(f.require("qwen3.block_count")), hidden=hidden, q_heads=q_heads,
                kv_heads=int(f.require("qwen3.attention.head_count_kv")), head_dim=head_dim,
                ffn=int(f.require("qwen3.feed_forward_length")), vocab=embd.rows,
                rope_base=float(f.metadata.get("qwen3.rope.freq_base", 10000.0)),
                rms_eps=float(f.require("qwen3.attention.layer_norm_rms_epsilon")))


def load_qwen3(path: str, **executor_options):
    """Open `path`, build a `QwenB200` for it and upload every tensor's encoded bytes as they are.
    A file without `output.weight` ties the head to the embedding table."""
    from .executor import QwenB200
    f = GgufFile(path)
    try:
        cfg = qwen3_config(f)
        ex = QwenB200(cfg, **executor_options)
        try:
            for name, t in f.tensors.items():
                if name.startswith("blk.") or name in ("token_embd.weight", "output_norm.weight", "output.weight"):
                    ex.load_tensor(name, t.ggml_type, t.rows, t.cols, f.tensor_bytes(name))
            if "output.weight" not in f.tensors:
                t = f.tensors["token_embd.weight"]
                ex.load_tensor("output.weight", t.ggml_type, t.rows, t.cols, f.tensor_bytes("token_embd.weight"))
            ex.finalize()
        except Exception:
            ex.close()
            raise
        return ex, cfg
    finally:
        f.close()


# ---- writer (tests and synthetic checkpoints) -----------------------------------------------
def _pack_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I", BOOL) + struct.pack("<B", int(v))
    if isinstance(v, str):
        return struct.pack("<I", STRING) + _pack_string(v)
    if isinstance(v, float):
        return struct.pack("<I", F32) + struct.pack("<f", v)
    if isinstance(v, int):
        return struct.pack("<I", U32) + struct.pack("<I", v) if 0 <= v < (1 << 32) else struct.pack("<I", I64) + struct.pack("<q", v)
    if isinstance(v, (list, tuple)) and all(isinstance(x, str) for x in v):
        return struct.pack("<I", ARRAY) + struct.pack("<I", STRING) + struct.pack("<Q", len(v)) + b"".join(_pack_string(x) for x in v)
    raise TypeError(f"cannot encode GGUF metadata value {v!r}")


def write_gguf(path: str, metadata: Dict[str, object], tensors: Dict[str, Tuple[int, int, int, np.ndarray]],
               alignment: int = DEFAULT_ALIGNMENT) -> None:
    """tensors: name -> (ggml type, rows, cols, encoded bytes); norms are written as 1-D tensors."""
    names: List[str] = list(tensors)
    head = struct.pack("<IIQQ", MAGIC, VERSION, len(names), len(metadata))
    for k, v in metadata.items():
        head += _pack_string(k) + _pack_value(v)
    blobs, offset, infos = [], 0, b""
    for name in names:
        kind, rows, cols, data = tensors[name]
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        dims = (cols,) if rows == 1 else (cols, rows)
        infos += _pack_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", kind, offset)
        pad = (-raw.size) % alignment
        blobs.append(raw.tobytes() + b"\0" * pad)
        offset += raw.size + pad
    head += infos
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)
