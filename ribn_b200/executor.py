"""Host-side mirror of ribn's ``GenerationExecutor`` for the B200 executor.

Names, argument meaning and error behaviour follow the reference trait
(crates/runtime/src/executor.rs:171-254) and its Qwen implementation
(crates/qwen/src/cuda.rs:70-109, crates/qwen/src/execution.rs): ``admit`` returns
an :class:`Admission`, ``prepare``/``submit``/``poll`` raise
:class:`ExecutionError` where the reference returns ``Err`` (which faults the
engine), ``poll`` returns ``None`` while the device is busy.
Everything is a thin ctypes call into ``libribn_b200.so``."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import BatchItemC, CompletionC, Config, Limits, PreparedRowC, SamplingC, lib


class ExecutionError(RuntimeError):
    """Bounded diagnostic (<= 4096 bytes), crates/runtime/src/executor.rs:134-152."""


class StepKind(enum.IntEnum):
    PREFILL = _lib.PREFILL
    DECODE = _lib.DECODE


@dataclass(frozen=True)
class BatchItem:
    sequence: int
    kind: StepKind
    prefix: int
    token_budget: int
    output_budget: int


@dataclass(frozen=True)
class Sampling:
    """TokenRequest.options.sampling (temperature 0 = greedy; anything else is rejected, as in the
    reference: crates/qwen/src/execution.rs:107-111)."""
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = 0


@dataclass(frozen=True)
class PreparedRow:
    """PreparedRow::{Ready(item), Deferred, Rejected} (crates/runtime/src/executor.rs:97-105)."""
    state: str                      # "ready" | "deferred" | "rejected"
    item: Optional[BatchItem] = None   # the granted row (budgets may have shrunk) when ready


@dataclass(frozen=True)
class StepCompletion:
    sequence: int
    prefix: int
    tokens: List[int] = field(default_factory=list)


@dataclass(frozen=True)
class GenerationLimits:
    context_tokens: int
    max_sequences: int
    max_batch_tokens: int
    max_decode_tokens: int


@dataclass(frozen=True)
class ExecutorInfo:
    name: str
    limits: GenerationLimits


class Admission:
    """Admission::{Ready, Rejected(err), Deferred} (crates/runtime/src/executor.rs:109-121)."""
    READY = "ready"
    REJECTED = "rejected"
    DEFERRED = "deferred"

    def __init__(self, state: str, reason: str = ""):
        self.state = state
        self.reason = reason

    def __repr__(self):
        return f"Admission.{self.state}({self.reason!r})" if self.reason else f"Admission.{self.state}"

    @property
    def ready(self) -> bool:
        return self.state == Admission.READY


def nccl_library_path() -> str:
    """The libnccl the host process uses: the one bundled with the Python environment when there is one."""
    import importlib.util
    import os
    spec = importlib.util.find_spec("nvidia.nccl")
    if spec is not None and spec.submodule_search_locations:
        for root in spec.submodule_search_locations:
            path = os.path.join(root, "lib", "libnccl.so.2")
            if os.path.exists(path):
                return path
    return "libnccl.so.2"


def tp_unique_id(nccl_library: Optional[str] = None) -> bytes:
    """Rank 0 of a tensor-parallel group: a fresh group id (128 bytes) to hand to the other ranks."""
    nid = _lib.NcclId()
    err = C.create_string_buffer(1024)
    rc = lib().ribn_b200_tp_unique_id((nccl_library or nccl_library_path()).encode(), C.byref(nid), err, len(err))
    if rc != _lib.OK:
        raise ExecutionError(err.value.decode(errors="replace"))
    return bytes(C.string_at(C.byref(nid), 128))


def tp_shard(model: dict, name: str, rows: int, cols: int, tp_size: int, tp_rank: int):
    """(row0, rows, col0, cols) of the part of whole tensor `name` that rank `tp_rank` of `tp_size` keeps."""
    cfg = Config(tp_size=tp_size, tp_rank=tp_rank, **model)
    out = [C.c_int64() for _ in range(4)]
    rc = lib().ribn_b200_tp_shard(C.byref(cfg), name.encode(), rows, cols, *[C.byref(o) for o in out])
    if rc != _lib.OK:
        raise ValueError(f"no tensor-parallel split of {name} for rank {tp_rank} of {tp_size}")
    return tuple(o.value for o in out)


def _items(items: Sequence[BatchItem]):
    arr = (BatchItemC * max(len(items), 1))()
    for i, it in enumerate(items):
        arr[i] = BatchItemC(it.sequence, int(it.kind), it.prefix, it.token_budget, it.output_budget)
    return arr


class QwenB200:
    """Dense-Qwen3 GGUF executor on one B200 (the `QwenCuda` replacement)."""

    def __init__(self, model: dict, *, context_tokens: int = 4096, max_sequences: int = 1,
                 max_batch_tokens: int = 128, kv_pages: int = 0, device: int = 0, flags: int = 0,
                 tp_size: int = 1, tp_rank: int = 0):
        cfg = Config(context_tokens=context_tokens, max_sequences=max_sequences,
                     max_batch_tokens=max_batch_tokens, kv_pages=kv_pages, device=device, flags=flags,
                     tp_size=tp_size, tp_rank=tp_rank, **model)
        self.cfg = cfg
        self._h = C.c_void_p()
        err = C.create_string_buffer(4096)
        rc = lib().ribn_b200_create(C.byref(cfg), C.byref(self._h), err, len(err))
        if rc != _lib.OK:
            self._h = None
            raise ExecutionError(err.value.decode(errors="replace"))
        self._rows = (CompletionC * max(max_sequences, 1))()

    # -- loading ----------------------------------------------------------
    def _err(self) -> str:
        buf = C.create_string_buffer(4097)
        lib().ribn_b200_last_error(self._h, buf, len(buf))
        return buf.value.decode(errors="replace")

    def _check(self, rc: int):
        if rc != _lib.OK:
            raise ExecutionError(self._err())

    def load_tensor(self, name: str, ggml_type: int, rows: int, cols: int, data) -> None:
        arr = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self._check(lib().ribn_b200_load_tensor(self._h, name.encode(), ggml_type, rows, cols,
                                                arr.ctypes.data_as(C.c_void_p), arr.size))

    def init_synthetic(self, seed: int, scheme: int) -> None:
        self._check(lib().ribn_b200_init_synthetic(self._h, seed, scheme))

    def read_tensor(self, name: str):
        t, r, c, n = C.c_int32(), C.c_int64(), C.c_int64(), C.c_size_t()
        self._check(lib().ribn_b200_read_tensor(self._h, name.encode(), C.byref(t), C.byref(r), C.byref(c), None, 0,
                                                C.byref(n)))
        out = np.empty(n.value, dtype=np.uint8)
        self._check(lib().ribn_b200_read_tensor(self._h, name.encode(), None, None, None,
                                                out.ctypes.data_as(C.c_void_p), out.size, None))
        return t.value, r.value, c.value, out

    def tensor_names(self) -> List[str]:
        names = []
        for l in range(self.cfg.layers):
            for n in ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_q_norm", "attn_k_norm", "attn_output",
                      "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"):
                names.append(f"blk.{l}.{n}.weight")
        return names + ["token_embd.weight", "output_norm.weight", "output.weight"]

    def tp_init(self, group_id: bytes, nccl_library: Optional[str] = None) -> None:
        """Join the tensor-parallel group (collective over all its ranks; call after create, before finalize)."""
        nid = _lib.NcclId()
        C.memmove(C.byref(nid), group_id, 128)
        self._check(lib().ribn_b200_tp_init(self._h, (nccl_library or nccl_library_path()).encode(), C.byref(nid)))

    def tp_time_allreduce(self, tokens: int, repeats: int = 50) -> float:
        """Average microseconds of one [tokens, hidden] F32 all-reduce (collective: every rank calls it)."""
        us = C.c_float()
        self._check(lib().ribn_b200_tp_time_allreduce(self._h, tokens, repeats, C.byref(us)))
        return us.value

    def finalize(self) -> None:
        self._check(lib().ribn_b200_finalize(self._h))

    # -- GenerationExecutor -------------------------------------------------
    def info(self) -> ExecutorInfo:
        lim = Limits()
        self._check(lib().ribn_b200_info(self._h, C.byref(lim)))
        return ExecutorInfo("ribn-b200-qwen3", GenerationLimits(lim.context_tokens, lim.max_sequences,
                                                                 lim.max_batch_tokens, lim.max_decode_tokens))

    def kv_pages(self):
        lim = Limits()
        self._check(lib().ribn_b200_info(self._h, C.byref(lim)))
        return lim.kv_pages_total, lim.kv_pages_free

    def admit(self, request_id: int, sequence: int, tokens: Sequence[int], max_output_tokens: int,
              temperature: float = 0.0, stop_tokens: Sequence[int] = (), sampling: Optional[Sampling] = None) -> Admission:
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        stops = np.ascontiguousarray(stop_tokens, dtype=np.uint32)
        sm = sampling or Sampling(temperature=temperature)
        sc = SamplingC(sm.temperature, sm.top_p, sm.top_k, 0, sm.seed)
        rc = lib().ribn_b200_admit(self._h, request_id, sequence, toks.ctypes.data_as(C.c_void_p), toks.size,
                                   max_output_tokens, C.byref(sc),
                                   stops.ctypes.data_as(C.c_void_p) if stops.size else None, stops.size)
        if rc == _lib.OK:
            return Admission(Admission.READY)
        if rc == _lib.REJECTED:
            return Admission(Admission.REJECTED, self._err())
        if rc == _lib.DEFERRED:
            return Admission(Admission.DEFERRED, self._err())
        raise ExecutionError(self._err())

    def prepare(self, batch: Sequence[BatchItem]) -> str:
        """Returns "ready" (BatchPreparation::Ready); raises on Err."""
        self._check(lib().ribn_b200_prepare(self._h, _items(batch), len(batch)))
        return "ready"

    def prepare_rows(self, batch: Sequence[BatchItem]):
        """prepare() with the per-row report: returns "ready" (BatchPreparation::Ready) or a list with one
        :class:`PreparedRow` per offered row (BatchPreparation::Selected); raises on Err."""
        rows = (PreparedRowC * max(len(batch), 1))()
        rc = lib().ribn_b200_prepare_rows(self._h, _items(batch), len(batch), rows)
        if rc == _lib.OK:
            return "ready"
        if rc != _lib.SELECTED:
            raise ExecutionError(self._err())
        out = []
        for it, r in zip(batch, rows):
            if r.state == _lib.ROW_READY:
                out.append(PreparedRow("ready", BatchItem(it.sequence, it.kind, it.prefix, r.token_budget, r.output_budget)))
            else:
                out.append(PreparedRow("deferred" if r.state == _lib.ROW_DEFERRED else "rejected"))
        return out

    def debug_inject(self, kind: int, value: int) -> None:
        self._check(lib().ribn_b200_debug_inject(self._h, kind, value))

    def debug_wait_expiry(self, spin_limit: int = 4096) -> None:
        self._check(lib().ribn_b200_debug_wait_expiry(self._h, spin_limit))

    def abandon_preparation(self) -> None:
        self._check(lib().ribn_b200_abandon_preparation(self._h))

    def submit(self, batch: Sequence[BatchItem]) -> int:
        sid = C.c_uint64()
        self._check(lib().ribn_b200_submit(self._h, _items(batch), len(batch), C.byref(sid)))
        return sid.value

    def poll(self, submission: int) -> Optional[List[StepCompletion]]:
        n = C.c_uint32()
        rc = lib().ribn_b200_poll(self._h, submission, self._rows, len(self._rows), C.byref(n))
        if rc == _lib.PENDING:
            return None
        self._check(rc)
        return [StepCompletion(r.sequence, r.prefix, [r.token] if r.n_tokens else [])
                for r in self._rows[: n.value]]

    def wait(self, submission: int) -> List[StepCompletion]:
        """Poll until the submission completes (the driver's poll loop,
        crates/runtime/src/driver/worker.rs:141-145, without the sleep)."""
        while True:
            done = self.poll(submission)
            if done is not None:
                return done

    def release(self, sequence: int) -> None:
        self._check(lib().ribn_b200_release(self._h, sequence))

    def synchronize(self) -> None:
        self._check(lib().ribn_b200_synchronize(self._h))

    # -- parity / measurement taps -------------------------------------------
    def copy_logits(self, row: int = 0) -> np.ndarray:
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        self._check(lib().ribn_b200_copy_logits(self._h, row, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def copy_kv(self, sequence: int, layer: int, which: int, tokens: int) -> np.ndarray:
        out = np.empty(tokens * self.cfg.kv_heads * self.cfg.head_dim, dtype=np.uint16)
        self._check(lib().ribn_b200_copy_kv(self._h, sequence, layer, which, tokens, out.ctypes.data_as(C.c_void_p)))
        return out

    def debug_set_context(self, sequence: int, tokens: int, next_token: int, seed: int = 1) -> None:
        self._check(lib().ribn_b200_debug_set_context(self._h, sequence, tokens, next_token, seed))

    def last_step_stats(self):
        ms, launches = C.c_float(), C.c_uint32()
        self._check(lib().ribn_b200_last_step_stats(self._h, C.byref(ms), C.byref(launches)))
        return ms.value, launches.value

    def step_bytes(self, context_tokens_total: int):
        w, kv = C.c_uint64(), C.c_uint64()
        self._check(lib().ribn_b200_step_bytes(self._h, context_tokens_total, C.byref(w), C.byref(kv)))
        return w.value, kv.value

    PROJECTIONS = {"qkv": 0, "attn_output": 1, "gate_up": 2, "down": 3, "head": 4}

    def time_projection(self, which: str, repeats: int = 72):
        """Average device microseconds per launch of one decode projection kernel (one row, weights
        streamed from HBM: consecutive launches take consecutive layers) and the encoded bytes a
        launch reads.  Only between steps: it overwrites the step's activation buffers."""
        us, nbytes = C.c_float(), C.c_uint64()
        self._check(lib().ribn_b200_time_projection(self._h, self.PROJECTIONS[which], repeats, C.byref(us),
                                                    C.byref(nbytes)))
        return us.value, nbytes.value

    def close(self) -> None:
        if self._h:
            lib().ribn_b200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
