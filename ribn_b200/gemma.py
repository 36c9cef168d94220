"""Python mirror of the Gemma-4 entry points of ``libribn_b200.so`` (``include/ribn_b200_gemma.h``).

``GemmaB200`` owns one model; ``GemmaSequence`` mirrors the reference's ``GemmaDecode`` backend trait
(crates/gemma4/src/executor/backend.rs:10-34: ``advance_prefill`` / ``prefill`` / ``decode`` /
``position`` / ``close``); ``GemmaExecutor`` mirrors ``Gemma4Executor`` (crates/gemma4/src/executor.rs:
55-294) behind the ``GenerationExecutor`` protocol, executing all rows of a submission in one batched
device step instead of the reference's serial per-row loop.  BF16 values travel as ``numpy.uint16``.
There is no CPU path: every call runs CUDA kernels or raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _lib
from .executor import (Admission, BatchItem, ExecutionError, ExecutorInfo, GenerationLimits, StepCompletion, StepKind)

GLOBAL_TENSORS = ("embed_tokens", "embed_tokens_per_layer", "per_layer_model_projection",
                  "per_layer_projection_norm", "norm")
LAYER_TENSORS = ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "input_layernorm",
                 "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm", "gate_proj",
                 "up_proj", "down_proj", "per_layer_input_gate", "per_layer_projection", "post_per_layer_input_norm",
                 "layer_scalar")
FLAG_TENSOR_CORE_PREFILL = 1   # RIBN_B200_GEMMA_FLAG_TENSOR_CORE_PREFILL

CONFIG_FIELDS = ("layers", "hidden", "heads", "kv_heads", "head_dim", "global_head_dim", "ffn", "vocab", "ple",
                 "ple_vocab", "window", "context", "kv_shared", "eps", "softcap", "theta_local", "theta_global")


def kv_owner(cfg: dict, layer: int) -> int:
    """Layer whose keys / values `layer` reads (crates/gemma4/src/config.rs:352-366)."""
    kinds = cfg["layer_types"]
    owners = cfg["layers"] - cfg["kv_shared"]
    if layer < owners:
        return layer
    for i in range(owners - 1, -1, -1):
        if kinds[i] == kinds[layer]:
            return i
    raise ValueError("a shared layer has no owner of its attention kind")


def tensor_names(cfg: dict) -> List[str]:
    names = list(GLOBAL_TENSORS)
    for layer in range(cfg["layers"]):
        for role in LAYER_TENSORS:
            if role in ("k_proj", "v_proj", "k_norm") and kv_owner(cfg, layer) != layer:
                continue
            names.append(f"layers.{layer}.{role}")
    return names


class GemmaB200:
    def __init__(self, cfg: dict, *, max_sequences: int = 4, max_batch_tokens: int = 64, device: int = 0,
                 tensor_core_prefill: bool = False):
        self.cfg = dict(cfg)
        c = _lib.GemmaConfig()
        for name in CONFIG_FIELDS:
            setattr(c, name, cfg[name])
        if len(cfg["layer_types"]) != cfg["layers"]:
            raise ValueError("one attention type per layer is required")
        for i, kind in enumerate(cfg["layer_types"]):
            if kind not in ("sliding", "full"):
                raise ValueError(f"unsupported attention: {kind}")
            c.full[i] = 1 if kind == "full" else 0
        c.max_sequences, c.max_batch_tokens, c.device = max_sequences, max_batch_tokens, device
        c.flags = FLAG_TENSOR_CORE_PREFILL if tensor_core_prefill else 0
        self.max_sequences, self.max_batch_tokens = max_sequences, max_batch_tokens
        self._lib = _lib.lib()
        handle = C.c_void_p()
        err = C.create_string_buffer(512)
        if self._lib.ribn_b200_gemma_create(C.byref(c), C.byref(handle), err, len(err)) != _lib.OK:
            raise ExecutionError(err.value.decode() or "ribn_b200_gemma_create failed")
        self._h = handle

    def _check(self, rc: int):
        if rc != _lib.OK:
            raise ExecutionError(self._lib.ribn_b200_gemma_last_error(self._h).decode())

    def load_tensor(self, name: str, values) -> None:
        a = np.ascontiguousarray(values, dtype=np.uint16).reshape(-1)
        self._check(self._lib.ribn_b200_gemma_load_tensor(self._h, name.encode(), a.ctypes.data_as(C.c_void_p), a.size))

    def init_synthetic(self, seed: int) -> None:
        self._check(self._lib.ribn_b200_gemma_init_synthetic(self._h, seed))

    def read_tensor(self, name: str) -> np.ndarray:
        count = C.c_size_t()
        self._check(self._lib.ribn_b200_gemma_read_tensor(self._h, name.encode(), None, 0, C.byref(count)))
        out = np.empty(count.value, dtype=np.uint16)
        self._check(self._lib.ribn_b200_gemma_read_tensor(self._h, name.encode(), out.ctypes.data_as(C.c_void_p), out.size, None))
        return out

    def tensor_names(self) -> List[str]:
        return tensor_names(self.cfg)

    def finalize(self) -> None:
        self._check(self._lib.ribn_b200_gemma_finalize(self._h))

    def open(self) -> "GemmaSequence":
        seq = C.c_uint64()
        rc = self._lib.ribn_b200_gemma_open(self._h, C.byref(seq))
        if rc == _lib.DEFERRED:
            raise BlockingIOError(self._lib.ribn_b200_gemma_last_error(self._h).decode())
        self._check(rc)
        return GemmaSequence(self, seq.value)

    def step(self, rows: Sequence[tuple], want_logits: bool = False):
        """rows: (sequence id, tokens, want_output).  Returns (tokens per row or None, logits per output row)."""
        n = len(rows)
        arr = (_lib.GemmaRow * n)()
        keep = []
        outputs = 0
        for i, (seq, tokens, want) in enumerate(rows):
            t = np.ascontiguousarray(tokens, dtype=np.uint32)
            keep.append(t)
            arr[i].sequence = seq
            arr[i].tokens = t.ctypes.data_as(C.POINTER(C.c_uint32))
            arr[i].n_tokens = t.size
            arr[i].want_output = 1 if want else 0
            outputs += 1 if want else 0
        out = np.zeros(n, dtype=np.uint32)
        logits = np.empty((outputs, self.cfg["vocab"]), dtype=np.uint16) if want_logits and outputs else None
        rc = self._lib.ribn_b200_gemma_step(self._h, arr, n, out.ctypes.data_as(C.c_void_p),
                                            logits.ctypes.data_as(C.c_void_p) if logits is not None else None)
        if rc == _lib.REJECTED:
            raise ValueError(self._lib.ribn_b200_gemma_last_error(self._h).decode())
        self._check(rc)
        tokens_out = [int(out[i]) if rows[i][2] else None for i in range(n)]
        return tokens_out, logits

    def synchronize(self) -> None:
        self._check(self._lib.ribn_b200_gemma_synchronize(self._h))

    def last_step_stats(self):
        ms, launches = C.c_float(), C.c_uint32()
        self._check(self._lib.ribn_b200_gemma_last_step_stats(self._h, C.byref(ms), C.byref(launches)))
        return ms.value, launches.value

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ribn_b200_gemma_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GemmaSequence:
    """One continuation: the reference's `GemmaDecode` (backend.rs:10-34)."""

    def __init__(self, model: GemmaB200, sequence: int):
        self.model, self.id, self._open = model, sequence, True

    def _call(self, tokens, want_logits: bool):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        m = self.model
        if not want_logits:
            rc = m._lib.ribn_b200_gemma_advance_prefill(m._h, self.id, t.ctypes.data_as(C.c_void_p), t.size)
            logits = None
        else:
            logits = np.empty(m.cfg["vocab"], dtype=np.uint16)
            rc = m._lib.ribn_b200_gemma_prefill(m._h, self.id, t.ctypes.data_as(C.c_void_p), t.size,
                                                logits.ctypes.data_as(C.c_void_p), None)
        if rc == _lib.REJECTED:
            raise ValueError(m._lib.ribn_b200_gemma_last_error(m._h).decode())
        m._check(rc)
        return logits

    def advance_prefill(self, tokens) -> None:
        self._call(tokens, False)

    def prefill(self, tokens) -> np.ndarray:
        return self._call(tokens, True)

    def decode(self, token: int) -> np.ndarray:
        return self._call([token], True)

    @property
    def position(self) -> int:
        out = C.c_uint32()
        self.model._check(self.model._lib.ribn_b200_gemma_position(self.model._h, self.id, C.byref(out)))
        return out.value

    def close(self) -> None:
        if self._open:
            self.model._check(self.model._lib.ribn_b200_gemma_close(self.model._h, self.id))
            self._open = False


class _Logical:
    """Model-local continuation (crates/gemma4/src/generation.rs:9-14)."""

    def __init__(self, prompt: List[int], output: int, decoder: GemmaSequence):
        self.prompt, self.cursor, self.input, self.remaining, self.decoder = prompt, 0, None, output, decoder


class GemmaExecutor:
    """The `GenerationExecutor` protocol for Gemma (crates/gemma4/src/executor.rs:179-294) with the
    reference's phases (idle / prepared / submitted / failed / closed) and whole-offer binding rules
    (crates/gemma4/src/generation.rs:77-160).  `poll` runs every bound row in ONE batched device step."""

    MEDIA_TOKENS: tuple = ()

    def __init__(self, model: GemmaB200, name: str = "gemma4 b200"):
        self.model = model
        self._info = ExecutorInfo(name, GenerationLimits(model.cfg["context"], model.max_sequences, 4096, 1))
        self._states: Dict[int, _Logical] = {}
        self._rows: List[tuple] = []   # (item, tokens)
        self._phase = "idle"
        self._next = 0
        self._submitted: Optional[int] = None

    def info(self) -> ExecutorInfo:
        return self._info

    def admit(self, request_id: int, sequence: int, tokens: Sequence[int], max_output_tokens: int,
              temperature: float = 0.0) -> Admission:
        if self._phase != "idle":
            self._phase = "failed"
            raise ExecutionError("Gemma execution is busy, faulted or closed")
        if sequence in self._states:
            self._phase = "failed"
            raise ExecutionError("sequence is already admitted")
        limits = self._info.limits
        if len(self._states) >= limits.max_sequences:
            return Admission(Admission.REJECTED, "sequence capacity is exhausted")
        if temperature != 0.0:
            return Admission(Admission.REJECTED, "Gemma executor currently supports greedy sampling only")
        prompt = [int(t) for t in tokens]
        if not prompt or max_output_tokens <= 0:
            return Admission(Admission.REJECTED, "prompt and output budget must be positive")
        if len(prompt) + max_output_tokens > limits.context_tokens:
            return Admission(Admission.REJECTED, "prompt and output exceed the context bound")
        if any(t in self.MEDIA_TOKENS for t in prompt):
            return Admission(Admission.REJECTED, "media placeholders require the multimodal processor")
        if any(t < 0 or t >= self.model.cfg["vocab"] for t in prompt):
            return Admission(Admission.REJECTED, "token ID outside model vocabulary")
        try:
            decoder = self.model.open()
        except BlockingIOError as e:
            return Admission(Admission.REJECTED, str(e))
        self._states[sequence] = _Logical(prompt, max_output_tokens, decoder)
        return Admission(Admission.READY)

    def _bind(self, item: BatchItem, state: _Logical):
        limits = self._info.limits
        end = item.prefix + item.token_budget
        if item.token_budget == 0 or item.prefix != state.cursor or end > limits.context_tokens or state.remaining == 0:
            raise ExecutionError("work disagrees with continuation or capacity")
        if item.kind == StepKind.PREFILL:
            if end > len(state.prompt) or item.output_budget != int(end == len(state.prompt)):
                raise ExecutionError("prefill boundary/output mismatch")
            return state.prompt[item.prefix:end]
        if item.token_budget != 1 or item.output_budget != 1 or item.prefix < len(state.prompt):
            raise ExecutionError("invalid ordinary decode row")
        if state.input is None:
            raise ExecutionError("ordinary decode has no input")
        return [state.input]

    def prepare(self, batch: Sequence[BatchItem]) -> str:
        if self._phase != "idle":
            raise ExecutionError("Gemma execution is busy, faulted or closed")
        limits = self._info.limits
        if not batch or len(batch) > limits.max_sequences or sum(i.token_budget for i in batch) > limits.max_batch_tokens:
            raise ExecutionError("Gemma batch exceeds prepared limits")
        rows = []
        for index, item in enumerate(batch):
            if any(old.sequence == item.sequence for old in batch[:index]):
                raise ExecutionError("duplicate Gemma sequence in batch")
            state = self._states.get(item.sequence)
            if state is None:
                raise ExecutionError("submitted sequence is not admitted")
            rows.append((item, self._bind(item, state)))
        for item, _ in rows:
            if self._states[item.sequence].decoder.position != self._states[item.sequence].cursor:
                raise ExecutionError("decoder disagrees with logical continuation")
        self._rows = rows
        self._phase = "prepared"
        return "ready"

    def abandon_preparation(self) -> None:
        if self._phase == "prepared":
            self._rows = []
            self._phase = "idle"
        elif self._phase not in ("idle", "closed"):
            raise ExecutionError("cannot abandon submitted or failed work")

    def submit(self, batch: Sequence[BatchItem]) -> int:
        if self._phase != "prepared" or [r[0] for r in self._rows] != list(batch):
            raise ExecutionError("submission differs from its preparation")
        self._next += 1
        self._submitted = self._next
        self._phase = "submitted"
        return self._next

    def poll(self, submission: int) -> Optional[List[StepCompletion]]:
        if self._phase != "submitted" or submission != self._submitted:
            raise ExecutionError("unknown Gemma submission")
        self._phase = "failed"  # anything that escapes below leaves the executor faulted
        step_rows = [(self._states[item.sequence].decoder.id, tokens, item.output_budget > 0) for item, tokens in self._rows]
        try:
            chosen, _ = self.model.step(step_rows)
        except ValueError as e:
            raise ExecutionError(str(e)) from e
        done = []
        for (item, _tokens), token in zip(self._rows, chosen):
            state = self._states[item.sequence]
            end = item.prefix + item.token_budget
            if state.decoder.position != end:
                raise ExecutionError("decoder did not complete the accepted range")
            state.cursor = end
            if token is not None:
                state.input = token
                state.remaining -= 1
            done.append(StepCompletion(item.sequence, end, [] if token is None else [token]))
        self._rows = []
        self._phase = "idle"
        return done

    def wait(self, submission: int) -> List[StepCompletion]:
        return self.poll(submission)

    def release(self, sequence: int) -> None:
        if self._phase == "failed" or any(item.sequence == sequence for item, _ in self._rows):
            raise ExecutionError("cannot release prepared, submitted or failed state")
        state = self._states.pop(sequence, None)
        if state is not None:
            state.decoder.close()

    def synchronize(self) -> None:
        if self._phase == "closed":
            return
        self.model.synchronize()
        self._rows = []
        for state in self._states.values():
            state.decoder.close()
        self._states.clear()
        self._phase = "closed"
