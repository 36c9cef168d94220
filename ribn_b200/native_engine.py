"""ctypes mirror of the native host engine (``include/ribn_b200_engine.h``): ribn's ``Engine`` rules in C++
over the executor's C ABI.  ``NativeEngine(model)`` drives a ``QwenB200`` executor directly (no Python in the
loop between the engine and the executor); ``NativeEngine(table=...)`` takes any executor expressed as the
header's table of C functions, which is how the host tests hand it a test double."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import EngineConfigC, EngineCountersC, ExecutorTable, RequestStatusC, SchedulePolicyC, lib
from .engine import EngineConfig, SchedulePolicy, TokenRequest
from .executor import ExecutionError

QUEUED, ACTIVE, FINISHED = 0, 1, 2


@dataclass
class RequestStatus:
    state: int
    finish: Optional[str]
    prompt_tokens: int
    prefix: int
    generated: int
    output: List[int]
    enqueue_ns: int
    first_token_ns: int
    last_token_ns: int


class NativeEngine:
    def __init__(self, model=None, config: EngineConfig = EngineConfig(), policy: SchedulePolicy = SchedulePolicy(),
                 table: Optional[ExecutorTable] = None):
        cfg = EngineConfigC(config.max_active_requests, config.max_queued_requests)
        pol = SchedulePolicyC(policy.max_batch_tokens, policy.prefill_chunk_tokens, policy.decode_tokens,
                              policy.max_decode_only_steps)
        handle = C.c_void_p()
        err = C.create_string_buffer(1024)
        if table is not None:
            self._table = table   # keeps the callbacks alive
            rc = lib().ribn_b200_engine_create(C.byref(table), C.byref(cfg), C.byref(pol), C.byref(handle), err, len(err))
        else:
            self._model = model
            rc = lib().ribn_b200_engine_create_for(model._h, C.byref(cfg), C.byref(pol), C.byref(handle), err, len(err))
        if rc != _lib.OK:
            raise ValueError(err.value.decode() or "engine creation failed")
        self._h = handle

    def close(self):
        if self._h:
            lib().ribn_b200_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _err(self) -> str:
        buf = C.create_string_buffer(4096)
        lib().ribn_b200_engine_last_error(self._h, buf, len(buf))
        return buf.value.decode(errors="replace")

    def enqueue(self, req: TokenRequest) -> int:
        toks = np.ascontiguousarray(req.tokens, dtype=np.uint32)
        stops = np.ascontiguousarray(req.stop_tokens, dtype=np.uint32)
        rid = C.c_uint64()
        rc = lib().ribn_b200_engine_enqueue(self._h, toks.ctypes.data_as(C.c_void_p), toks.size, req.max_output_tokens,
                                            stops.ctypes.data_as(C.c_void_p) if stops.size else None, stops.size,
                                            req.temperature, C.byref(rid))
        if rc == _lib.REJECTED:
            raise RuntimeError("queue full")
        if rc != _lib.OK:
            raise ExecutionError(self._err())
        return rid.value

    def step(self) -> bool:
        progressed = C.c_int32()
        if lib().ribn_b200_engine_step(self._h, C.byref(progressed)) != _lib.OK:
            raise ExecutionError(self._err())
        return bool(progressed.value)

    def idle(self) -> bool:
        return bool(lib().ribn_b200_engine_idle(self._h))

    def run_until_idle(self):
        while not self.idle():
            self.step()

    def counters(self) -> EngineCountersC:
        out = EngineCountersC()
        if lib().ribn_b200_engine_counters(self._h, C.byref(out)) != _lib.OK:
            raise ExecutionError(self._err())
        return out

    @property
    def faulted(self) -> bool:
        return bool(self.counters().faulted)

    @property
    def steps(self) -> int:
        return int(self.counters().steps)

    def token_times(self, request: int) -> np.ndarray:
        """Commit times of the request's output tokens in seconds on the monotonic clock (``time.perf_counter``'s
        clock on Linux)."""
        count = C.c_uint32()
        lib().ribn_b200_engine_token_times(self._h, request, None, 0, C.byref(count))
        out = np.empty(max(count.value, 1), dtype=np.uint64)
        lib().ribn_b200_engine_token_times(self._h, request, out.ctypes.data_as(C.c_void_p), out.size, C.byref(count))
        return out[:count.value].astype(np.float64) * 1e-9

    @property
    def in_flight(self) -> bool:
        return self.counters().in_flight_rows > 0

    def status(self, request: int) -> RequestStatus:
        st = RequestStatusC()
        if lib().ribn_b200_engine_status(self._h, request, C.byref(st)) != _lib.OK:
            raise ExecutionError(self._err())
        out = np.empty(max(st.output_tokens, 1), dtype=np.uint32)
        count = C.c_uint32()
        lib().ribn_b200_engine_output(self._h, request, out.ctypes.data_as(C.c_void_p), out.size, C.byref(count))
        reason = None
        if st.state == FINISHED:
            buf = C.create_string_buffer(1024)
            lib().ribn_b200_engine_finish_reason(self._h, request, buf, len(buf))
            reason = buf.value.decode(errors="replace")
        return RequestStatus(st.state, reason, st.prompt_tokens, st.prefix, st.generated, out[:count.value].tolist(),
                             st.enqueue_ns, st.first_token_ns, st.last_token_ns)
