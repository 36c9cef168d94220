"""A small host engine that drives an executor the way ribn's ``Engine`` does.

It restates the scheduling rules that decide the batch shapes the executor
sees — decode rows first, then prefill chunks, under a token budget, with a
forced prefill after ``max_decode_only_steps`` decode-only steps
(crates/runtime/src/engine/scheduling.rs:6-96), one batch in flight
(crates/runtime/src/engine.rs:344-398), whole-batch validation before any
commit (crates/runtime/src/engine/completion.rs:45-131), the pre-submit
negotiation over the offered rows with parked (deferred) sequences
(crates/runtime/src/engine/preparation.rs:5-140) — and nothing else of the
runtime (no mailboxes, credits, cancellation or driver thread)."""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

from .executor import Admission, BatchItem, ExecutionError, StepKind


@dataclass
class EngineConfig:  # crates/runtime/src/config.rs:5-30
    max_active_requests: int = 8
    max_queued_requests: int = 64


@dataclass
class SchedulePolicy:  # crates/runtime/src/config.rs:32-56
    max_batch_tokens: int = 128
    prefill_chunk_tokens: int = 16
    decode_tokens: int = 1
    max_decode_only_steps: int = 8


@dataclass
class TokenRequest:
    tokens: Sequence[int]
    max_output_tokens: int
    stop_tokens: Sequence[int] = ()
    temperature: float = 0.0


@dataclass
class _Slot:
    request: int
    sequence: int
    req: TokenRequest
    prompt_tokens: int
    prefix: int = 0
    generated: int = 0
    output: List[int] = field(default_factory=list)
    finish: Optional[str] = None
    enqueue_time: float = 0.0
    token_times: List[float] = field(default_factory=list)
    parked_epoch: int = -1


class Engine:
    def __init__(self, model, config: EngineConfig = EngineConfig(), policy: SchedulePolicy = SchedulePolicy()):
        info = model.info()
        # validate_policy, crates/runtime/src/config.rs:58-72; Engine::new, engine.rs:100-148
        if (policy.max_batch_tokens <= 0 or policy.prefill_chunk_tokens <= 0 or policy.decode_tokens <= 0
                or policy.max_decode_only_steps <= 0
                or policy.max_batch_tokens > info.limits.max_batch_tokens
                or policy.decode_tokens > info.limits.max_decode_tokens
                or config.max_active_requests > info.limits.max_sequences):
            raise ValueError("invalid engine configuration for this executor")
        self.model, self.config, self.policy = model, config, policy
        self.waiting: Deque[int] = deque()
        self.prefill: Deque[int] = deque()
        self.decode: Deque[int] = deque()
        self.parked: Deque[int] = deque()   # rows the executor deferred: offered again after a release
        self.resource_epoch = 0             # bumped by every release (the ReadinessWait's `changed`)
        self.slots: Dict[int, _Slot] = {}
        self.finished: Dict[int, _Slot] = {}
        self.decode_only_steps = 0
        self.in_flight = None  # (submission id, batch, slot keys)
        self._next_id = 1
        self.steps = 0
        self.faulted = False

    # -- requests -----------------------------------------------------------
    def enqueue(self, req: TokenRequest) -> int:
        if len(self.waiting) >= self.config.max_queued_requests:
            raise RuntimeError("queue full")
        rid = self._next_id
        self._next_id += 1
        self.slots[rid] = _Slot(rid, rid, req, len(req.tokens), enqueue_time=time.perf_counter())
        self.waiting.append(rid)
        return rid

    def active(self) -> int:
        return (len(self.prefill) + len(self.decode) + len(self.parked)
                + (len(self.in_flight[2]) if self.in_flight else 0))

    def idle(self) -> bool:
        return not (self.waiting or self.prefill or self.decode or self.parked or self.in_flight)

    # -- one step -------------------------------------------------------------
    def step(self) -> bool:
        """Engine::step: poll, release terminals, admit, build, prepare, submit.
        Returns True when it made progress."""
        if self.faulted:
            raise ExecutionError("engine is faulted")
        progressed = False
        try:
            if self.in_flight is not None:
                done = self.model.poll(self.in_flight[0])
                if done is None:
                    return False
                self._commit(done)
                progressed = True
            self._reactivate_parked()
            self._admit_waiters()
            batch, keys = self._build_batch()
            if batch:
                batch, keys = self._prepare(batch, keys)
            if batch:
                sid = self.model.submit(batch)
                self.in_flight = (sid, batch, keys)
                self._record(batch)
                self.steps += 1
                progressed = True
            elif self.parked and self.in_flight is None and not (self.prefill or self.decode):
                self._unblock_parked()
                progressed = True
        except ExecutionError:
            self.faulted = True  # fault_all, crates/runtime/src/engine.rs:578-594
            raise
        return progressed

    def run_until_idle(self):
        while not self.idle():
            self.step()

    # -- internals --------------------------------------------------------------
    def _prepare(self, batch, keys):
        """Engine::prepare_batch (preparation.rs:5-86): Ready keeps the batch; Selected keeps its ready rows
        (with the granted budgets), parks the deferred ones and fails the rejected ones."""
        negotiate = getattr(self.model, "prepare_rows", None)
        prepared = negotiate(batch) if negotiate else self.model.prepare(batch)
        if prepared == "ready":
            return batch, keys
        if len(prepared) != len(batch):
            self.model.abandon_preparation()
            raise ExecutionError("preparation does not match its offered rows or budgets")
        kept, kept_keys = [], []
        for row, offered, rid in zip(prepared, batch, keys):
            s = self.slots[rid]
            if row.state == "ready":
                it = row.item
                end = it.prefix + it.token_budget
                ok = (it.sequence == offered.sequence and it.kind == offered.kind and it.prefix == offered.prefix
                      and 0 < it.token_budget <= offered.token_budget and it.output_budget <= offered.output_budget)
                if it.kind == StepKind.PREFILL:
                    ok = ok and end <= s.prompt_tokens and it.output_budget == int(end == s.prompt_tokens)
                else:
                    ok = ok and it.output_budget == it.token_budget
                if not ok:
                    self.model.abandon_preparation()
                    raise ExecutionError("preparation does not match its offered rows or budgets")
                kept.append(it)
                kept_keys.append(rid)
            elif row.state == "deferred":
                s.parked_epoch = self.resource_epoch
                self.parked.append(rid)
            else:
                self._finish(rid, "failed: rejected at preparation")
        if not kept:
            self.model.abandon_preparation()
        return kept, kept_keys

    def _reactivate_parked(self):
        """reactivate_parked (preparation.rs:118-140): a parked row returns to its queue once the resource it
        waits for has changed (here: any release since it was parked)."""
        for _ in range(len(self.parked)):
            rid = self.parked.popleft()
            s = self.slots[rid]
            if s.parked_epoch == self.resource_epoch:
                self.parked.append(rid)
                continue
            (self.prefill if s.prefix < s.prompt_tokens else self.decode).append(rid)

    def _unblock_parked(self):
        """Every live sequence is parked and nothing is in flight, so no release can come: the most recently
        admitted one gives its pages back (it fails with a resource diagnostic) and the others are offered again.
        The reference leaves this policy to the executor's ReadinessWait source."""
        victim = max(self.parked)
        self.parked.remove(victim)
        self._finish(victim, "failed: KV arena exhausted")

    def _finish(self, rid, reason):
        s = self.slots[rid]
        s.finish = reason
        self.model.release(s.sequence)
        self.resource_epoch += 1
        self.finished[rid] = self.slots.pop(rid)

    def _admit_waiters(self):
        for _ in range(len(self.waiting)):
            if self.active() >= self.config.max_active_requests:
                break
            rid = self.waiting[0]
            slot = self.slots[rid]
            adm = self.model.admit(rid, slot.sequence, slot.req.tokens, slot.req.max_output_tokens,
                                   slot.req.temperature, slot.req.stop_tokens)
            if adm.state == Admission.DEFERRED:
                break
            self.waiting.popleft()
            if adm.state == Admission.REJECTED:
                slot.finish = "rejected: " + adm.reason
                self.finished[rid] = self.slots.pop(rid)
                continue
            self.prefill.append(rid)

    def _build_batch(self):
        batch: List[BatchItem] = []
        keys: List[int] = []
        budget = self.policy.max_batch_tokens
        force = bool(self.prefill) and self.decode_only_steps >= self.policy.max_decode_only_steps
        if force:
            budget = self._schedule(StepKind.PREFILL, budget, 1, batch, keys)
        budget = self._schedule(StepKind.DECODE, budget, 1 << 30, batch, keys)
        self._schedule(StepKind.PREFILL, budget, 1 << 30, batch, keys)
        return batch, keys

    def _schedule(self, kind, budget, limit, batch, keys):
        queue = self.prefill if kind == StepKind.PREFILL else self.decode
        selected = 0
        for _ in range(len(queue)):
            if selected >= limit or len(batch) >= self.config.max_active_requests or budget == 0:
                break
            rid = queue.popleft()
            s = self.slots[rid]
            if kind == StepKind.PREFILL:
                tokens = min(s.prompt_tokens - s.prefix, self.policy.prefill_chunk_tokens, budget)
                outputs = 1 if s.prefix + tokens == s.prompt_tokens else 0
            else:
                tokens = min(self.policy.decode_tokens, s.req.max_output_tokens - s.generated, budget)
                outputs = tokens
            if tokens == 0:
                queue.append(rid)
                continue
            batch.append(BatchItem(s.sequence, kind, s.prefix, tokens, outputs))
            keys.append(rid)
            budget -= tokens
            selected += 1
        return budget

    def _record(self, batch):
        if any(it.kind == StepKind.PREFILL for it in batch):
            self.decode_only_steps = 0
        elif batch and self.prefill:
            self.decode_only_steps += 1

    def _commit(self, rows):
        _, batch, keys = self.in_flight
        # Validate every row before committing any (completion.rs:45-92).
        if len(rows) != len(batch):
            raise ExecutionError("malformed completion: row count")
        for row, item, rid in zip(rows, batch, keys):
            s = self.slots[rid]
            advance = row.prefix - item.prefix
            ok = row.sequence == item.sequence and s.prefix == item.prefix and 0 < advance <= item.token_budget
            if item.kind == StepKind.PREFILL:
                ok = ok and (len(row.tokens) == 1 if row.prefix == s.prompt_tokens else len(row.tokens) == 0)
            else:
                ok = ok and len(row.tokens) == advance and len(row.tokens) <= item.output_budget
            if not ok:
                raise ExecutionError("malformed completion")
        now = time.perf_counter()
        self.in_flight = None
        for row, rid in zip(rows, keys):
            s = self.slots[rid]
            s.prefix = row.prefix
            reason = None
            for token in row.tokens:
                s.generated += 1
                if token in s.req.stop_tokens:
                    reason = "stop"
                    break
                s.output.append(token)
                s.token_times.append(now)
                if s.generated == s.req.max_output_tokens:
                    reason = "length"
                    break
            if reason:
                self._finish(rid, reason)
            elif s.prefix < s.prompt_tokens:
                self.prefill.append(rid)
            else:
                self.decode.append(rid)
