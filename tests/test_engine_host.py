"""Host scheduling rules, checked against a fake executor in the style of the
reference's runtime contract tests (crates/runtime/tests/contract.rs:12-178):
a shared control block of fault switches, a delayed first poll, and a record
of every batch the engine offered."""
from dataclasses import dataclass, field

import pytest

from ribn_b200.engine import Engine as PyEngine, EngineConfig, SchedulePolicy, TokenRequest
from ribn_b200.executor import (Admission, BatchItem, ExecutionError, ExecutorInfo, GenerationLimits, PreparedRow,
                                StepCompletion, StepKind)


@dataclass
class Control:
    defer: bool = False
    reject_admission: bool = False
    fail_submit: bool = False
    fail_poll: bool = False
    malformed: bool = False
    delay: int = 0
    batches: list = field(default_factory=list)
    released: list = field(default_factory=list)


class Fake:
    def __init__(self, control, max_sequences=8, max_batch_tokens=64):
        self.c = control
        self.limits = GenerationLimits(256, max_sequences, max_batch_tokens, 1)
        self.pending = None
        self.prepared = None
        self.sid = 0

    def info(self):
        return ExecutorInfo("fake", self.limits)

    def admit(self, request_id, sequence, tokens, max_output_tokens, temperature=0.0, stop_tokens=()):
        if self.c.defer:
            return Admission(Admission.DEFERRED, "no capacity")
        if self.c.reject_admission:
            return Admission(Admission.REJECTED, "refused")
        return Admission(Admission.READY)

    def prepare(self, batch):
        assert self.pending is None and self.prepared is None
        self.prepared = list(batch)
        return "ready"

    def submit(self, batch):
        assert list(batch) == self.prepared
        self.prepared = None
        if self.c.fail_submit:
            raise ExecutionError("submit failed")
        self.c.batches.append(list(batch))
        self.sid += 1
        self.pending = (self.sid, list(batch), self.c.delay)
        return self.sid

    def poll(self, sid):
        if self.c.fail_poll:
            raise ExecutionError("poll failed")
        pid, batch, delay = self.pending
        assert pid == sid
        if delay > 0:
            self.pending = (pid, batch, delay - 1)
            return None
        self.pending = None
        rows = []
        for it in batch:
            tokens = [100 + it.prefix] if it.output_budget else []
            rows.append(StepCompletion(it.sequence, it.prefix + it.token_budget, tokens))
        if self.c.malformed:
            rows[0] = StepCompletion(rows[0].sequence, rows[0].prefix + 1, rows[0].tokens)
        return rows

    def release(self, sequence):
        self.c.released.append(sequence)


class TableAdapter:
    """A Python executor double behind the C table of include/ribn_b200_engine.h: every callback forwards to the
    double's method and turns its answer (or its ExecutionError) into the ABI's return codes."""

    def __init__(self, fake):
        import ctypes as C
        from ribn_b200 import _lib
        self.fake, self.error = fake, b""
        L = _lib

        def guard(fn):
            def wrapped(*args):
                try:
                    return fn(*args)
                except ExecutionError as exc:
                    self.error = str(exc).encode()
                    return L.ERROR
            return wrapped

        def info(_self, out):
            lim = fake.info().limits
            out[0].context_tokens, out[0].max_sequences = lim.context_tokens, lim.max_sequences
            out[0].max_batch_tokens, out[0].max_decode_tokens = lim.max_batch_tokens, lim.max_decode_tokens
            return L.OK

        def admit(_self, request_id, sequence, tokens, n, max_out, sampling, stops, n_stops):
            adm = fake.admit(request_id, sequence, [tokens[i] for i in range(n)], max_out, sampling[0].temperature,
                             [stops[i] for i in range(n_stops)])
            self.error = (adm.reason or "").encode()
            return {Admission.READY: L.OK, Admission.REJECTED: L.REJECTED, Admission.DEFERRED: L.DEFERRED}[adm.state]

        def items_of(items, n):
            return [BatchItem(items[i].sequence, StepKind(items[i].kind), items[i].prefix, items[i].token_budget,
                              items[i].output_budget) for i in range(n)]

        def prepare_rows(_self, items, n, rows):
            batch = items_of(items, n)
            negotiate = getattr(fake, "prepare_rows", None)
            got = negotiate(batch) if negotiate else fake.prepare(batch)
            if got == "ready":
                return L.OK
            for i, row in enumerate(got):
                rows[i].state = {"ready": 0, "deferred": 1, "rejected": 2}[row.state]
                if row.state == "ready":
                    rows[i].token_budget, rows[i].output_budget = row.item.token_budget, row.item.output_budget
            return L.SELECTED

        def abandon(_self):
            fake.abandon_preparation()
            return L.OK

        def submit(_self, items, n, sid):
            sid[0] = fake.submit(items_of(items, n))
            return L.OK

        def poll(_self, sid, rows, capacity, count):
            done = fake.poll(sid)
            if done is None:
                return L.PENDING
            count[0] = len(done)
            for i, row in enumerate(done[:capacity]):
                rows[i].sequence, rows[i].prefix, rows[i].n_tokens = row.sequence, row.prefix, len(row.tokens)
                rows[i].token = row.tokens[0] if row.tokens else 0
            return L.OK

        def release(_self, sequence):
            fake.release(sequence)
            return L.OK

        def last_error(_self, buf, capacity):
            text = self.error[:max(capacity - 1, 0)]
            C.memmove(buf, text + b"\0", len(text) + 1)
            return len(text)

        self.table = L.ExecutorTable(None, L._INFO_FN(guard(info)), L._ADMIT_FN(guard(admit)), L._PREPARE_FN(guard(prepare_rows)),
                                     L._ABANDON_FN(guard(abandon)), L._SUBMIT_FN(guard(submit)), L._POLL_FN(guard(poll)),
                                     L._RELEASE_FN(guard(release)), L._LAST_ERROR_FN(last_error))


class NativeFacade:
    """The native engine behind the attribute names the tests below use on the Python engine."""

    def __init__(self, fake, config, policy):
        from ribn_b200.native_engine import NativeEngine
        self.adapter = TableAdapter(fake)
        self.engine = NativeEngine(config=config, policy=policy, table=self.adapter.table)
        self.requests = []

    def enqueue(self, req):
        rid = self.engine.enqueue(req)
        self.requests.append(rid)
        return rid

    def step(self):
        return self.engine.step()

    def idle(self):
        return self.engine.idle()

    @property
    def faulted(self):
        return self.engine.faulted

    def _by_state(self, states):
        out = {}
        for rid in self.requests:
            st = self.engine.status(rid)
            if st.state in states:
                out[rid] = st
        return out

    @property
    def finished(self):
        return self._by_state((2,))

    @property
    def slots(self):
        return self._by_state((0, 1))

    @property
    def waiting(self):
        return list(self._by_state((0,)))

    @property
    def parked(self):
        return [None] * self.engine.counters().parked


@pytest.fixture(params=["python", "native"])
def Engine(request, built_library):
    """The Python engine and the native one (include/ribn_b200_engine.h) under the same cases."""
    if request.param == "python":
        return PyEngine
    return NativeFacade


def run(engine, limit=10000):
    for _ in range(limit):
        if engine.idle():
            return
        engine.step()
    raise AssertionError("engine did not drain")


def test_prefill_is_chunked_then_decode_runs_one_token_steps(Engine):
    c = Control()
    e = Engine(Fake(c), EngineConfig(max_active_requests=4), SchedulePolicy(64, 16, 1, 8))
    rid = e.enqueue(TokenRequest(list(range(40)), 3))
    run(e)
    kinds = [(b[0].kind, b[0].prefix, b[0].token_budget, b[0].output_budget) for b in c.batches]
    assert kinds[:3] == [(StepKind.PREFILL, 0, 16, 0), (StepKind.PREFILL, 16, 16, 0), (StepKind.PREFILL, 32, 8, 1)]
    assert kinds[3:] == [(StepKind.DECODE, 40, 1, 1), (StepKind.DECODE, 41, 1, 1)]
    done = e.finished[rid]
    assert done.finish == "length" and done.output == [132, 140, 141] and c.released == [rid]


def test_decode_rows_come_first_and_share_the_token_budget(Engine):
    c = Control()
    e = Engine(Fake(c, max_batch_tokens=20), EngineConfig(max_active_requests=4), SchedulePolicy(20, 16, 1, 8))
    a = e.enqueue(TokenRequest(list(range(4)), 50))
    e.step(); e.step()          # prefill a (one chunk), then its first decode is built with...
    b = e.enqueue(TokenRequest(list(range(100)), 2))
    e.step()
    batch = c.batches[-1]
    assert [it.kind for it in batch] == [StepKind.DECODE, StepKind.PREFILL]
    assert batch[1].token_budget == 16 and sum(it.token_budget for it in batch) <= 20
    assert a != b


def test_forced_prefill_after_decode_only_steps(Engine):
    c = Control()
    # budget 1: a decode row always exhausts it, so prefill starves until forced
    e = Engine(Fake(c), EngineConfig(max_active_requests=4), SchedulePolicy(1, 1, 1, 3))
    e.enqueue(TokenRequest([1], 100))
    e.step(); e.step()
    e.enqueue(TokenRequest([1, 2, 3], 1))
    for _ in range(12):
        e.step()
    kinds = [b[0].kind for b in c.batches]
    window = kinds[2:10]
    assert StepKind.PREFILL in window
    first = window.index(StepKind.PREFILL)
    assert first <= 4  # at most max_decode_only_steps (+1 in flight) decode-only steps before the forced prefill


def test_pending_poll_makes_no_progress_and_keeps_one_batch_in_flight(Engine):
    c = Control(delay=2)
    e = Engine(Fake(c), EngineConfig(max_active_requests=2), SchedulePolicy(64, 64, 1, 8))
    e.enqueue(TokenRequest([1, 2, 3], 1))
    assert e.step() is True
    assert e.step() is False and e.step() is False
    assert len(c.batches) == 1
    run(e)
    assert len(c.batches) == 1 and len(e.finished) == 1


def test_malformed_completion_faults_before_any_commit(Engine):
    c = Control(malformed=True)
    e = Engine(Fake(c), EngineConfig(max_active_requests=2), SchedulePolicy(64, 64, 1, 8))
    rid = e.enqueue(TokenRequest([1, 2, 3], 4))
    e.step()
    with pytest.raises(ExecutionError):
        e.step()
    assert e.faulted and e.slots[rid].prefix == 0 and e.slots[rid].output == []
    with pytest.raises(ExecutionError):
        e.step()


@pytest.mark.parametrize("switch", ["fail_submit", "fail_poll"])
def test_executor_errors_fault_the_engine(Engine, switch):
    c = Control()
    e = Engine(Fake(c), EngineConfig(max_active_requests=2), SchedulePolicy(64, 64, 1, 8))
    e.enqueue(TokenRequest([1, 2, 3], 4))
    if switch == "fail_poll":
        e.step()
    setattr(c, switch, True)
    with pytest.raises(ExecutionError):
        e.step()
    assert e.faulted


def test_rejected_and_deferred_admission(Engine):
    c = Control(reject_admission=True)
    e = Engine(Fake(c), EngineConfig(max_active_requests=2), SchedulePolicy(64, 64, 1, 8))
    rid = e.enqueue(TokenRequest([1], 1))
    e.step()
    assert e.finished[rid].finish.startswith("rejected") and e.idle()
    c.reject_admission, c.defer = False, True
    rid2 = e.enqueue(TokenRequest([1], 1))
    e.step()
    assert list(e.waiting) == [rid2] and not c.batches
    c.defer = False
    run(e)
    assert e.finished[rid2].finish == "length"


def test_policy_must_fit_executor_limits(Engine):
    with pytest.raises(ValueError):
        Engine(Fake(Control(), max_batch_tokens=32), EngineConfig(2), SchedulePolicy(64, 16, 1, 8))
    with pytest.raises(ValueError):
        Engine(Fake(Control(), max_sequences=2), EngineConfig(4), SchedulePolicy(32, 16, 1, 8))


class PagedFake(Fake):
    """A fake whose `prepare_rows` negotiates 16-token pages from a small pool the way the executor does:
    a row that needs more pages than are free is deferred (or, for a prefill row, shortened)."""

    def __init__(self, control, pages):
        super().__init__(control)
        self.free, self.held = pages, {}

    def admit(self, request_id, sequence, tokens, max_output_tokens, temperature=0.0, stop_tokens=()):
        self.held[sequence] = 0
        return Admission(Admission.READY)

    def prepare_rows(self, batch):
        assert self.pending is None and self.prepared is None
        rows, unchanged = [], True
        for it in batch:
            need = -(-(it.prefix + it.token_budget) // 16) - self.held[it.sequence]
            if need <= self.free:
                self.free -= max(need, 0)
                self.held[it.sequence] += max(need, 0)
                rows.append(PreparedRow("ready", it))
                continue
            unchanged = False
            fits = (self.held[it.sequence] + self.free) * 16
            if it.kind == StepKind.PREFILL and fits > it.prefix:
                self.held[it.sequence] += self.free
                self.free = 0
                rows.append(PreparedRow("ready", BatchItem(it.sequence, it.kind, it.prefix, fits - it.prefix, 0)))
            else:
                rows.append(PreparedRow("deferred"))
        self.prepared = [r.item for r in rows if r.state == "ready"]
        return "ready" if unchanged else rows

    def abandon_preparation(self):
        self.prepared = None

    def release(self, sequence):
        super().release(sequence)
        self.free += self.held.pop(sequence)


def test_deferred_rows_are_parked_and_offered_again_after_a_release(Engine):
    c = Control()
    fake = PagedFake(c, pages=3)
    e = Engine(fake, EngineConfig(max_active_requests=4), SchedulePolicy(64, 32, 1, 8))
    a = e.enqueue(TokenRequest(list(range(20)), 2))     # 2 pages for the prompt, decode stays inside them
    b = e.enqueue(TokenRequest(list(range(30)), 2))     # needs 2 pages: only 1 is free at first
    run(e)
    assert e.finished[a].finish == "length" and e.finished[b].finish == "length"
    first = c.batches[0]
    assert [(it.sequence, it.token_budget, it.output_budget) for it in first] == [(a, 20, 1), (b, 16, 0)]  # b shortened
    # b's remaining 14 prompt tokens waited (parked) until a finished and gave its pages back
    later = [it for batch in c.batches[1:] for it in batch if it.sequence == b and it.kind == StepKind.PREFILL]
    assert [(it.prefix, it.token_budget, it.output_budget) for it in later] == [(16, 14, 1)]
    assert fake.free == 3 and not e.parked


def test_a_pool_that_can_never_serve_every_sequence_fails_the_newest_one(Engine):
    c = Control()
    fake = PagedFake(c, pages=2)
    e = Engine(fake, EngineConfig(max_active_requests=4), SchedulePolicy(64, 16, 1, 8))
    a = e.enqueue(TokenRequest(list(range(16)), 40))    # grows to 4 pages: can never finish beside b
    b = e.enqueue(TokenRequest(list(range(16)), 40))
    run(e)
    assert sorted([e.finished[a].finish, e.finished[b].finish]) == ["failed: KV arena exhausted"] * 2 or \
        "failed: KV arena exhausted" in (e.finished[a].finish, e.finished[b].finish)
    assert fake.free == 2 and e.idle()


def test_native_engine_stamps_tokens_on_the_monotonic_clock(built_library):
    """Token commit times come from the steady clock, the clock of time.perf_counter on Linux: the benchmark
    subtracts one from the other for the time to first token."""
    import time
    from ribn_b200.native_engine import NativeEngine
    c = Control()
    adapter = TableAdapter(Fake(c))
    e = NativeEngine(config=EngineConfig(max_active_requests=2), policy=SchedulePolicy(64, 16, 1, 8), table=adapter.table)
    before = time.perf_counter()
    rid = e.enqueue(TokenRequest(list(range(20)), 3))
    e.run_until_idle()
    after = time.perf_counter()
    stamps = e.token_times(rid)
    st = e.status(rid)
    assert len(stamps) == 3 == len(st.output) and list(stamps) == sorted(stamps)
    assert before <= st.enqueue_ns * 1e-9 <= stamps[0] <= stamps[-1] <= after
    assert abs(stamps[0] - st.first_token_ns * 1e-9) < 1e-6 and abs(stamps[-1] - st.last_token_ns * 1e-9) < 1e-6
    assert not e.in_flight and e.steps == 4
    e.close()


def test_native_engine_argument_and_queue_errors(built_library):
    """Creation refuses an incomplete executor table and a policy beyond the executor's limits; a full queue
    refuses the request without faulting; unknown requests are errors; a stop token ends a request before it
    reaches the output."""
    import ctypes as C
    from ribn_b200 import _lib
    from ribn_b200.native_engine import NativeEngine
    c = Control()
    adapter = TableAdapter(Fake(c))
    broken = _lib.ExecutorTable()
    C.memmove(C.byref(broken), C.byref(adapter.table), C.sizeof(broken))
    broken.submit = _lib._SUBMIT_FN()      # a NULL entry
    with pytest.raises(ValueError, match="incomplete"):
        NativeEngine(config=EngineConfig(2), policy=SchedulePolicy(64, 16, 1, 8), table=broken)
    with pytest.raises(ValueError, match="invalid engine configuration"):
        NativeEngine(config=EngineConfig(2), policy=SchedulePolicy(64, 0, 1, 8), table=adapter.table)
    e = NativeEngine(config=EngineConfig(max_active_requests=1, max_queued_requests=2), policy=SchedulePolicy(64, 16, 1, 8),
                     table=adapter.table)
    a = e.enqueue(TokenRequest([1, 2, 3], 5, stop_tokens=[103]))    # the fake samples 100 + the row's prefix: 100, then 103
    b = e.enqueue(TokenRequest([4], 1))
    with pytest.raises(RuntimeError, match="queue full"):
        e.enqueue(TokenRequest([5], 1))
    assert not e.faulted
    with pytest.raises(ExecutionError, match="unknown request"):
        e.status(99)
    e.run_until_idle()
    sa, sb = e.status(a), e.status(b)
    assert sa.finish == "stop" and sa.output == [100] and sa.generated == 2
    assert sb.finish == "length" and sb.output == [100]
    assert c.released == [a, b] and e.counters().resource_epoch == 2
    e.close()


class GreedyFake(PagedFake):
    """Answers Selected with a row whose granted budget exceeds what was offered."""

    def prepare_rows(self, batch):
        self.prepared = list(batch)
        it = batch[0]
        return [PreparedRow("ready", BatchItem(it.sequence, it.kind, it.prefix, it.token_budget + 1, it.output_budget))]


def test_a_preparation_that_grants_more_than_offered_faults_the_engine(Engine):
    """prepare_batch checks every Selected row against the offer (preparation.rs:40-86): a granted budget above the
    offered one abandons the preparation and is a final fault."""
    c = Control()
    fake = GreedyFake(c, pages=8)
    e = Engine(fake, EngineConfig(max_active_requests=2), SchedulePolicy(64, 16, 1, 8))
    e.enqueue(TokenRequest(list(range(10)), 2))
    with pytest.raises(ExecutionError, match="does not match"):
        e.step()
    assert e.faulted and fake.prepared is None and not c.batches
    with pytest.raises(ExecutionError):
        e.step()
