"""Gemma-4 path on the GPU against the CPU oracle (oracle/gemma.c), through the C ABI of
include/ribn_b200_gemma.h.  Tolerance for logits is the stated one: max-abs 2e-2 / rel 1e-2; the
reference's own host path rounds to BF16 after every operation, and so does the device path, so most
values agree bit for bit and the rest by one BF16 step of an intermediate."""
import numpy as np
import pytest

import ribn_b200
from ribn_b200 import BatchItem, StepKind
from oracle import gemma_binding as G

pytestmark = pytest.mark.gpu

SMALL = dict(layers=4, hidden=64, heads=2, kv_heads=1, head_dim=16, global_head_dim=32, ffn=128, vocab=96, ple=16,
             ple_vocab=104, window=4, context=64, kv_shared=2, eps=1.0e-6, softcap=30.0, theta_local=1.0e4,
             theta_global=1.0e6, layer_types=["sliding", "full", "sliding", "full"])


def build_pair(cfg, seed, **limits):
    model = ribn_b200.GemmaB200(cfg, **limits)
    model.init_synthetic(seed)
    tensors = {name: model.read_tensor(name) for name in model.tensor_names()}
    model.finalize()
    return model, G.GemmaOracle(cfg, tensors)


def logits_close(got, want):
    g, w = G.to_f32(got), G.to_f32(want)
    err = np.abs(g - w)
    assert np.all(err <= 2e-2 + 1e-2 * np.abs(w)), float(err.max())
    return float(err.max()), float(np.mean(got == want))


def test_small_model_prefill_and_decode_match_the_oracle():
    model, oracle = build_pair(SMALL, 11, max_sequences=2, max_batch_tokens=8)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, SMALL["vocab"], 13).tolist()
    dev, ref = model.open(), oracle.new_sequence()
    dev.advance_prefill(prompt[:5]); ref.advance_prefill(prompt[:5])
    assert dev.position == ref.position == 5
    got, want = dev.prefill(prompt[5:]), ref.prefill(prompt[5:])   # 8 rows: one full pass
    worst, same = logits_close(got, want)
    token = G.argmax(want)
    agree = int(G.argmax(got) == token)
    for _ in range(10):  # the sliding window (4) and the shared-cache layers are all in play
        got, want = dev.decode(token), ref.decode(token)
        e, s = logits_close(got, want)
        worst, same = max(worst, e), min(same, s)
        agree += int(G.argmax(got) == G.argmax(want))
        token = G.argmax(want)
    assert dev.position == ref.position == 23
    assert agree >= 10, agree
    assert same > 0.9, same   # nearly every logit is bit-identical
    dev.close(); model.close(); oracle.close()


def test_chunking_and_batching_do_not_change_any_bit():
    model, _ = build_pair(SMALL, 12, max_sequences=4, max_batch_tokens=8)
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, SMALL["vocab"], n).tolist() for n in (3, 11, 20)]
    # one sequence at a time, whole prompt in one call (several passes for the longer ones)
    alone = []
    for p in prompts:
        s = model.open()
        first = s.prefill(p)
        second = s.decode(G.argmax(first))
        alone.append((first, second))
        s.close()
    # all three in one batched step, the long prompt cut into chunks first
    seqs = [model.open() for _ in prompts]
    seqs[2].advance_prefill(prompts[2][:7])
    tokens, logits = model.step([(seqs[0].id, prompts[0], True), (seqs[1].id, prompts[1], True),
                                 (seqs[2].id, prompts[2][7:], True)], want_logits=True)
    for i in range(3):
        assert np.array_equal(logits[i], alone[i][0])
        assert tokens[i] == G.argmax(alone[i][0])
    tokens2, logits2 = model.step([(s.id, [t], True) for s, t in zip(seqs, tokens)], want_logits=True)
    for i in range(3):
        assert np.array_equal(logits2[i], alone[i][1])
    model.close()


def test_invalid_rows_are_rejected_without_advancing():
    model, _ = build_pair(SMALL, 13, max_sequences=2, max_batch_tokens=8)
    s = model.open()
    s.advance_prefill([1, 2, 3])
    with pytest.raises(ValueError):
        s.prefill([SMALL["vocab"]])          # token outside the vocabulary
    with pytest.raises(ValueError):
        s.advance_prefill([1] * SMALL["context"])  # beyond the context
    with pytest.raises(ValueError):
        model.step([(s.id, [1], True), (s.id, [2], True)])  # the same sequence twice
    with pytest.raises(ValueError):
        model.step([(99, [1], True)])
    assert s.position == 3
    other = model.open()
    with pytest.raises(BlockingIOError):
        model.open()                          # both slots are open
    other.close(); other.close()              # close is idempotent
    model.close()


def test_executor_protocol_runs_the_reference_batch_rules():
    model, oracle = build_pair(SMALL, 14, max_sequences=3, max_batch_tokens=16)
    ex = ribn_b200.GemmaExecutor(model)
    assert ex.info().limits.max_decode_tokens == 1
    rng = np.random.default_rng(7)
    prompts = {1: rng.integers(0, SMALL["vocab"], 9).tolist(), 2: rng.integers(0, SMALL["vocab"], 4).tolist()}
    assert not ex.admit(0, 7, [1, 2], 4, temperature=0.7).ready          # greedy only
    assert not ex.admit(0, 7, [SMALL["vocab"]], 4).ready                 # token outside the vocabulary
    assert not ex.admit(0, 7, [1] * 60, 10).ready                        # prompt + output beyond the context
    for seq, p in prompts.items():
        assert ex.admit(seq, seq, p, 3).ready
    with pytest.raises(ribn_b200.ExecutionError):
        ex.prepare([BatchItem(1, StepKind.PREFILL, 0, 9, 0)])            # the prompt's end must ask for output
    batch = [BatchItem(1, StepKind.PREFILL, 0, 5, 0), BatchItem(2, StepKind.PREFILL, 0, 4, 1)]
    ex.prepare(batch)
    with pytest.raises(ribn_b200.ExecutionError):
        ex.submit(batch[:1])                                             # differs from its preparation
    done = ex.poll(ex.submit(batch))
    assert [(d.sequence, d.prefix, len(d.tokens)) for d in done] == [(1, 5, 0), (2, 4, 1)]
    refs = {seq: oracle.new_sequence() for seq in prompts}
    want2 = G.argmax(refs[2].prefill(prompts[2]))
    assert done[1].tokens == [want2]
    batch = [BatchItem(1, StepKind.PREFILL, 5, 4, 1), BatchItem(2, StepKind.DECODE, 4, 1, 1)]
    ex.prepare(batch)
    done = ex.poll(ex.submit(batch))
    assert done[0].tokens == [G.argmax(refs[1].prefill(prompts[1]))]
    assert done[1].tokens == [G.argmax(refs[2].decode(want2))]
    ex.release(2); ex.release(2)
    ex.synchronize()
    model.close(); oracle.close()


def test_reduced_gemma4_prompts_agree_with_the_oracle_under_teacher_forcing():
    """The reference's CPU-runnable configuration: 6 layers (5 sliding-512 + 1 full), hidden 1152, 4 q / 1 kv
    heads of 256, GeGLU 6912, vocab 32768; prompts of 17 / 64 / 129 / 300 uniform-random ids.  The oracle's
    greedy token is fed to both sides; every step's logits must sit within the tolerance."""
    cfg = ribn_b200.GEMMA4_REDUCED
    model, oracle = build_pair(cfg, 21, max_sequences=4, max_batch_tokens=64)
    rng = np.random.default_rng(8)
    new_tokens = 32
    steps = agree = 0
    worst, same = 0.0, 1.0
    for length in (17, 64, 129, 300):
        prompt = rng.integers(0, cfg["vocab"], length).tolist()
        dev, ref = model.open(), oracle.new_sequence()
        got, want = dev.prefill(prompt), ref.prefill(prompt)
        for _ in range(new_tokens):
            e, s = logits_close(got, want)
            worst, same = max(worst, e), min(same, s)
            steps += 1
            agree += int(G.argmax(got) == G.argmax(want))
            token = G.argmax(want)
            got, want = dev.decode(token), ref.decode(token)
        dev.close(); ref.close()
    print(f"gemma reduced: {steps} steps, greedy agreement {agree}/{steps}, max |logit diff| {worst:.3e}, "
          f"bit-identical logits >= {same:.4f}")
    assert agree >= 0.99 * steps
    assert same > 0.999
    model.close(); oracle.close()


def test_tensor_core_prefill_projections_keep_the_greedy_tokens_but_not_the_logit_tolerance():
    """RIBN_B200_GEMMA_FLAG_TENSOR_CORE_PREFILL: prefill passes multiply on the tensor cores (FP32 sums in the
    tensor core's order instead of source order).  On the reduced configuration the greedy tokens still agree
    with the oracle's, but the logits leave the 2e-2 / 1e-2 tolerance (unscaled attention scores amplify a
    one-step change of a BF16 intermediate), which is why the flag is off by default.  The divergence is
    printed; the test holds the mode to token agreement and to a loose bound on the typical logit."""
    cfg = ribn_b200.GEMMA4_REDUCED
    model = ribn_b200.GemmaB200(cfg, max_sequences=4, max_batch_tokens=64, tensor_core_prefill=True)
    model.init_synthetic(21)
    tensors = {name: model.read_tensor(name) for name in model.tensor_names()}
    model.finalize()
    oracle = G.GemmaOracle(cfg, tensors)
    rng = np.random.default_rng(8)
    steps = agree = 0
    worst, medians = 0.0, []
    for length in (17, 64, 129, 300):
        prompt = rng.integers(0, cfg["vocab"], length).tolist()
        dev, ref = model.open(), oracle.new_sequence()
        got, want = dev.prefill(prompt), ref.prefill(prompt)
        for _ in range(16):
            err = np.abs(G.to_f32(got) - G.to_f32(want))
            worst = max(worst, float(err.max()))
            medians.append(float(np.median(err)))
            steps += 1
            agree += int(G.argmax(got) == G.argmax(want))
            token = G.argmax(want)
            got, want = dev.decode(token), ref.decode(token)
        dev.close(); ref.close()
    print(f"gemma reduced, tensor-core prefill projections: greedy agreement {agree}/{steps}, "
          f"max |logit diff| {worst:.3e}, median |logit diff| per step up to {max(medians):.3e}")
    assert agree >= 0.99 * steps
    assert max(medians) < 0.5
    model.close(); oracle.close()


def test_reduced_gemma4_batch_of_four_prompts_through_the_executor():
    """The same configuration as a batch: four prompts admitted together, prefilled in 64-token chunks and
    decoded as one four-row step per token (32 greedy tokens each), against the oracle run one sequence at
    a time on its own greedy tokens."""
    cfg = ribn_b200.GEMMA4_REDUCED
    model, oracle = build_pair(cfg, 22, max_sequences=4, max_batch_tokens=128)
    ex = ribn_b200.GemmaExecutor(model)
    rng = np.random.default_rng(9)
    prompts = {i + 1: rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate((17, 64, 129, 300))}
    new_tokens = 32
    want = {}
    for seq, p in prompts.items():
        ref = oracle.new_sequence()
        token = G.argmax(ref.prefill(p))
        want[seq] = [token]
        for _ in range(new_tokens - 1):
            token = G.argmax(ref.decode(token))
            want[seq].append(token)
        ref.close()
    for seq, p in prompts.items():
        assert ex.admit(seq, seq, p, new_tokens).ready
    got = {seq: [] for seq in prompts}
    cursor = {seq: 0 for seq in prompts}
    while any(len(got[s]) < new_tokens for s in prompts):
        batch = []
        for seq, p in prompts.items():
            if len(got[seq]) >= new_tokens:
                continue
            if cursor[seq] < len(p):
                n = min(64, len(p) - cursor[seq])
                batch.append(BatchItem(seq, StepKind.PREFILL, cursor[seq], n, int(cursor[seq] + n == len(p))))
            else:
                batch.append(BatchItem(seq, StepKind.DECODE, cursor[seq], 1, 1))
        ex.prepare(batch)
        for done in ex.poll(ex.submit(batch)):
            cursor[done.sequence] = done.prefix
            got[done.sequence].extend(done.tokens)
    total = sum(len(v) for v in want.values())
    agree = sum(int(a == b) for s in prompts for a, b in zip(got[s], want[s]))
    print(f"gemma reduced, executor batch of 4: greedy agreement {agree}/{total}")
    assert agree >= 0.99 * total
    for seq in prompts:
        ex.release(seq)
    ex.synchronize()
    model.close(); oracle.close()
