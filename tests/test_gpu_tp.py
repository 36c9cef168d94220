"""Tensor parallelism on two GPUs (one process per GPU, NCCL all-reduce after the attention output and the ffn
down projections): a reduced-width dense-Qwen3 model whose ffn splits unevenly (5 blocks: 3 + 2), prefill
through the batched kernels and greedy decode through the GEMV chain (replayed from a captured graph), logits
within max-abs 2e-2 / rel 1e-2 of the CPU oracle on the WHOLE model and the same tokens on both ranks."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TP_MODEL = dict(layers=3, hidden=1024, q_heads=8, kv_heads=2, head_dim=128, ffn=1280, vocab=2048, rope_base=1.0e6,
                rms_eps=1.0e-6)


def _rank(rank: int, world: int, group_id: bytes, scheme: str, out):
    sys.path.insert(0, ROOT)
    import ribn_b200
    from ribn_b200 import BatchItem, StepKind
    from tests import helpers as H
    tensors = H.make_model(TP_MODEL, seed=23, scheme=scheme)          # the same whole checkpoint on every rank
    ex = ribn_b200.QwenB200(TP_MODEL, context_tokens=128, max_sequences=2, max_batch_tokens=32, device=rank,
                            flags=ribn_b200.FLAG_KEEP_LOGITS, tp_size=world, tp_rank=rank)
    for name, (kind, rows, cols, data) in tensors.items():
        ex.load_tensor(name, kind, rows, cols, data)                   # whole tensors in; each rank keeps its shard
    kind, rows, cols, shard = ex.read_tensor("blk.1.ffn_down.weight")
    shard_shape = (rows, cols)
    ex.tp_init(group_id)
    ex.finalize()
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, TP_MODEL["vocab"], size=21).tolist()
    assert ex.admit(1, 1, prompt, 12).ready
    item = BatchItem(1, StepKind.PREFILL, 0, len(prompt), 1)
    ex.prepare([item])
    done = ex.wait(ex.submit([item]))
    logits = [ex.copy_logits(0)]
    tokens = [done[0].tokens[0]]
    for step in range(10):
        item = BatchItem(1, StepKind.DECODE, len(prompt) + step, 1, 1)
        ex.prepare([item])
        done = ex.wait(ex.submit([item]))
        logits.append(ex.copy_logits(0))
        tokens.append(done[0].tokens[0])
    _, launches = ex.last_step_stats()
    ex.release(1)
    ex.close()
    out.put((rank, shard_shape, tokens, np.stack(logits), launches))


@pytest.mark.parametrize("scheme", ["q4_k_m", "q8_0"])
def test_two_rank_tensor_parallel_logits_match_the_oracle(built_library, scheme):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import ribn_b200
    from oracle import binding as orc
    from tests import helpers as H
    group_id = ribn_b200.tp_unique_id()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, group_id, scheme, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted((out.get(timeout=300) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, shape0, tokens0, logits0, launches0), (_, shape1, tokens1, logits1, _) = results
    assert shape0 == (1024, 768) and shape1 == (1024, 512)             # ffn 1280 = 5 blocks: 3 + 2
    assert tokens0 == tokens1
    assert np.array_equal(logits0.view(np.uint32), logits1.view(np.uint32))   # the replicated head sees the same bits
    # the oracle runs the whole model
    tensors = H.make_model(TP_MODEL, seed=23, scheme=scheme)
    orc.set_threads(8)
    oracle = orc.Qwen3Oracle(H.oracle_config(TP_MODEL, 128), tensors)
    seq = oracle.new_sequence()
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, TP_MODEL["vocab"], size=21).tolist()
    for t in prompt[:-1]:
        seq.step(t, want_logits=False)
    want = seq.step(prompt[-1])
    worst = 0.0
    for step, token in enumerate(tokens0):
        err = np.abs(logits0[step] - want)
        worst = max(worst, float(err.max()))
        assert np.all((err < 2e-2) | (err < 1e-2 * np.abs(want))), (step, float(err.max()))
        assert token == orc.argmax(logits0[step])
        want = seq.step(token)                                         # teacher-forced with the device's token
    print(f"tp2 {scheme}: max |logit diff| {worst:.3e}, {launches0} launches per decode step")
    seq.close(); oracle.close()
