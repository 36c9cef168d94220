"""Tensor-parallel partition arithmetic on CPU ranks (gloo, world size 2): every rank slices whole tensors with
the library's shard plan, the shards travel through an all-gather and reassemble to the whole tensor, and the
split matmuls add up: column-split projections concatenate, K-split projections sum (what the NCCL all-reduce
does on the GPUs).  The uneven eight-way split of FFN 25600 (13,13,13,13,12,12,12,12 blocks) is checked without
a process group."""
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = dict(layers=1, hidden=512, q_heads=8, kv_heads=2, head_dim=128, ffn=1280, vocab=256, rope_base=1.0e6, rms_eps=1.0e-6)
SHAPES = {"attn_q": (1024, 512), "attn_k": (256, 512), "attn_v": (256, 512), "attn_output": (512, 1024),
          "ffn_gate": (1280, 512), "ffn_up": (1280, 512), "ffn_down": (512, 1280), "attn_norm": (1, 512)}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, out):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import ribn_b200
    dist.init_process_group("gloo")
    rng = np.random.default_rng(5)                       # the same whole tensors on every rank
    whole = {n: rng.normal(0, 1, size=s).astype(np.float32) for n, s in SHAPES.items()}
    x = rng.normal(0, 1, size=512).astype(np.float32)
    ok = True
    parts = {}
    for name, w in whole.items():
        r0, nr, c0, nc = ribn_b200.tp_shard(SMALL, f"blk.0.{name}.weight", w.shape[0], w.shape[1], world, rank)
        mine = np.ascontiguousarray(w[r0:r0 + nr, c0:c0 + nc])
        parts[name] = mine
        gathered = [None] * world
        dist.all_gather_object(gathered, (r0, nr, c0, nc, mine))
        back = np.zeros_like(w)
        covered = np.zeros(w.shape, dtype=np.int32)
        for g0, gn, h0, hn, piece in gathered:
            back[g0:g0 + gn, h0:h0 + hn] = piece
            covered[g0:g0 + gn, h0:h0 + hn] += 1
        replicated = nr == w.shape[0] and nc == w.shape[1]
        ok = ok and np.array_equal(back, w) and (np.all(covered == world) if replicated else np.all(covered == 1))
    # the layer's data flow on the shards: q | k | v and gate | up are column splits, o and down K splits + all-reduce
    q = parts["attn_q"] @ x                               # this rank's heads
    o_partial = torch.from_numpy(parts["attn_output"] @ q)
    dist.all_reduce(o_partial)
    ok = ok and np.allclose(o_partial.numpy(), whole["attn_output"] @ (whole["attn_q"] @ x), rtol=1e-4, atol=1e-3)
    act = (parts["ffn_gate"] @ x) * (parts["ffn_up"] @ x)
    d_partial = torch.from_numpy(parts["ffn_down"] @ act)
    dist.all_reduce(d_partial)
    want = whole["ffn_down"] @ ((whole["ffn_gate"] @ x) * (whole["ffn_up"] @ x))
    ok = ok and np.allclose(d_partial.numpy(), want, rtol=1e-4, atol=1e-2)
    out.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_shards_reassemble_and_split_matmuls_add_up_on_two_ranks(built_library):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]


def test_uneven_eight_way_split_of_the_32b_ffn(built_library):
    import ribn_b200
    model = ribn_b200.QWEN3_32B
    col0, widths = [], []
    for rank in range(8):
        r0, nr, c0, nc = ribn_b200.tp_shard(model, "blk.7.ffn_down.weight", 5120, 25600, 8, rank)
        assert (r0, nr) == (0, 5120) and c0 % 256 == 0 and nc % 256 == 0
        g0, gn, h0, hn = ribn_b200.tp_shard(model, "blk.7.ffn_gate.weight", 25600, 5120, 8, rank)
        assert (g0, gn, h0, hn) == (c0, nc, 0, 5120)                       # gate / up rows match down's columns
        col0.append(c0); widths.append(nc // 256)
    assert widths == [13, 13, 13, 13, 12, 12, 12, 12]
    assert col0 == list(np.cumsum([0] + [w * 256 for w in widths[:-1]]))
    # heads: 64 q / 8 kv over eight ranks = 8 q heads and 1 kv head each; o_proj splits K on 1024-column boundaries
    assert ribn_b200.tp_shard(model, "blk.0.attn_q.weight", 8192, 5120, 8, 3) == (3072, 1024, 0, 5120)
    assert ribn_b200.tp_shard(model, "blk.0.attn_k.weight", 1024, 5120, 8, 3) == (384, 128, 0, 5120)
    assert ribn_b200.tp_shard(model, "blk.0.attn_output.weight", 5120, 8192, 8, 3) == (0, 5120, 3072, 1024)
    for name, shape in (("token_embd.weight", (151936, 5120)), ("output.weight", (151936, 5120)),
                        ("blk.0.attn_norm.weight", (1, 5120)), ("output_norm.weight", (1, 5120))):
        assert ribn_b200.tp_shard(model, name, shape[0], shape[1], 8, 5) == (0, shape[0], 0, shape[1])   # replicated
    import pytest
    with pytest.raises(ValueError):
        ribn_b200.tp_shard(dict(model, kv_heads=6), "blk.0.attn_k.weight", 768, 5120, 8, 0)
