"""The bench's multi-rank plumbing on two CPU ranks (gloo): replicas shard by request with no
data-path collective, rank timings are reduced with MAX, and the whole-job figure is every rank's
tokens over the slowest rank's time."""
import os
import socket
import sys

import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, out):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    import bench
    r, w, local, dist = bench.dist_setup(world, backend="gloo")
    assert (r, w, local) == (rank, world, rank)
    bench.barrier(dist, local)
    seconds = 2.0 + rank                      # rank 1 is the slow replica
    slowest = bench.all_max(dist, seconds, local)
    value = bench.replica_throughput(dist, w, rows=64, steps=10, seconds=seconds, device=local)
    bench.barrier(dist, local)
    out.put((rank, slowest, value))
    dist.destroy_process_group()


def test_two_ranks_reduce_to_the_slowest_replica():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, slowest, value in results:
        assert slowest == 3.0
        assert abs(value - 2 * 64 * 10 / 3.0) < 1e-9


def test_single_process_needs_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    for key in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(key, None)
    rank, world, local, dist = bench.dist_setup(1)
    assert (rank, world, local, dist) == (0, 1, 0, None)
    assert bench.all_max(None, 1.5, 0) == 1.5
    assert bench.replica_throughput(None, 1, rows=1, steps=30, seconds=0.1, device=0) == 300.0
