#!/usr/bin/env python
"""Decode benchmark: Qwen3-8B-architecture, Q4_K_M-style GGUF weights, paged F16 KV.

One "step" is one decode step of the whole batch through the executor's public
protocol (prepare -> submit -> poll).  Metric: decode tok/s per GPU at batch 1
(`value`) and batch 64 (`batch64`), with the step's fraction of the HBM
roofline (bytes of quantised weights + KV read per step over measured HBM
bandwidth).  Weights are seeded N(0, 0.02) quantised on the device; token ids
and cached K/V are seeded synthetic; every step streams 4.9 GB of weights, far
beyond L2, so no explicit L2 flush is needed between steps.

The default line also carries a bounded serving leg (Poisson arrivals below saturation through the
engine: p50 / p95 time to first token and inter-token latency) and the reduced Gemma-4 job.

`--impl reference` times the reference's host CPU decoder (restated in
oracle/oracle.c; the Rust original cannot be built here) on the same weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    "qwen3-8b": dict(layers=36, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=12288, vocab=151936,
                     rope_base=1.0e6, rms_eps=1.0e-6),
    "qwen3-0.6b": dict(layers=28, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, ffn=3072, vocab=151936,
                       rope_base=1.0e6, rms_eps=1.0e-6),
    # profiling aid: Qwen3-8B layer and head shapes, 4 layers (fits an ncu capture's size rule)
    "qwen3-8b-4l": dict(layers=4, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=12288, vocab=151936,
                        rope_base=1.0e6, rms_eps=1.0e-6),
    "qwen3-32b": dict(layers=64, hidden=5120, q_heads=64, kv_heads=8, head_dim=128, ffn=25600, vocab=151936,
                      rope_base=1.0e6, rms_eps=1.0e-6),
    "tiny": dict(layers=2, hidden=512, q_heads=8, kv_heads=2, head_dim=128, ffn=1024, vocab=2048,
                 rope_base=1.0e6, rms_eps=1.0e-6),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML in this process (reads only), or
    an `nvidia-smi` loop when NVML cannot be opened."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None
        self.nvml, self.handle, self.stop = None, None, threading.Event()

    def _nvml_open(self):
        """NVML in this process (reads only): samples every few milliseconds from the first instant of the timed region."""
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            physical = int(ids[self.index]) if ids and all(v.isdigit() for v in ids) and self.index < len(ids) else self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.nvml = pynvml
            return True
        except Exception:
            self.nvml = None
            return False

    def _nvml_sample(self):
        n = self.nvml
        mhz = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
        try:
            bits = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        flag = lambda b: "Active" if bits & b else "Not Active"
        # order of the fields after the two clocks: hw_slowdown, hw_thermal_slowdown, sw_thermal_slowdown, sw_power_cap
        self.samples.append([str(mhz), str(self.max_mhz), flag(0x8), flag(0x40), flag(0x20), flag(0x4)])

    def _nvml_loop(self):
        while not self.stop.is_set():
            try:
                self._nvml_sample()
            except Exception:
                return
            self.stop.wait(0.005)

    def __enter__(self):
        if self._nvml_open():
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.nvml is not None:
            self.stop.set()
            self.thread.join(timeout=1)
            if not self.samples:
                try:
                    self._nvml_sample()  # a region shorter than one polling interval: the clock right at its end
                except Exception:
                    pass
            return
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in self.samples), "sm_max_mhz": int(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}


def dist_setup(n_gpus: int, backend: str = "nccl"):
    """One process per GPU (torchrun's RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*).  Replicas exchange
    nothing on the data path; the process group only carries the barrier and the max-over-ranks of
    the timings.  `backend="gloo"` runs the same plumbing on CPU ranks (host-side tests)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch
        import torch.distributed as dist
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
        return rank, world, local, dist
    return rank, world, local, None


def _on_gpu(dist) -> bool:
    return dist is not None and dist.get_backend() == "nccl"


def all_max(dist, value: float, device: int) -> float:
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=f"cuda:{device}" if _on_gpu(dist) else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(dist, device: int):
    if dist is not None:
        dist.barrier()
        if _on_gpu(dist):
            import torch
            torch.cuda.synchronize(device)


def replica_throughput(dist, world: int, rows: int, steps: int, seconds: float, device: int) -> float:
    """Whole-job tokens per second of `world` independent replicas: all ranks' tokens over the slowest rank's time."""
    return world * rows * steps / all_max(dist, seconds, device)


EXTRA_FLAGS = 0      # set from --operand-cache: ribn_b200.FLAG_OPERAND_CACHE on every Qwen executor of the run
SCHEME = "q4_k_m"   # set from --scheme: "q4_k_m" (Q4_K; Q6_K for attn_v, ffn_down, output) or "q8_0"


def build_executor(model: dict, batch: int, context: int, decode_tokens: int, device: int, keep_logits: bool):
    import ribn_b200
    span = context + decode_tokens + 16
    ex = ribn_b200.QwenB200(model, context_tokens=span, max_sequences=batch, max_batch_tokens=max(batch, 16),
                            device=device, flags=(ribn_b200.FLAG_KEEP_LOGITS if keep_logits else 0) | EXTRA_FLAGS)
    ex.init_synthetic(0x5EED, ribn_b200.SCHEME_Q8_0 if SCHEME == "q8_0" else ribn_b200.SCHEME_Q4_K_M)
    return ex


def seed_sequences(ex, model: dict, batch: int, context: int, decode_tokens: int, seed: int):
    rng = np.random.default_rng(seed)
    for s in range(batch):
        prompt = rng.integers(0, model["vocab"], size=context, dtype=np.uint32)
        adm = ex.admit(s + 1, s + 1, prompt, decode_tokens + 8)
        if not adm.ready:
            raise RuntimeError(f"admission failed: {adm}")
        ex.debug_set_context(s + 1, context, int(rng.integers(0, model["vocab"])), seed=seed * 1000 + s)


def decode_steps(ex, sequences, positions, steps: int):
    """Runs `steps` decode steps over `sequences`; returns (wall seconds, [device ms], launches)."""
    from ribn_b200 import BatchItem, StepKind
    device_ms, launches = [], 0
    ex.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        items = [BatchItem(s, StepKind.DECODE, positions[s], 1, 1) for s in sequences]
        ex.prepare(items)
        done = ex.wait(ex.submit(items))          # H2D of the row records and D2H of the sampled tokens inside
        for row in done:
            positions[row.sequence] = row.prefix
        ms, n = ex.last_step_stats()
        device_ms.append(ms)
        launches += n
    ex.synchronize()
    return time.perf_counter() - t0, device_ms, launches


def oracle_for(ex, model: dict, context_capacity: int):
    from oracle import binding as orc
    tensors = {name: ex.read_tensor(name) for name in ex.tensor_names()}
    cfg = dict(model, context=context_capacity, eps=model["rms_eps"])
    cfg.pop("rms_eps")
    return orc, orc.Qwen3Oracle(cfg, tensors)


def oracle_sequence(orc, oracle, ex, model, sequence: int, context: int):
    seq = oracle.new_sequence()
    row = model["kv_heads"] * model["head_dim"]
    keys = np.empty((model["layers"], context * row), dtype=np.uint16)
    values = np.empty_like(keys)
    for l in range(model["layers"]):
        keys[l] = ex.copy_kv(sequence, l, 0, context)
        values[l] = ex.copy_kv(sequence, l, 1, context)
    seq.fill(keys, values, context)
    return seq


# dram__bytes_read.sum + dram__bytes_write.sum of one ffn gate|up launch of gemv_mma_kernel, from an ncu
# capture of this kernel on the 4-layer model (the per-layer launch is the same at 36 layers).
GATE_UP_DRAM_BYTES = {"qwen3-8b": 56843264, "qwen3-8b-4l": 56843264}
REPEATS = 5   # the headline is the median over this many blocks of --steps steps


def decode_workload(args, batch: int) -> dict:
    """The `config` object of the decode workload: the same for both arms."""
    return {"workload": f"{args.model} {args.scheme.upper()}-style decode, batch 1 and {batch}, context {args.context}, "
                        f"16-token KV pages, one replica per GPU",
            "l2": "inputs larger than L2 (4.9 GB of weights streamed per step)",
            "operand_cache": bool(EXTRA_FLAGS)}


def run_ours(args):
    rank, world, local, dist = dist_setup(args.gpus)
    import ribn_b200
    model = MODELS[args.model]
    B = args.batch
    total_steps = REPEATS * args.steps + args.warmup + 2
    ex = build_executor(model, B, args.context, 2 * total_steps + 4, local, keep_logits=True)
    ex.finalize()
    seed_sequences(ex, model, B, args.context, 2 * total_steps + 4, seed=1 + rank)
    positions = {s + 1: args.context for s in range(B)}
    hbm_gbs, peak_kind = measured_peaks()

    # ---- CPU baseline + full-size parity on rank 0, one GPU only --------------------------
    cpu = None
    parity = None
    if rank == 0 and world == 1 and not args.no_cpu:
        orc, oracle = oracle_for(ex, model, args.context + 8)
        cores = os.cpu_count() or 1
        orc.set_threads(cores)
        seq = oracle_sequence(orc, oracle, ex, model, 1, args.context)
        from ribn_b200 import BatchItem, StepKind
        # the device's pending input token for sequence 1 is reproduced from the seeding rule
        rng = np.random.default_rng(1 + rank)
        rng.integers(0, model["vocab"], size=args.context, dtype=np.uint32)
        token = int(rng.integers(0, model["vocab"]))
        item = BatchItem(1, StepKind.DECODE, positions[1], 1, 1)
        ex.prepare([item])
        done = ex.wait(ex.submit([item]))
        positions[1] = done[0].prefix
        got = ex.copy_logits(0)
        t0 = time.perf_counter()
        want = seq.step(token)
        cpu_s = time.perf_counter() - t0
        err = np.abs(got - want)
        parity = {"max_abs_logit_diff": float(err.max()), "argmax_equal": bool(orc.argmax(want) == done[0].tokens[0]),
                  "tolerance": "max-abs 2e-2 / rel 1e-2", "checked": "1 decode step at full size here; 256 greedy tokens and a "
                  "batch-64 step at full size in tests/test_gpu_fullsize.py",
                  "oracle": "CPU restatement pinned primitive by primitive; the reference has no end-to-end vector for dense Qwen3"}
        cpu = {"value": 1.0 / cpu_s, "unit": "tok/s", "cores": cores, "kind": "port",
               "sample": f"1 decode token at batch 1, context {args.context}, {args.model} {args.scheme.upper()}-style, "
                         f"oracle/oracle.c with OpenMP over output rows"}
        # the reference's CPU decoder is single-threaded: the same token step on one thread
        orc.set_threads(1)
        t0 = time.perf_counter()
        seq.step(orc.argmax(want))
        cpu["single_thread"] = {"value": 1.0 / (time.perf_counter() - t0), "unit": "tok/s", "cores": 1,
                                "sample": "the next decode token of the same sequence on one thread"}
        orc.set_threads(cores)
        seq.close(); oracle.close()

    def phase(sequences, repeats):
        """`repeats` blocks of exactly --steps steps, each bracketed by a barrier and timed on the device as the
        maximum over ranks; the reported block is the median one (by device time)."""
        decode_steps(ex, sequences, positions, args.warmup)
        blocks = []
        with ClockSampler(local) as clocks:
            for _ in range(repeats):
                barrier(dist, local)
                wall, device_ms, launches = decode_steps(ex, sequences, positions, args.steps)
                barrier(dist, local)
                blocks.append((all_max(dist, sum(device_ms) / 1e3, local), all_max(dist, wall, local), launches))
        blocks.sort()
        dev, wall, launches = blocks[len(blocks) // 2]
        spread = {"repeats": repeats, "ms_per_step_min": blocks[0][0] / args.steps * 1e3,
                  "ms_per_step_max": blocks[-1][0] / args.steps * 1e3}
        return wall, dev, launches, clocks.summary(), spread

    def step_roofline(batch_rows, dev_seconds):
        """Whole step: algorithmic bytes of one decode step over its device time (every kernel included)."""
        ctx_avg = args.context + args.warmup + REPEATS * args.steps / 2.0
        w_bytes, kv_bytes = ex.step_bytes(int(batch_rows * ctx_avg))
        per_step = w_bytes + kv_bytes
        achieved = per_step / (dev_seconds / args.steps) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                "of": peak_kind, "algorithmic_bytes_per_step": per_step, "weight_bytes": w_bytes, "kv_bytes": kv_bytes}

    def kernel_roofline():
        """The dominant kernel (gemv_mma_kernel: every projection of a batch-1 step) over ALL its launches of one
        step: encoded weight bytes of the 4 x layers + 1 launches over the sum of their CUDA-event durations, each
        launch kind timed live here on the executor's stream with weights streamed from HBM."""
        L = model["layers"]
        kinds = {}
        for name in ("qkv", "attn_output", "gate_up", "down", "head"):
            t_us, b = ex.time_projection(name, repeats=(8 if name == "head" else 2 * L))
            count = 1 if name == "head" else L
            kinds[name] = {"us": t_us, "bytes": b, "GB/s": b / t_us / 1e3, "frac": b / t_us / 1e3 / hbm_gbs,
                           "launches_per_step": count}
        total_bytes = sum(k["bytes"] * k["launches_per_step"] for k in kinds.values())
        total_us = sum(k["us"] * k["launches_per_step"] for k in kinds.values())
        launches = sum(k["launches_per_step"] for k in kinds.values())
        achieved = total_bytes / total_us / 1e3
        traffic = GATE_UP_DRAM_BYTES.get(args.model) if args.scheme == "q4_k_m" else None
        return {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                "traffic": traffic, "traffic_of": "one ffn gate|up launch (ncu dram bytes; its algorithmic bytes are "
                                                  f"{kinds['gate_up']['bytes']})",
                "of": peak_kind,
                "kernel": f"gemv_mma_kernel, byte-weighted over its {launches} launches of one batch-1 step",
                "algorithmic_bytes_per_launch": total_bytes / launches, "us_per_launch": total_us / launches,
                "algorithmic_bytes_per_step": total_bytes, "us_per_step": total_us, "other_launches": kinds}

    # ---- batch 1 -----------------------------------------------------------------------
    wall1, dev1, launches1, clocks1, spread1 = phase([1], REPEATS)
    value1 = world * 1 * args.steps / dev1   # dev1 / wall1 are already the maximum over ranks
    e2e1 = world * 1 * args.steps / wall1
    out = {
        "metric": f"{args.model} {args.scheme.upper()} decode tok/s at batch 1 (per GPU x replicas)", "value": value1,
        "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev1 / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": f"u8 x s8 integer tensor-core products over {'Q8_0' if args.scheme == 'q8_0' else 'Q4_K,Q6_K'} weights, f32 block scales and accumulation, f16 KV",
        "data": "synthetic",
        "config": dict(decode_workload(args, B), parallelism=f"replicas x{world}"),
        "e2e": {"value": e2e1, "unit": "tok/s", "h2d_bytes_per_step": 32, "d2h_bytes_per_step": 4},
        "gpu_launches": launches1, "roofline": kernel_roofline(), "step_roofline": step_roofline(1, dev1),
        "clocks": clocks1, "spread": spread1,
    }
    if cpu:
        out["cpu_baseline"] = cpu
        out["parity"] = parity
    # ---- batch B -------------------------------------------------------------------------
    if B > 1:
        wallb, devb, launchesb, clocksb, spreadb = phase(list(range(1, B + 1)), 3)
        out["batch64"] = {"batch": B, "value": world * B * args.steps / devb, "unit": "tok/s",
                          "ms_per_step": devb / args.steps * 1e3,
                          "e2e": {"value": world * B * args.steps / wallb, "unit": "tok/s",
                                  "h2d_bytes_per_step": 32 * B, "d2h_bytes_per_step": 4 * B},
                          "gpu_launches": launchesb, "step_roofline": step_roofline(B, devb), "clocks": clocksb,
                          "spread": spreadb,
                          "x_batch1": (world * B * args.steps / devb) / value1}
    ex.close()
    if B >= 3 and not EXTRA_FLAGS and not args.no_cache_leg and args.scheme == "q4_k_m":
        # the same batch once more on an executor that keeps the K-quant matrices as tensor-core operands
        # (RIBN_B200_FLAG_OPERAND_CACHE: 2 or 4 bytes of HBM per weight; same logits bit for bit)
        # An extra: if the larger executor cannot be built on some rank (memory taken by someone else), every rank
        # skips the leg together and the line says so.
        ex, problem = None, ""
        try:
            ex = ribn_b200.QwenB200(model, context_tokens=args.context + 2 * total_steps + 20, max_sequences=B,
                                    max_batch_tokens=max(B, 16), device=local, flags=ribn_b200.FLAG_OPERAND_CACHE)
            ex.init_synthetic(0x5EED, ribn_b200.SCHEME_Q4_K_M)
            ex.finalize()
            seed_sequences(ex, model, B, args.context, 2 * total_steps + 4, seed=1 + rank)
        except Exception as exc:   # noqa: BLE001
            problem = str(exc) or type(exc).__name__
        if all_max(dist, 1.0 if problem else 0.0, local) > 0.0:
            out["batch64"]["operand_cache"] = {"unavailable": problem or "another rank could not build the executor"}
        else:
            positions = {s + 1: args.context for s in range(B)}
            _, devc, launchesc, _, spreadc = phase(list(range(1, B + 1)), 3)
            out["batch64"]["operand_cache"] = {"value": world * B * args.steps / devc, "unit": "tok/s",
                                               "ms_per_step": devc / args.steps * 1e3, "gpu_launches": launchesc,
                                               "spread": spreadc,
                                               "note": "K-quant matrices also kept as binary16 operand planes (Q4_K 2 B, Q6_K 4 B per weight)"}
        if ex is not None:
            try:
                ex.close()
            except Exception:   # noqa: BLE001
                pass
    if not args.no_serving:
        # p50 time to first token is part of the metric: a bounded serving leg below saturation
        srv = serving_job(args, rank, world, local, dist, n=args.serving_requests, rate=args.arrival_rate_default,
                          workload="serving")
        out["ttft_ms"], out["itl_ms"] = srv["ttft_ms"], srv["itl_ms"]
        out["serving"] = {k: srv[k] for k in ("value", "unit", "prompt_tokens", "generated_tokens", "makespan_s", "clocks")}
        out["serving"]["workload"] = srv["config"]["workload"]
    if world == 1 and not args.no_cpu and not args.no_gemma:
        # the reference's CPU-runnable configuration, as a second workload of the same library
        out["gemma_reduced"] = gemma_job(args, rank, world, local, dist, 3, 3, True)
    if rank == 0:
        print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


def run_prefill(args):
    """`--workload prefill`: one prompt of --context tokens prefilled in 2048-token chunks, per replica; device time of
    every chunk (the executor's own CUDA events), repeated --steps times after --warmup prompts."""
    import ribn_b200
    from ribn_b200 import BatchItem, StepKind
    rank, world, local, dist = dist_setup(args.gpus)
    model = MODELS[args.model]
    chunk = 2048
    length = max(chunk, args.context // chunk * chunk)
    ex = ribn_b200.QwenB200(model, context_tokens=length + 16, max_sequences=2, max_batch_tokens=chunk, device=local, flags=EXTRA_FLAGS)
    ex.init_synthetic(0x5EED, ribn_b200.SCHEME_Q8_0 if SCHEME == "q8_0" else ribn_b200.SCHEME_Q4_K_M)
    ex.finalize()
    rng = np.random.default_rng(7 + rank)
    chunks = length // chunk
    per_chunk = np.zeros((args.steps, chunks))
    launches = 0
    barrier(dist, local)
    with ClockSampler(local) as clocks:
        wall0 = None
        for rep in range(args.warmup + args.steps):
            if rep == args.warmup:
                barrier(dist, local)
                wall0 = time.perf_counter()
            prompt = rng.integers(0, model["vocab"], size=length, dtype=np.uint32)
            assert ex.admit(100 + rep, 100 + rep, prompt, 2).ready
            for c in range(chunks):
                item = BatchItem(100 + rep, StepKind.PREFILL, c * chunk, chunk, 1 if c == chunks - 1 else 0)
                ex.prepare([item])
                ex.wait(ex.submit([item]))
                ms, n = ex.last_step_stats()
                if rep >= args.warmup:
                    per_chunk[rep - args.warmup, c] = ms
                    launches += n
            ex.release(100 + rep)
        barrier(dist, local)
        wall = time.perf_counter() - wall0
    ex.close()
    dev = all_max(dist, float(per_chunk.sum()) / 1e3, local)
    wall = all_max(dist, wall, local)
    tokens = world * args.steps * length
    out = {
        "metric": f"{args.model} {args.scheme.upper()} prefill prompt tok/s (per GPU x replicas)", "value": tokens / dev,
        "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": f"f16 x f16 tensor-core products over exact {'Q8_0 values' if args.scheme == 'q8_0' else 'K-quant integers'}, f32 scales and accumulation, f16 KV",
        "data": "synthetic",
        "config": {"workload": f"{args.model} {args.scheme.upper()}-style prefill of one {length}-token prompt per step in {chunk}-token chunks, "
                               f"16-token KV pages, one replica per GPU", "l2": "inputs larger than L2", "parallelism": f"replicas x{world}",
                   "operand_cache": bool(EXTRA_FLAGS)},
        "e2e": {"value": tokens / wall, "unit": "tok/s", "h2d_bytes_per_step": 4 * length, "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "chunk_ms": [float(v) for v in np.median(per_chunk, axis=0)],
        "clocks": clocks.summary(),
    }
    if rank == 0:
        print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


def run_serving(args):
    """`--workload serving|mixed`: the serving job alone, one line."""
    rank, world, local, dist = dist_setup(args.gpus)
    out = serving_job(args, rank, world, local, dist, n=args.requests, rate=args.arrival_rate, workload=args.workload)
    if rank == 0:
        print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


def serving_job(args, rank, world, local, dist, n, rate, workload):
    """Continuous batching through the engine (scheduling rules of the reference's Engine restated in
    ribn_b200/engine.py).  serving: Poisson arrivals, prompts ~U[128, 2048], outputs ~U[64, 512], up to 64 active
    requests, 2048-token prefill chunks, 16-token KV pages.  mixed: 32 long prompts (log-uniform 512 .. 16384,
    chunk 2048) interleaved with 32 decode-heavy requests at context 1024 .. 4096, all queued at time zero.
    Reports whole-job generated tok/s, the time to first token (planned arrival -> first token, as the
    reference's serving bench measures it) and the gaps between a request's successive tokens."""
    import ribn_b200
    from ribn_b200.engine import Engine, EngineConfig, SchedulePolicy, TokenRequest
    model = MODELS[args.model]
    rng = np.random.default_rng(0xC3 + rank)
    if workload == "mixed":
        long_n = n // 2
        prompt_hi = args.serving_prompt_max if args.serving_prompt_max > 2048 else 16384
        prompts = np.concatenate([np.exp(rng.uniform(np.log(512), np.log(prompt_hi), size=long_n)).astype(np.int64),
                                  rng.integers(1024, 4097, size=n - long_n)])
        outputs = np.concatenate([np.full(long_n, 8), np.full(n - long_n, min(256, args.serving_output_max))])
        order = rng.permutation(n)
        prompts, outputs = prompts[order], outputs[order]
        arrivals = np.zeros(n)
        described = (f"{long_n} prompts log-uniform [512,{prompt_hi}] (8 outputs) interleaved with {n - long_n} decode-heavy "
                     f"requests (context U[1024,4096], {int(outputs.max())} outputs), all queued at time zero")
    else:
        prompt_hi = min(2048, args.serving_prompt_max)
        prompts = rng.integers(min(128, prompt_hi), prompt_hi + 1, size=n)
        outputs = rng.integers(min(64, args.serving_output_max), args.serving_output_max + 1, size=n)
        arrivals = np.cumsum(rng.exponential(1.0 / rate, size=n))
        described = (f"Poisson arrivals {rate}/s, prompts U[{min(128, prompt_hi)},{prompt_hi}], outputs "
                     f"U[{min(64, args.serving_output_max)},{args.serving_output_max}]")
    active = min(64, n)
    chunk = min(2048, int(prompts.max()))
    pages = int(sum((int(p) + int(o) + 15) // 16 for p, o in zip(prompts, outputs))) + active
    ex = ribn_b200.QwenB200(model, context_tokens=int((prompts + outputs).max() + 16), max_sequences=active,
                            max_batch_tokens=chunk + active, kv_pages=pages, device=local, flags=EXTRA_FLAGS)
    ex.init_synthetic(0x5EED, ribn_b200.SCHEME_Q8_0 if SCHEME == "q8_0" else ribn_b200.SCHEME_Q4_K_M)
    ex.finalize()
    native = getattr(args, "engine", "python") == "native"
    if native:
        from ribn_b200.native_engine import NativeEngine as Engine   # the C++ engine of include/ribn_b200_engine.h
    engine = Engine(ex, EngineConfig(max_active_requests=active, max_queued_requests=n),
                    SchedulePolicy(max_batch_tokens=chunk + active, prefill_chunk_tokens=chunk, decode_tokens=1,
                                   max_decode_only_steps=8))
    tokens = [rng.integers(0, model["vocab"], size=int(p), dtype=np.uint32) for p in prompts]
    barrier(dist, local)
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        nxt, ids = 0, {}
        while nxt < n or not engine.idle():
            now = time.perf_counter() - t0
            while nxt < n and arrivals[nxt] <= now:
                ids[engine.enqueue(TokenRequest(tokens[nxt], int(outputs[nxt])))] = nxt
                nxt += 1
            if not engine.step():
                time.sleep(50e-6 if engine.in_flight else min(1e-3, max(0.0, arrivals[nxt] - now)) if nxt < n else 50e-6)
        ex.synchronize()
        makespan = time.perf_counter() - t0
    barrier(dist, local)
    ttft, itl, generated = [], [], 0
    if native:
        finished = {rid: list(engine.token_times(rid)) for rid in ids}
    else:
        finished = {rid: slot.token_times for rid, slot in engine.finished.items()}
    for rid, token_times in finished.items():
        i = ids[rid]
        generated += len(token_times)
        if token_times:
            ttft.append(token_times[0] - t0 - arrivals[i])
            itl.extend(np.diff(token_times).tolist())
    makespan = all_max(dist, makespan, local)
    out = {
        "metric": f"{args.model} {args.scheme.upper()} continuous-batching generated tok/s (per GPU x replicas)",
        "value": world * generated / makespan, "unit": "tok/s", "n_gpus": world, "steps": engine.steps, "warmup": 0,
        "ms_per_step": makespan / max(engine.steps, 1) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": f"u8 x s8 / f16 tensor-core products over {'Q8_0' if args.scheme == 'q8_0' else 'Q4_K,Q6_K'} weights, f32 scales and accumulation, f16 KV",
        "data": "synthetic",
        "config": {"workload": f"{args.model} {args.scheme.upper()}-style {workload}: {n} requests per GPU, {described}, {active} active, "
                               f"{chunk}-token prefill chunks, 16-token KV pages",
                   "parallelism": f"replicas x{world}", "operand_cache": bool(EXTRA_FLAGS),
                   "engine": "native" if native else "python"},
        "ttft_ms": {"p50": float(np.percentile(ttft, 50) * 1e3), "p95": float(np.percentile(ttft, 95) * 1e3),
                    "definition": "planned arrival -> first token", "arrival_rate_per_s": rate if workload != "mixed" else None,
                    "requests": n},
        "itl_ms": {"p50": float(np.percentile(itl, 50) * 1e3), "p95": float(np.percentile(itl, 95) * 1e3)} if itl else None,
        "prompt_tokens": int(prompts.sum()), "generated_tokens": int(generated), "makespan_s": makespan,
        "clocks": clocks.summary(),
    }
    ex.close()
    return out


def run_tp(args):
    """Tensor-parallel decode (`--tp N`, one rank per GPU): the Qwen3-32B-class configuration.  Every rank holds one
    shard of each layer (heads for q | k | v, columns for gate | up, K blocks for the attention output and ffn down
    projections, kv heads for the cache) and the replicated head; the ranks' partial sums meet in an NCCL
    all-reduce after o_proj and down_proj.  All ranks run the same schedule: `--batch` sequences at contexts
    U[512, --context-max], one decode token per step.  Strong scaling: the model is fixed, N grows."""
    rank, world, local, dist = dist_setup(args.gpus)
    import torch
    import ribn_b200
    if world != args.tp:
        raise SystemExit(f"--tp {args.tp} needs {args.tp} ranks (torchrun --nproc-per-node {args.tp}), got {world}")
    model = MODELS[args.model]
    B = args.batch
    rng = np.random.default_rng(0xC5)                         # the same on every rank
    contexts = rng.integers(512, args.context_max + 1, size=B)
    steps_total = args.warmup + REPEATS * args.steps + 4
    span = int(contexts.max()) + steps_total + 16
    pages = int(sum((int(c) + steps_total + 16 + 15) // 16 for c in contexts)) + B
    ex = ribn_b200.QwenB200(model, context_tokens=span, max_sequences=B, max_batch_tokens=max(B, 16), kv_pages=pages,
                            device=local, flags=EXTRA_FLAGS, tp_size=world, tp_rank=rank)
    ex.init_synthetic(0x5EED, ribn_b200.SCHEME_Q8_0 if SCHEME == "q8_0" else ribn_b200.SCHEME_Q4_K_M)
    ids = [ribn_b200.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    ex.tp_init(ids[0])
    ex.finalize()
    positions = {}
    for s in range(B):
        prompt = rng.integers(0, model["vocab"], size=int(contexts[s]), dtype=np.uint32)
        adm = ex.admit(s + 1, s + 1, prompt, steps_total + 8)
        if not adm.ready:
            raise RuntimeError(f"admission failed: {adm}")
        ex.debug_set_context(s + 1, int(contexts[s]), int(rng.integers(0, model["vocab"])), seed=5000 + s)
        positions[s + 1] = int(contexts[s])
    sequences = list(range(1, B + 1))
    hbm_gbs, peak_kind = measured_peaks()
    decode_steps(ex, sequences, positions, args.warmup)
    blocks = []
    with ClockSampler(local) as clocks:
        for _ in range(REPEATS):
            barrier(dist, local)
            wall, device_ms, launches = decode_steps(ex, sequences, positions, args.steps)
            barrier(dist, local)
            blocks.append((all_max(dist, sum(device_ms) / 1e3, local), all_max(dist, wall, local), launches))
    blocks.sort()
    dev, wall, launches = blocks[len(blocks) // 2]
    ar_us = ex.tp_time_allreduce(B, 50)
    w_bytes, kv_bytes = ex.step_bytes(int(contexts.sum()) + B * (args.warmup + REPEATS * args.steps // 2))
    step_s = dev / args.steps
    achieved = (w_bytes + kv_bytes) / step_s / 1e9
    out = {
        "metric": f"{args.model} {args.scheme.upper()} tensor-parallel decode tok/s (whole job, tp{world})",
        "value": B * args.steps / dev, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 x f16 tensor-core products over exact K-quant integers, f32 scales and accumulation, f16 KV, f32 all-reduce",
        "data": "synthetic",
        "config": {"workload": f"{args.model} {args.scheme.upper()}-style decode, {B} concurrent sequences, contexts U[512,{args.context_max}], "
                               f"16-token KV pages, tensor parallel over {world} GPUs (NCCL all-reduce after o_proj and down_proj)",
                   "l2": "inputs larger than L2", "parallelism": f"tp{world}", "operand_cache": bool(EXTRA_FLAGS)},
        "e2e": {"value": B * args.steps / wall, "unit": "tok/s", "h2d_bytes_per_step": 32 * B, "d2h_bytes_per_step": 4 * B},
        "gpu_launches": launches, "clocks": clocks.summary(),
        "per_rank": {"weight_bytes": w_bytes, "kv_bytes_per_step": kv_bytes,
                     "step_roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s",
                                       "frac": achieved / hbm_gbs, "of": peak_kind}},
        "all_reduce": {"us": ar_us, "per_step": 2 * model["layers"], "bytes": B * model["hidden"] * 4,
                       "share_of_step": 2 * model["layers"] * ar_us * 1e-6 / step_s},
        "spread": {"repeats": REPEATS, "ms_per_step_min": blocks[0][0] / args.steps * 1e3,
                   "ms_per_step_max": blocks[-1][0] / args.steps * 1e3},
    }
    ex.close()
    if rank == 0:
        print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


def run_gemma(args):
    """The reduced Gemma-4 configuration (6 layers: 5 sliding-512 + 1 full; hidden 1152; 4 q / 1 kv heads of 256;
    GeGLU 6912; vocab 32768; BF16 random-init N(0, 0.02)): four prompts of 17 / 64 / 129 / 300 uniform-random
    ids, 32 greedy tokens each, through the executor protocol with all four sequences batched.  A step is one
    whole job.  The CPU figure is the host decoder restated in oracle/gemma.c (the reference's own CPU path for
    this configuration), timed on a bounded sample and checked token for token against the GPU."""
    rank, world, local, dist = dist_setup(args.gpus)
    out = gemma_job(args, rank, world, local, dist, args.steps, args.warmup, not args.no_cpu)
    if rank == 0:
        print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


def gemma_job(args, rank, world, local, dist, steps, warmup, with_cpu):
    """Runs the reduced Gemma-4 job `steps` times and returns its result line."""
    import ribn_b200
    from ribn_b200 import BatchItem, StepKind
    cfg = ribn_b200.GEMMA4_REDUCED
    model = ribn_b200.GemmaB200(cfg, max_sequences=4, max_batch_tokens=128, device=local)
    model.init_synthetic(0x5EED)
    tensors = None
    if rank == 0 and with_cpu:
        tensors = {name: model.read_tensor(name) for name in model.tensor_names()}
    model.finalize()
    rng = np.random.default_rng(0xC1 + rank)
    prompts = {i + 1: rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate((17, 64, 129, 300))}
    new_tokens = args.gemma_new_tokens

    decode_ms = []   # device time of the last job's decode steps with all four sequences

    def job():
        ex = ribn_b200.GemmaExecutor(model)
        for seq, p in prompts.items():
            assert ex.admit(seq, seq, p, new_tokens).ready
        got = {seq: [] for seq in prompts}
        cursor = {seq: 0 for seq in prompts}
        launches, device_ms = 0, 0.0
        decode_ms.clear()
        while any(len(got[q]) < new_tokens for q in prompts):
            batch = []
            for seq, p in prompts.items():
                if len(got[seq]) >= new_tokens:
                    continue
                if cursor[seq] < len(p):
                    n = min(128 // 4, len(p) - cursor[seq])
                    batch.append(BatchItem(seq, StepKind.PREFILL, cursor[seq], n, int(cursor[seq] + n == len(p))))
                else:
                    batch.append(BatchItem(seq, StepKind.DECODE, cursor[seq], 1, 1))
            ex.prepare(batch)
            for done in ex.poll(ex.submit(batch)):
                cursor[done.sequence] = done.prefix
                got[done.sequence].extend(done.tokens)
            ms, n_launch = model.last_step_stats()
            launches += n_launch
            device_ms += ms
            if len(batch) == 4 and all(it.kind == StepKind.DECODE for it in batch):
                decode_ms.append(ms)
        ex.synchronize()
        return got, launches, device_ms

    for _ in range(warmup):
        job()
    barrier(dist, local)
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        launches = 0
        device_ms = 0.0
        for _ in range(steps):
            got, n_launch, ms = job()
            launches += n_launch
            device_ms += ms
        seconds = time.perf_counter() - t0
    barrier(dist, local)
    seconds = all_max(dist, seconds, local)
    generated = 4 * new_tokens
    prompt_tokens = sum(len(p) for p in prompts.values())
    out = {
        "metric": "reduced Gemma-4 BF16 greedy generation, generated tok/s (per GPU x replicas)",
        "value": world * generated * steps / (device_ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": seconds / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 storage, f32 arithmetic, one bf16 rounding per operation", "data": "synthetic",
        "config": {"workload": "reduced Gemma-4 (6 layers, hidden 1152, 4q/1kv x 256, GeGLU 6912, vocab 32768): prompts "
                               f"17/64/129/300, {new_tokens} greedy tokens each, four sequences batched",
                   "l2": "weights (0.41 GB) exceed L2", "parallelism": f"replicas x{world}"},
        "e2e": {"value": world * generated * steps / seconds, "unit": "tok/s",
                "h2d_bytes_per_step": 4 * (prompt_tokens + generated), "d2h_bytes_per_step": 4 * generated},
        "gpu_launches": launches, "prompt_tokens": prompt_tokens, "generated_tokens": generated,
        "clocks": clocks.summary(),
    }
    if decode_ms:
        # one decode step of the four sequences: every BF16 matrix read once (the tied head included; the per-layer
        # token table is only gathered) over the step's CUDA-event time
        H, F, ple, L = cfg["hidden"], cfg["ffn"], cfg["ple"], cfg["layers"]
        qd, kd = cfg["heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
        per_layer = 2 * qd * H + 2 * kd * H + 3 * F * H + 2 * ple * H
        weight_bytes = 2 * (L * per_layer + cfg["vocab"] * H + L * ple * H)
        step_ms = statistics.median(decode_ms)
        hbm_gbs, peak_kind = measured_peaks()
        achieved = weight_bytes / (step_ms / 1e3) / 1e9
        out["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                           "of": peak_kind, "traffic": None,
                           "kernel": "one decode step of four sequences (every kernel; gm_project_kernel is ~80 % of it)",
                           "algorithmic_bytes_per_step": weight_bytes, "ms_per_step": step_ms,
                           "note": "the projections add every FP32 sum in source order (bit parity with the host decoder), "
                                   "which bounds them by latency, not by HBM"}
    if rank == 0 and tensors is not None:
        from oracle import gemma_binding as G
        oracle = G.GemmaOracle(cfg, tensors)
        ref = oracle.new_sequence()
        t0 = time.perf_counter()
        token = G.argmax(ref.prefill(prompts[1]))
        want = [token]
        for _ in range(7):
            token = G.argmax(ref.decode(token))
            want.append(token)
        cpu_seconds = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": (len(prompts[1]) + 7) / cpu_seconds, "unit": "tok/s (prompt and generated tokens processed)",
                               "cores": os.cpu_count(), "kind": "port",
                               "sample": "the 17-token prompt and 8 greedy tokens, oracle/gemma.c with OpenMP over output columns"}
        out["parity"] = {"greedy_tokens_equal": want == got[1][:8], "checked": 8}
        out["tokens_processed_per_s"] = world * (prompt_tokens + generated) * steps / seconds
        oracle.close()
    model.close()
    return out


def run_reference(args):
    """The reference's host CPU decoder (restated: oracle/oracle.c) on the GPU box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model = MODELS[args.model]
    cores = os.cpu_count() or 1
    # The synthetic checkpoint comes from the library's device generator (not timed).
    ex = build_executor(model, 1, args.context, 8, 0, keep_logits=False)
    ex.finalize()
    seed_sequences(ex, model, 1, args.context, 8, seed=1)
    orc, oracle = oracle_for(ex, model, args.context + args.steps + args.warmup + 8)
    orc.set_threads(cores)
    seq = oracle_sequence(orc, oracle, ex, model, 1, args.context)
    ex.close()
    token = 1
    budget, t_start = 240.0, time.perf_counter()
    for _ in range(args.warmup):
        token = orc.argmax(seq.step(token))
        if time.perf_counter() - t_start > budget / 3:
            break
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        token = orc.argmax(seq.step(token))
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget:
            break
    total = sum(times)
    value = len(times) / total
    sample = (f"{len(times)} decode tokens at batch 1, context {args.context}, {args.model} Q4_K_M-style, "
              f"oracle/oracle.c (restated host decoder), OpenMP over output rows")
    print(json.dumps({
        "impl": "reference", "metric": f"{args.model} {args.scheme.upper()} decode tok/s at batch 1 (per GPU x replicas)",
        "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": total / len(times) * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": dict(decode_workload(args, args.batch), parallelism=f"replicas x{args.gpus}"),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b", choices=sorted(MODELS))
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline / full-size parity leg")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving", "mixed", "gemma", "prefill"],
                    help="decode: steady batch-1 / batch-N decode steps (the headline); serving: Poisson arrivals through the engine; "
                         "mixed: long chunked prefills interleaved with decode-heavy requests; gemma: the reduced Gemma-4 BF16 job; "
                         "prefill: one prompt of --context tokens per step in 2048-token chunks")
    ap.add_argument("--requests", type=int, default=None, help="requests per GPU (default: serving 96; mixed 64 = 32 long prompts + 32 decodes)")
    ap.add_argument("--no-serving", action="store_true", help="decode: skip the bounded serving leg (time to first token)")
    ap.add_argument("--serving-requests", type=int, default=32, help="decode: requests of the bounded serving leg")
    ap.add_argument("--arrival-rate-default", type=float, default=4.0,
                    help="decode: Poisson arrival rate of the bounded serving leg (below saturation), requests per second per GPU")
    ap.add_argument("--arrival-rate", type=float, default=8.0, help="serving: Poisson arrival rate, requests per second per GPU")
    ap.add_argument("--serving-prompt-max", type=int, default=2048)
    ap.add_argument("--serving-output-max", type=int, default=512)
    ap.add_argument("--no-gemma", action="store_true", help="decode: skip the reduced Gemma-4 job appended to the default line")
    ap.add_argument("--gemma-new-tokens", type=int, default=32, help="gemma: greedy tokens per prompt")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel group size (= ranks); runs the tensor-parallel decode workload")
    ap.add_argument("--context-max", type=int, default=8192, help="tp: contexts are uniform in [512, this]")
    ap.add_argument("--engine", default="python", choices=["python", "native"],
                    help="serving / mixed: the host engine that drives the executor (ribn_b200/engine.py or the C++ one)")
    ap.add_argument("--no-cache-leg", action="store_true", help="decode: skip the extra batch leg with the operand cache on")
    ap.add_argument("--operand-cache", default="off", choices=["on", "off"],
                    help="keep the K-quant matrices also as tensor-core operands in HBM (RIBN_B200_FLAG_OPERAND_CACHE)")
    ap.add_argument("--scheme", default="q4_k_m", choices=["q4_k_m", "q8_0"], help="synthetic checkpoint's block types")
    args = ap.parse_args()
    global SCHEME, EXTRA_FLAGS
    SCHEME = args.scheme
    if args.operand_cache == "on" and args.impl != "reference":
        import ribn_b200
        EXTRA_FLAGS = ribn_b200.FLAG_OPERAND_CACHE
    if args.warmup < 3:
        args.warmup = 3
    if args.requests is None:
        args.requests = 64 if args.workload == "mixed" else 96
    if args.impl == "reference":
        run_reference(args)
    elif args.tp > 1:
        run_tp(args)
    elif args.workload in ("serving", "mixed"):
        run_serving(args)
    elif args.workload == "gemma":
        run_gemma(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
