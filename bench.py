#!/usr/bin/env python
"""Benchmark of the paged GQA decode path: achieved HBM GB/s and us/call.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...     # the CPU restatement of the reference, timed

One "step" is one ``attention_b200.gqa_decode`` call over one synthetic batch.  The headline
workload is the long-context batch (the largest single-GPU configuration).  The timed region
is R blocks of K calls (R chosen so that it lasts at least 50 ms); ``ms_per_step`` is the
median block divided by K, max over ranks.  At N > 1 every rank holds its own batch, page pool
and block table of the same lengths (weak scaling, no collective on the data path).

The one JSON line printed by rank 0 also carries
  per_config   the five benchmark configurations, each timed the same way
  strong_c5    ONE skewed serving batch sharded longest-first over the N GPUs (strong
               scaling), with the check that sharded and unsharded results are bit-identical
  secondary    dense prefill and paged latent (MLA) decode (N = 1 only)
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from attention_b200 import synth  # noqa: E402

DEFAULT_WORKLOAD = "c4_longctx_bf16"
METRIC = "gqa_decode_achieved_hbm_gbps"
UNIT = "GB/s"
NOMINAL_HBM_GBPS = 8000.0
FALLBACK_PEAK_GBPS = 6650.0
L2_BYTES = 126 * 1024 * 1024
MIN_TIMED_MS = 50.0
DTYPE_NAME = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}

# DRAM bytes (read + write) per decode-kernel launch from the ncu captures summarised under
# profiles/, as a ratio to the algorithmic bytes of the captured case (the long-context and
# the skewed workload were captured on cuts to their first 2 and 64 sequences; traffic grows
# in proportion to the tokens).
NCU_TRAFFIC_RATIO = {"c2_qwen3_8b_bf16": 1.010, "c3_qwen25_7b_fp16": 1.013,
                     "c4_longctx_bf16": 1.013, "c5_skewed_bf16": 1.010}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=["b200", "reference"], default="b200")
    p.add_argument("--op", choices=["decode", "prefill", "mla"], default="decode",
                   help="decode (the headline metric, default), the dense prefill operator, or "
                        "paged latent (MLA) decode attention")
    p.add_argument("--mla-workload", default="m2_deepseek_h128_bf16", choices=list(synth.MLA_WORKLOADS))
    p.add_argument("--mla-kernel", default="auto", choices=["auto", "simt", "tcgen05"])
    p.add_argument("--mla-stage", default="attend", choices=["attend", "decode"],
                   help="attend: mla_latent_attention alone; decode: absorb + attention + value projection")
    p.add_argument("--mla-splits", type=int, default=0)
    p.add_argument("--prefill-batch", type=int, default=4)
    p.add_argument("--prefill-seq", type=int, default=4096)
    p.add_argument("--prefill-kernel", default="auto", choices=["auto", "simt", "mma", "tcgen05"])
    p.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(synth.WORKLOADS))
    p.add_argument("--batch", type=int, default=0,
                   help="cut the workload to its first BATCH sequences (small profiler captures)")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--kernel", default="auto", choices=["auto", "simt", "mma"])
    p.add_argument("--chunk-tokens", type=int, default=0)
    p.add_argument("--phases", type=int, default=0,
                   help="0 = the default path; 7 = plan + decode + merge; 8 = one launch (decode kernel "
                        "plans and merges); 16 = two launches (self-planning decode, merge)")
    p.add_argument("--cpu-seconds", type=float, default=10.0,
                   help="target CPU time of the cpu_baseline sample")
    p.add_argument("--spinup-seconds", type=float, default=1.0,
                   help="extra untimed warm-up so the SM clock is out of idle")
    p.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                   help="headline at N > 1. weak: every GPU gets its own batch of the workload "
                        "(default); strong: ONE batch is sharded over the GPUs (longest-first)")
    p.add_argument("--only-headline", action="store_true",
                   help="skip per_config, strong_c5, secondary and the CPU baselines")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-per-config", action="store_true")
    p.add_argument("--no-strong", action="store_true")
    p.add_argument("--no-secondary", action="store_true")
    return p.parse_args()


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except (OSError, KeyError, ValueError):
        return FALLBACK_PEAK_GBPS, "fallback (6650 GB/s, earlier measurement on this pool)"


def measured_tensor_peak():
    try:
        return (float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"]),
                "measured (MEASURED_PEAKS.json bf16_tflops, burst)")
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def elem_size(dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def workload_bytes(w, lens) -> int:
    return synth.algorithmic_bytes(lens.cpu(), batch=w.batch, q_heads=w.q_heads,
                                   kv_heads=w.kv_heads, head_dim=w.head_dim,
                                   elem_size=elem_size(w.dtype))


def resolve_workload(name, batch):
    w = synth.WORKLOADS[name]
    if batch and batch < w.batch:
        w = synth.scaled(w, batch=batch, fixed_pool_blocks=0)
    return w


def l2_note(nbytes: int) -> str:
    if nbytes > 2 * L2_BYTES:
        return f"inputs {nbytes / 1e6:.0f} MB per GPU, larger than the 126 MB L2; no flush"
    return (f"inputs {nbytes / 1e6:.1f} MB per GPU, smaller than the 126 MB L2: calls rotate over "
            "copies of the page pools that together exceed twice the L2")


def config_of(w, seed):
    """Names the workload; the same dict in both arms (nothing arm-specific in it)."""
    lens = synth.draw_lengths(w, torch.Generator().manual_seed(seed))
    return {
        "workload": w.name, "batch": w.batch, "q_heads": w.q_heads, "kv_heads": w.kv_heads,
        "head_dim": w.head_dim, "block_size": w.block_size, "context_lens":
        f"{w.len_dist}[{w.len_lo},{w.len_hi}]", "pool_factor": w.pool_factor, "seed": seed,
        "bytes_per_step_per_gpu": workload_bytes(w, lens),
        "l2": l2_note(workload_bytes(w, lens)),
        "parallelism": "batch-sharded, one page pool per GPU, no collective",
    }


# --------------------------------------------------------------------------- CPU arm
def cpu_sample_workload(w, seed, n_seq):
    """The first ``n_seq`` sequences of the workload (same lengths as the GPU arm draws),
    with a fresh CPU page pool of the same layout."""
    lens = synth.draw_lengths(w, torch.Generator().manual_seed(seed))[:n_seq].clone()
    return synth.make_workload_for_lengths(w, lens, seed=seed, kv_threaded=True)


def time_cpu_oracle(w, seed, target_seconds, repeats=1):
    """Time the C/OpenMP restatement of the reference on a bounded sample.

    Calibrates on one sequence, then sizes the sample (whole sequences, in batch order)
    for about ``target_seconds`` of CPU work.  Returns (GB/s, seconds, threads, description,
    sample workload, sample inputs).
    """
    from oracle import gqa_oracle
    threads = len(os.sched_getaffinity(0))
    sw, inputs = cpu_sample_workload(w, seed, 1)
    gqa_oracle.gqa_decode_c(*inputs, threads=threads)            # warm the pages and the pool
    t0 = time.perf_counter()
    gqa_oracle.gqa_decode_c(*inputs, threads=threads)
    t1 = max(time.perf_counter() - t0, 1e-6)
    rate = workload_bytes(sw, inputs[4]) / t1
    all_lens = synth.draw_lengths(w, torch.Generator().manual_seed(seed))
    per_seq = all_lens.to(torch.int64) * w.kv_heads * w.head_dim * 2 * elem_size(w.dtype)
    budget = rate * target_seconds
    n = int((per_seq.cumsum(0) <= budget).sum().item())
    n = max(1, min(n, w.batch))
    sw, inputs = cpu_sample_workload(w, seed, n)
    if n == w.batch:   # the whole batch is cheaper than the target: repeat it instead
        whole = max(per_seq.sum().item() / rate, 1e-3)
        repeats = max(repeats, min(20, int(target_seconds / whole)))
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        gqa_oracle.gqa_decode_c(*inputs, threads=threads)
        best = min(best, time.perf_counter() - t0)
    nbytes = workload_bytes(sw, inputs[4])
    desc = (f"first {n} of {w.batch} sequences of {w.name} ({int(inputs[4].sum())} tokens, "
            f"{nbytes / 1e6:.1f} MB algorithmic), C/OpenMP restatement of the reference oracle")
    return nbytes / best / 1e9, best, threads, desc, sw, inputs


def time_reference_python(w, seed, max_tokens=150_000):
    """The reference's own CPU function ``reference_gqa_decode`` (attention/reference/gqa.py:7-44),
    loaded from the unmodified install under baseline/_ref when that travelled with the
    repository, on the first sequences of the workload (at most ``max_tokens`` tokens: the
    function materialises fp32 copies of every query head's keys and values).  None if absent."""
    path = ROOT / "baseline" / "_ref" / "attention" / "reference" / "gqa.py"
    if not path.is_file():
        return None
    try:
        spec = importlib.util.spec_from_file_location("_reference_gqa_oracle", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        all_lens = synth.draw_lengths(w, torch.Generator().manual_seed(seed))
        n = int((all_lens.to(torch.int64).cumsum(0) <= max_tokens).sum().item())
        n = max(1, min(n, w.batch))
        sw, inputs = cpu_sample_workload(w, seed, n)
        threads = len(os.sched_getaffinity(0))
        torch.set_num_threads(threads)
        mod.reference_gqa_decode(*inputs)
        t0 = time.perf_counter()
        mod.reference_gqa_decode(*inputs)
        dt = time.perf_counter() - t0
        nbytes = workload_bytes(sw, inputs[4])
        return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "reference",
                "seconds": dt,
                "sample": f"first {n} of {w.batch} sequences of {w.name} ({int(inputs[4].sum())} tokens), "
                          "the reference's reference_gqa_decode (torch, CPU) from baseline/_ref"}
    except Exception as exc:   # noqa: BLE001 - a side measurement must not fail the line
        return {"error": str(exc)[:160]}


def run_reference(args):
    """--impl reference: the reference's CPU algorithm (C/OpenMP restatement) on host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = resolve_workload(args.workload, args.batch)
    from oracle import gqa_oracle
    total_steps = max(1, args.steps + args.warmup)
    per_step = min(10.0, 150.0 / total_steps)
    gbps, _, threads, desc, sw, inputs = time_cpu_oracle(w, args.seed, per_step)
    for _ in range(args.warmup):
        gqa_oracle.gqa_decode_c(*inputs, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        gqa_oracle.gqa_decode_c(*inputs, threads=threads)
    dt = time.perf_counter() - t0
    nbytes = workload_bytes(sw, inputs[4])
    value = nbytes * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE_NAME[w.dtype], "data": "synthetic",
        "config": config_of(w, args.seed),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_cpu_baseline:
        py = time_reference_python(w, args.seed)
        if py is not None:
            line["cpu_baseline_reference_python"] = py
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {
        0x0000000000000008: "hw_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000004: "sw_power_cap",
    }

    def __init__(self, index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:   # NVML missing: report nulls rather than fail the benchmark
            self._nv = None

    def sample(self):
        if self._nv is None:
            return
        try:
            self.samples.append(int(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM)))
            mask = int(self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _loop(self):
        while not self._stop.wait(0.004):
            self.sample()

    def __enter__(self):
        self.samples, self.reasons = [], set()
        self._stop.clear()
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except (ValueError, IndexError):
            pass
    return local_index


# --------------------------------------------------------------------------- GPU arm
class Dist:
    """The harness's view of the process group: barrier and MAX / SUM of a few floats."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None

    def init(self):
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, values, op):
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.dist is not None:
            self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, op))
        return [float(x) for x in t.cpu()]

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def pool_copies(k, v, nbytes):
    """Enough copies of the page pools that consecutive calls never find their rows in L2
    (only for workloads smaller than twice the L2; larger ones defeat it by themselves)."""
    if nbytes > 2 * L2_BYTES:
        return [(k, v)]
    n = int(math.ceil(2.0 * L2_BYTES / max(1, 2 * k.numel() * k.element_size()))) + 1
    return [(k, v)] + [(k.clone(), v.clone()) for _ in range(n - 1)]


def time_decode(attn, D, sampler, w, inputs, kw, K, W, spin_s):
    """Times ``gqa_decode`` on resident inputs.

    W warm-up calls, ``spin_s`` seconds of untimed calls (SM clock out of idle), then R blocks
    of K back-to-back calls, R such that the region lasts >= MIN_TIMED_MS; one CUDA event
    between blocks; barrier + synchronize on both sides.  Then the decode kernel alone (events
    around single launches) and, from the same inputs in pinned host
    memory, the end-to-end step.  Returns a dict of rank-local numbers.
    """
    q, k, v, table, lens = inputs
    nbytes = workload_bytes(w, lens)
    pools = pool_copies(k, v, nbytes)
    n_pools = len(pools)
    calls = [0]

    def call(**extra):
        kk, vv = pools[calls[0] % n_pools]
        calls[0] += 1
        return attn.gqa_decode(q, kk, vv, table, lens, **kw, **extra)

    for _ in range(W):
        call()
    torch.cuda.synchronize()
    t_spin = time.perf_counter()
    n_spin = 0
    while time.perf_counter() - t_spin < spin_s:
        for _ in range(10):
            call()
        n_spin += 10
        torch.cuda.synchronize()
    est_ms = (time.perf_counter() - t_spin) * 1e3 / max(1, n_spin) if n_spin else 1.0
    R = max(3, int(math.ceil(MIN_TIMED_MS / max(1e-3, est_ms * K))))
    R = min(R, 2000)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(R + 1)]
    D.barrier()
    with sampler:
        marks[0].record()
        for r in range(R):
            for _ in range(K):
                out = call()
            marks[r + 1].record()
            sampler.sample()        # one sample per block from this thread as well (the sampling
                                    # thread gets few turns while this loop holds the interpreter)
        sampler.sample()            # and one while the queue is still draining
        torch.cuda.synchronize()
    D.barrier()
    clocks = sampler.summary()
    blocks = [marks[r].elapsed_time(marks[r + 1]) for r in range(R)]
    block_ms = statistics.median(blocks)

    # ---- the decode kernel alone, its own events on the launching stream: the self-planning
    #      decode kernel is launched by itself (phases 32) between the two events and the merge
    #      kernel (phases 4) after the closing one; above 2048 sequences plan / decode / merge ----
    ws = torch.zeros(attn.workspace_bytes(w.batch, w.q_heads, w.kv_heads, w.head_dim, w.block_size,
                                          table.shape[1], kw.get("chunk_tokens", 0)),
                     dtype=torch.uint8, device=q.device)
    out2 = torch.empty_like(q)
    kwk = {k_: v_ for k_, v_ in kw.items() if k_ != "phases"}
    self_plan = w.batch <= 2048
    n_k = max(K, min(200, int(math.ceil(20.0 / max(1e-3, est_ms)))))
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
             for _ in range(n_k)]
    for a, b in pairs:
        kk, vv = pools[calls[0] % n_pools]
        calls[0] += 1
        if self_plan:
            a.record()
            attn.gqa_decode(q, kk, vv, table, lens, out=out2, workspace=ws, phases=32, **kwk)
            b.record()
        else:
            attn.gqa_decode(q, kk, vv, table, lens, out=out2, workspace=ws, phases=1, **kwk)
            a.record()
            attn.gqa_decode(q, kk, vv, table, lens, out=out2, workspace=ws, phases=2, **kwk)
            b.record()
        attn.gqa_decode(q, kk, vv, table, lens, out=out2, workspace=ws, phases=4, **kwk)
    torch.cuda.synchronize()
    kernel_ms = statistics.median(a.elapsed_time(b) for a, b in pairs)
    if kw.get("phases", 0) in (0, 16):
        assert torch.equal(out, out2), "phased launches must reproduce the one-call result"

    # ---- e2e: a decode step through the public API with per-step inputs in pinned host
    #      memory: H2D of q, the new token's key/value, block table, lengths; kv_append;
    #      gqa_decode; D2H of the output.  The page pool is device-resident state.  All
    #      per-step host inputs live in ONE pinned staging buffer (as a serving engine packs
    #      its step metadata), mirrored by one device buffer the operator's tensors view. ----
    def carve(specs, device, pin):
        offs, total = [], 0
        for shape, dtype in specs:
            total = (total + 255) // 256 * 256
            offs.append(total)
            total += int(torch.Size(shape).numel()) * elem_size(dtype)
        buf = torch.empty(total, dtype=torch.uint8, device=device)
        if pin:
            buf = buf.pin_memory()
        views = [buf[o:o + int(torch.Size(sh).numel()) * elem_size(dt)].view(dt).view(sh)
                 for o, (sh, dt) in zip(offs, specs)]
        return buf, views

    kv_row = (w.batch, w.kv_heads, w.head_dim)
    specs = [(tuple(q.shape), q.dtype), (kv_row, w.dtype), (kv_row, w.dtype),
             (tuple(table.shape), torch.int32), (tuple(lens.shape), torch.int32)]
    hbuf, (hq, hkey, hval, ht, hl) = carve(specs, "cpu", True)
    dbuf, (dq, dkey, dval, dt_, dl) = carve(specs, q.device, False)
    hq.copy_(q)
    hkey.copy_(torch.randn(kv_row).to(w.dtype))
    hval.copy_(torch.randn(kv_row).to(w.dtype))
    ht.copy_(table)
    hl.copy_(lens)
    hout = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    pos = (lens - 1).clamp_(min=0)

    def e2e_step():
        kk, vv = pools[calls[0] % n_pools]
        calls[0] += 1
        dbuf.copy_(hbuf, non_blocking=True)
        attn.kv_append(dkey, dval, kk, vv, dt_, pos)
        o = attn.gqa_decode(dq, kk, vv, dt_, dl, **kw)
        hout.copy_(o, non_blocking=True)

    for _ in range(W):
        e2e_step()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(R + 1)]
    D.barrier()
    marks[0].record()
    for r in range(R):
        for _ in range(K):
            e2e_step()
        marks[r + 1].record()
    torch.cuda.synchronize()
    D.barrier()
    e2e_block_ms = statistics.median(marks[r].elapsed_time(marks[r + 1]) for r in range(R))
    return {"bytes": nbytes, "block_ms": block_ms, "blocks": R, "block_ms_min": min(blocks),
            "block_ms_max": max(blocks), "kernel_ms": kernel_ms, "e2e_block_ms": e2e_block_ms,
            "h2d": hbuf.numel(), "d2h": hout.numel() * hout.element_size(), "clocks": clocks,
            "pool_copies": n_pools}


def decode_kernel_name(w, kernel):
    return ("gqa_decode_mma_kernel" if w.dtype != torch.float32 and kernel != "simt"
            else "gqa_decode_simt_kernel")


def summarise(D, w, local, K, peak, kernel):
    """Reduce one workload's rank-local timings over ranks (MAX time, SUM bytes)."""
    block_ms, e2e_ms, kernel_ms_max = D.reduce([local["block_ms"], local["e2e_block_ms"],
                                                local["kernel_ms"]], "MAX")
    (all_bytes,) = D.reduce([float(local["bytes"])], "SUM")
    value = all_bytes * K / (block_ms * 1e-3) / 1e9
    achieved = local["bytes"] / (local["kernel_ms"] * 1e-3) / 1e9
    ratio = NCU_TRAFFIC_RATIO.get(w.name)
    return {
        "value": value, "unit": UNIT, "us_per_call": block_ms / K * 1e3, "ms_per_step": block_ms / K,
        "pct_of_nominal_8TBps": 100.0 * value / D.world / NOMINAL_HBM_GBPS,
        "pct_of_measured_peak": 100.0 * value / D.world / peak,
        "bytes_per_step_per_gpu": local["bytes"],
        "timed_blocks": local["blocks"],
        "us_per_call_min_max_block": [local["block_ms_min"] / K * 1e3, local["block_ms_max"] / K * 1e3],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "kernel": decode_kernel_name(w, kernel),
                     "kernel_us": local["kernel_ms"] * 1e3,
                     "kernel_us_max_over_ranks": kernel_ms_max * 1e3,
                     "algorithmic_bytes": local["bytes"],
                     "traffic": None if ratio is None else ratio * local["bytes"]},
        "e2e": {"value": all_bytes * K / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": local["h2d"], "d2h_bytes_per_step": local["d2h"],
                "ms_per_step": e2e_ms / K},
        "l2": l2_note(local["bytes"]),
        "clocks": local["clocks"],
    }


def make_rank_workload(w, seed, D, scaling="weak"):
    """This rank's tensors.  weak: the SAME lengths on every rank (so that SUM(bytes) is N times
    rank 0's and the efficiency measures time only), contents drawn with seed + rank.  strong:
    one batch sharded longest-first; returns the load imbalance too."""
    all_lens = synth.draw_lengths(w, torch.Generator().manual_seed(seed))
    if scaling == "strong":
        from attention_b200 import sharding
        shards = sharding.lpt_assign(all_lens.tolist(), D.world)
        imbalance = sharding.load_imbalance(all_lens.tolist(), shards)
        mine = all_lens[torch.as_tensor(shards[D.rank], dtype=torch.int64)]
        lw, inputs = synth.make_workload_for_lengths(w, mine, seed=seed + D.rank, device=D.dev,
                                                     kv_on_device=True)
        return lw, inputs, imbalance
    if D.rank == 0:
        return w, synth.make_workload(w, seed=seed, device=D.dev, kv_on_device=True), None
    lw, inputs = synth.make_workload_for_lengths(w, all_lens, seed=seed + D.rank, device=D.dev,
                                                 kv_on_device=True)
    return lw, inputs, None


def sharded_bit_identity(attn, D, seed):
    """Every rank decodes its shard (own page pool, own table) of one small skewed batch with a
    fixed chunk length; rank 0 gathers the rows (harness-only all_gather, after the timing) and
    compares them with its own unsharded run."""
    from attention_b200 import sharding
    w = synth.scaled("c5_skewed_bf16", batch=32, len_hi=4096)
    q, k, v, table, lens = synth.make_workload(w, seed=seed)          # the same case on every rank
    shards = sharding.lpt_assign(lens.tolist(), D.world)
    local = sharding.extract_shard(q, k, v, table, lens, shards[D.rank], device=D.dev)
    if len(shards[D.rank]):
        mine = attn.gqa_decode(*local, chunk_tokens=512)
    else:
        mine = torch.empty((0,) + tuple(q.shape[1:]), dtype=q.dtype, device=D.dev)
    biggest = max(len(s) for s in shards)
    padded = torch.zeros((biggest,) + tuple(q.shape[1:]), dtype=q.dtype, device=D.dev)
    padded[: mine.shape[0]] = mine
    if D.dist is not None:
        parts = [torch.empty_like(padded) for _ in range(D.world)]
        D.dist.all_gather(parts, padded)
    else:
        parts = [padded]
    if D.rank != 0:
        return None
    parts = [p[: len(s)] for p, s in zip(parts, shards)]
    whole = sharding.scatter_outputs(parts, shards, w.batch)
    single = attn.gqa_decode(q.to(D.dev), k.to(D.dev), v.to(D.dev), table.to(D.dev), lens.to(D.dev),
                             chunk_tokens=512)
    return bool(torch.equal(whole, single))


def run_b200(args):
    import attention_b200 as attn

    D = Dist()
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback)")
    if not attn.is_cuda_extension_loaded():
        raise RuntimeError("C-ABI library missing: python -m attention_b200.build")
    D.init()
    peak, peak_src = measured_peak()
    sampler = ClockSampler(physical_gpu_index(D.local_rank))
    kw = dict(kernel=args.kernel, chunk_tokens=args.chunk_tokens, phases=args.phases)
    K, W = args.steps, max(args.warmup, 3)
    extras = not args.only_headline

    # ---- headline ----
    w = resolve_workload(args.workload, args.batch)
    scaling = args.scaling if D.world > 1 else "weak"
    lw, inputs, imbalance = make_rank_workload(w, args.seed, D, scaling)
    local = time_decode(attn, D, sampler, lw, inputs, kw, K, W, args.spinup_seconds)
    head = summarise(D, w, local, K, peak, args.kernel)
    del inputs
    torch.cuda.empty_cache()

    # ---- the five configurations, each timed the same way ----
    per_config = {}
    if extras and not args.no_per_config:
        for name, cw in synth.WORKLOADS.items():
            if name == w.name and not args.batch and scaling == "weak":
                per_config[name] = {k: v for k, v in head.items()}
                continue
            clw, cin, _ = make_rank_workload(cw, args.seed, D, "weak")
            cl = time_decode(attn, D, sampler, clw, cin, kw, K, W, min(args.spinup_seconds, 0.3))
            per_config[name] = summarise(D, cw, cl, K, peak, args.kernel)
            del cin
            torch.cuda.empty_cache()

    # ---- one skewed serving batch sharded over the N GPUs (strong scaling) ----
    strong = None
    if extras and not args.no_strong:
        cw = synth.WORKLOADS["c5_skewed_bf16"]
        slw, sin, simb = make_rank_workload(cw, args.seed, D, "strong")
        sl = time_decode(attn, D, sampler, slw, sin, kw, K, W, min(args.spinup_seconds, 0.3))
        s = summarise(D, cw, sl, K, peak, args.kernel)
        del sin
        torch.cuda.empty_cache()
        identical = sharded_bit_identity(attn, D, args.seed)
        strong = {"workload": cw.name, "n_gpus": D.world, "value": s["value"], "unit": UNIT,
                  "us_per_call": s["us_per_call"], "lpt_load_imbalance": simb,
                  "rank0_bytes_per_step": sl["bytes"], "kernel_us_max_over_ranks":
                  s["roofline"]["kernel_us_max_over_ranks"], "e2e": s["e2e"], "clocks": s["clocks"],
                  "sharded_bit_identical": identical,
                  "note": "ONE batch of the workload split longest-first over the GPUs, each rank "
                          "with its own page pool and block table; max-over-ranks time; compare "
                          "value with the same block of the N = 1 run"}

    if D.rank != 0:
        D.close()
        return

    # decode + merge kernels per call (one launch for small static shapes, three above 2048 sequences)
    launches_per_step = {7: 3, 8: 1, 16: 2}.get(args.phases, 2 if w.batch <= 2048 else 3)
    line = {
        "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": D.world, "steps": K,
        "warmup": W, "ms_per_step": head["ms_per_step"], "us_per_call": head["us_per_call"],
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": DTYPE_NAME[w.dtype], "data": "synthetic",
        "config": config_of(w, args.seed),
        "details": {"kernel": args.kernel, "chunk_tokens": args.chunk_tokens,
                    "lpt_load_imbalance": imbalance, "timed_blocks": head["timed_blocks"],
                    "timed_region_ms": head["timed_blocks"] * head["ms_per_step"] * K,
                    "us_per_call_min_max_block": head["us_per_call_min_max_block"],
                    "ms_per_step_is": "median over timed_blocks blocks of `steps` calls each, "
                                      "max over ranks"},
        "pct_of_nominal_8TBps": head["pct_of_nominal_8TBps"],
        "pct_of_measured_peak": head["pct_of_measured_peak"],
        "roofline": dict(head["roofline"], peak_source=peak_src),
        "e2e": dict(head["e2e"], note="per step: pinned-host q, new key/value row, block table and "
                                      "lengths copied in (one packed buffer), kv_append + gqa_decode, "
                                      "output copied back; the page pool is device-resident state"),
        "gpu_launches": launches_per_step * K * head["timed_blocks"],
        "clocks": head["clocks"],
    }
    if per_config:
        line["per_config"] = per_config
    if strong is not None:
        line["strong_c5"] = strong
    if extras and D.world == 1 and not args.no_secondary:
        line["secondary"] = run_secondary(args)
    if extras and D.world == 1 and not args.no_cpu_baseline:
        gbps, secs, threads, desc, _, _ = time_cpu_oracle(w, args.seed, args.cpu_seconds)
        line["cpu_baseline"] = {"value": gbps, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": desc, "seconds": secs}
        py = time_reference_python(w, args.seed)
        if py is not None:
            line["cpu_baseline_reference_python"] = py
    print(json.dumps(line), flush=True)
    D.close()


# --------------------------------------------------------------------------- secondary operators
def run_secondary(args):
    """Dense prefill and paged latent (MLA) decode on few steps, as one block of the decode line."""
    out = {}
    sub = argparse.Namespace(**vars(args))
    sub.steps, sub.warmup, sub.spinup_seconds, sub.no_cpu_baseline = 10, 3, 0.3, True
    for key, fn, setup in (
        ("prefill", measure_prefill, {}),
        ("mla_attend", measure_mla, {"mla_stage": "attend"}),
        ("mla_decode", measure_mla, {"mla_stage": "decode"}),
    ):
        for name, val in setup.items():
            setattr(sub, name, val)
        try:
            full = fn(sub)
            keep = {k: full[k] for k in ("metric", "value", "unit", "ms_per_step", "clocks") if k in full}
            keep["workload"] = full["config"]["workload"]
            r = full["roofline"]
            keep["roofline"] = {k: r[k] for k in ("bound", "achieved", "peak", "unit", "frac") if k in r}
            if "tensor_frac" in r:
                keep["tensor_frac"] = r["tensor_frac"]
            if "tc_status" in full:
                keep["tc_status"] = full["tc_status"]
            out[key] = keep
        except Exception as exc:   # noqa: BLE001 - a secondary line must not fail the headline
            out[key] = {"error": str(exc)[:200]}
        torch.cuda.empty_cache()
    return out


def measure_prefill(args):
    """Dense GQA prefill throughput: TFLOP/s of one ``gqa_prefill`` call on a full causal batch
    (4 * B * Hq * D * T^2 / 2 flops), the roofline against the measured dense bf16 tensor peak,
    and the CPU restatement of the reference timed on a bounded sample."""
    import attention_b200 as attn

    if not torch.cuda.is_available() or not attn.is_cuda_extension_loaded():
        raise RuntimeError("needs a CUDA device and the built C-ABI library (no CPU fallback)")
    dev = torch.device("cuda", torch.cuda.current_device())
    b, t, hq, hkv, d = args.prefill_batch, args.prefill_seq, 32, 8, 128
    gen = torch.Generator(device=dev).manual_seed(args.seed)
    q = torch.empty(b, t, hq, d, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    k = torch.empty(b, t, hkv, d, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    v = torch.empty(b, t, hkv, d, device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    lens = torch.full((b,), t, dtype=torch.int32, device=dev)

    def step():
        return attn.gqa_prefill(q, k, v, lens, lens, causal=True, kernel=args.prefill_kernel)

    for _ in range(max(args.warmup, 3)):
        step()
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < args.spinup_seconds:
        step()
        torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(dev.index))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        sampler.sample()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * b * hq * d * t * t * 0.5
    tflops = flops / ms / 1e9
    peak, src = measured_tensor_peak()
    line = {
        "metric": "gqa_prefill_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "vs_baseline": None,
        "config": {"workload": f"dense causal prefill B{b} T{t} {hq}/{hkv} heads D{d}",
                   "kernel": args.prefill_kernel, "flops_per_step": flops},
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s",
                     "frac": tflops / peak, "peak_source": src, "traffic": None},
        "gpu_launches": args.steps, "clocks": sampler.summary(),
    }
    if not args.no_cpu_baseline:
        from oracle import gqa_oracle
        n = min(t, 512)     # bounded sample: the first 512 query rows / keys of one sequence
        cq, ck, cv = q[:1, :n].cpu(), k[:1, :n].cpu(), v[:1, :n].cpu()
        cl = torch.tensor([n], dtype=torch.int32)
        threads = len(os.sched_getaffinity(0))
        torch.set_num_threads(threads)
        gqa_oracle.reference_gqa_prefill(cq, ck, cv, cl, cl)
        t0 = time.perf_counter()
        gqa_oracle.reference_gqa_prefill(cq, ck, cv, cl, cl)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 4.0 * hq * d * n * n * 0.5 / dt / 1e12, "unit": "TFLOP/s",
                                "cores": threads, "kind": "port", "seconds": dt,
                                "sample": f"first {n} rows/keys of one sequence, torch fp32 "
                                          "restatement of the reference oracle"}
    return line


def measure_mla(args):
    """Paged latent (MLA) decode attention: the achieved GB/s over the algorithmic bytes (every
    visible cache row once, queries in, latent output back), the roofline against the measured
    HBM peak (and the tensor-core time beside it: at 128 heads the operator sits at the ridge),
    and the CPU restatement timed on a bounded sample."""
    import attention_b200 as attn
    from attention_b200.mla import mla_tc_status

    if not torch.cuda.is_available() or not attn.is_cuda_extension_loaded():
        raise RuntimeError("needs a CUDA device and the built C-ABI library (no CPU fallback)")
    dev = torch.device("cuda", torch.cuda.current_device())
    w = synth.MLA_WORKLOADS[args.mla_workload]
    c = synth.make_mla_case(w, seed=args.seed, device=dev, cache_on_device=True)
    scale = 1.0 / math.sqrt(w.dn + w.dr)
    qa = attn.mla_query_absorb(c["q_nope"], c["w_uk"])

    if args.mla_stage == "attend":
        def step():
            return attn.mla_latent_attention(qa, c["q_rope"], c["cache"], c["block_table"], c["lengths"],
                                             c["positions"], scale=scale, kernel=args.mla_kernel,
                                             splits=args.mla_splits)
    else:
        def step():
            return attn.mla_decode(c["q_nope"], c["q_rope"], c["cache"], c["block_table"], c["lengths"],
                                   c["positions"], c["w_uk"], c["w_uv"])

    for _ in range(max(args.warmup, 3)):
        step()
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < args.spinup_seconds:
        step()
        torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(dev.index))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        sampler.sample()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    lens = c["lengths"].cpu()
    nbytes = synth.mla_algorithmic_bytes(lens, w)
    tokens = int(lens.to(torch.int64).sum())
    flops = 2.0 * tokens * w.tq * w.heads * (w.dc + w.dr + w.dc)
    gbps = nbytes / ms / 1e6
    peak, src = measured_peak()
    tpeak, _ = measured_tensor_peak()
    line = {
        "metric": f"mla_{args.mla_stage}_gbps", "value": gbps, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "dtype": str(w.dtype).replace("torch.", ""), "data": "synthetic", "vs_baseline": None,
        "config": {"workload": w.name, "batch": w.batch, "tq": w.tq, "heads": w.heads, "dc": w.dc, "dr": w.dr,
                   "page": w.page, "lengths": f"uniform[{w.len_lo},{w.len_hi}]", "kernel": args.mla_kernel,
                   "stage": args.mla_stage, "bytes_per_step": nbytes, "flops_per_step": flops,
                   "cache": "page pool larger than L2; no flush between steps"},
        "roofline": {"bound": "hbm", "achieved": gbps, "peak": peak, "unit": "GB/s", "frac": gbps / peak,
                     "peak_source": src, "traffic": None,
                     "tensor_tflops": flops / ms / 1e9, "tensor_frac": flops / ms / 1e9 / tpeak},
        "gpu_launches": args.steps * (3 if args.mla_stage == "attend" else 5), "clocks": sampler.summary(),
        "tc_status": mla_tc_status(),
    }
    if args.no_cpu_baseline:       # the short form used inside the decode line
        return line
    # ---- end to end: one decode step through the public API with the per-step inputs in pinned
    #      host memory (queries, the new token's latent and rotated key rows, its cache slots,
    #      lengths, positions, block table), copies in, latent_kv_write + mla_decode, result back.
    #      The page pool and the weights are device-resident state, as in a serving loop. ----
    try:
        pin = lambda t: t.cpu().pin_memory()   # noqa: E731
        h_in = {k: pin(c[k]) for k in ("q_nope", "q_rope", "block_table", "lengths", "positions")}
        h_lat = pin(torch.randn(w.batch, w.dc).to(w.dtype))
        h_rope = pin(torch.randn(w.batch, w.dr).to(w.dtype))
        last = (lens.to(torch.int64) - 1).clamp_(min=0)          # rewrite the last token of every sequence
        tbl = c["block_table"].cpu().to(torch.int64)
        h_slots = pin(tbl[torch.arange(w.batch), last // w.page] * w.page + last % w.page)
        h_out = torch.empty(w.batch, w.tq, w.heads, w.dv, dtype=w.dtype).pin_memory()
        d_in = {k: torch.empty_like(v, device=dev) for k, v in h_in.items()}
        d_lat, d_rope, d_slots = (torch.empty_like(t, device=dev) for t in (h_lat, h_rope, h_slots))

        def e2e_step():
            for k, v in h_in.items():
                d_in[k].copy_(v, non_blocking=True)
            d_lat.copy_(h_lat, non_blocking=True)
            d_rope.copy_(h_rope, non_blocking=True)
            d_slots.copy_(h_slots, non_blocking=True)
            attn.latent_kv_write(d_lat, d_rope, c["cache"], d_slots)
            out = attn.mla_decode(d_in["q_nope"], d_in["q_rope"], c["cache"], d_in["block_table"],
                                  d_in["lengths"], d_in["positions"], c["w_uk"], c["w_uv"])
            h_out.copy_(out, non_blocking=True)

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        n_e2e = max(5, args.steps // 4)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / n_e2e
        h2d = sum(v.numel() * v.element_size() for v in h_in.values()) + sum(
            t.numel() * t.element_size() for t in (h_lat, h_rope, h_slots))
        line["e2e"] = {"value": nbytes / e2e_ms / 1e6, "unit": "GB/s", "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": h_out.numel() * h_out.element_size(),
                       "what": "latent_kv_write + mla_decode with per-step inputs copied from pinned host memory"}
    except RuntimeError as exc:   # pinned memory unavailable: report, do not fail the line
        line["e2e"] = {"error": str(exc)[:120]}
    from oracle import mla_oracle
    n = 1                                   # bounded sample: the first sequence
    sl = {k: (v[:n].cpu() if k in ("q_rope", "block_table", "lengths", "positions") else v.cpu())
          for k, v in c.items() if k != "cache"}
    used = int((int(lens[0]) + w.page - 1) // w.page)
    pages = sl["block_table"][0, :used].long()
    cache = c["cache"][pages.to(dev)].cpu()                     # only that sequence's pages
    table = torch.arange(used, dtype=torch.int32).view(1, used)
    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    args_cpu = (qa[:n].cpu(), sl["q_rope"], cache, table, sl["lengths"], sl["positions"])
    mla_oracle.reference_mla_latent_attention(*args_cpu, scale=scale)
    t0 = time.perf_counter()
    mla_oracle.reference_mla_latent_attention(*args_cpu, scale=scale)
    dt = time.perf_counter() - t0
    sample_bytes = synth.mla_algorithmic_bytes(lens[:n], synth.scaled_mla(w, batch=n))
    line["cpu_baseline"] = {"value": sample_bytes / dt / 1e9, "unit": "GB/s", "cores": threads,
                            "kind": "port", "seconds": dt,
                            "sample": f"first sequence ({int(lens[0])} tokens), torch fp32 restatement "
                                      "of the reference oracle (latent attention only)"}
    return line


def main():
    args = parse_args()
    if args.op == "prefill":
        print(json.dumps(measure_prefill(args)), flush=True)
        return
    if args.op == "mla":
        print(json.dumps(measure_mla(args)), flush=True)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
