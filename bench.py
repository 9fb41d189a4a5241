#!/usr/bin/env python
"""Benchmark of the paged GQA decode path: achieved HBM GB/s and us/call.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...     # the CPU restatement of the reference, timed

One "step" is one ``attention_b200.gqa_decode`` call over one synthetic batch
(plan + decode + merge kernels).  At N > 1 every rank holds its own batch, page
pool and block table (different seed per rank, same shape): weak scaling, no
collective on the data path.  Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
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

DEFAULT_WORKLOAD = "c2_qwen3_8b_bf16"
METRIC = "gqa_decode_achieved_hbm_gbps"
UNIT = "GB/s"
NOMINAL_HBM_GBPS = 8000.0
FALLBACK_PEAK_GBPS = 6650.0
DTYPE_NAME = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}

# DRAM bytes (read + write) per decode-kernel launch from the ncu capture summarised
# under profiles/, as a ratio to the algorithmic bytes of the captured case.
NCU_TRAFFIC_RATIO = {"c2_qwen3_8b_bf16": 1.010}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=20)
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
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--kernel", default="auto", choices=["auto", "simt", "mma"])
    p.add_argument("--chunk-tokens", type=int, default=0)
    p.add_argument("--cpu-seconds", type=float, default=10.0,
                   help="target CPU time of the cpu_baseline sample")
    p.add_argument("--spinup-seconds", type=float, default=1.0,
                   help="extra untimed warm-up so the SM clock is out of idle")
    p.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                   help="weak: every GPU gets its own batch of the workload (default); strong: "
                        "ONE batch of the workload is sharded over the GPUs (longest-first)")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-cold-cache", action="store_true")
    return p.parse_args()


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except (OSError, KeyError, ValueError):
        return FALLBACK_PEAK_GBPS, "fallback (6650 GB/s, earlier measurement on this pool)"


def workload_bytes(w, lens) -> int:
    return synth.algorithmic_bytes(lens.cpu(), batch=w.batch, q_heads=w.q_heads,
                                   kv_heads=w.kv_heads, head_dim=w.head_dim,
                                   elem_size=torch.empty((), dtype=w.dtype).element_size())


def config_of(w, extra=None):
    cfg = {
        "workload": w.name, "batch": w.batch, "q_heads": w.q_heads, "kv_heads": w.kv_heads,
        "head_dim": w.head_dim, "block_size": w.block_size, "context_lens":
        f"{w.len_dist}[{w.len_lo},{w.len_hi}]", "pool_factor": w.pool_factor,
        "parallelism": "batch-sharded, one page pool per GPU, no collective",
    }
    cfg.update(extra or {})
    return cfg


# --------------------------------------------------------------------------- CPU arm
def cpu_sample_workload(w, seed, n_seq):
    """The first ``n_seq`` sequences of the workload (same lengths as the GPU arm draws),
    with a fresh CPU page pool of the same layout."""
    gen = torch.Generator().manual_seed(seed)
    lens = synth.draw_lengths(w, gen)[:n_seq].clone()
    sw = synth.scaled(w, batch=int(lens.numel()), fixed_pool_blocks=0)
    q = torch.randn(sw.batch, w.q_heads, w.head_dim, generator=gen).to(w.dtype)
    pool = synth.pool_blocks_for(sw, lens)
    shape = (pool, w.block_size, w.kv_heads, w.head_dim)
    k = torch.randn(shape, generator=gen).to(w.dtype)
    v = torch.randn(shape, generator=gen).to(w.dtype)
    table = synth.build_block_table(lens, w.block_size, pool, gen)
    return sw, (q, k, v, table, lens)


def time_cpu_oracle(w, seed, target_seconds, repeats=1):
    """Time the C/OpenMP restatement of the reference on a bounded sample.

    Calibrates on one sequence, then sizes the sample (whole sequences, in batch order)
    for about ``target_seconds`` of CPU work.  Returns (GB/s, seconds, threads, description).
    """
    from oracle import gqa_oracle
    threads = len(os.sched_getaffinity(0))
    sw, inputs = cpu_sample_workload(w, seed, 1)
    gqa_oracle.gqa_decode_c(*inputs, threads=threads)            # warm the pages and the pool
    t0 = time.perf_counter()
    gqa_oracle.gqa_decode_c(*inputs, threads=threads)
    t1 = max(time.perf_counter() - t0, 1e-6)
    rate = workload_bytes(sw, inputs[4]) / t1
    gen = torch.Generator().manual_seed(seed)
    all_lens = synth.draw_lengths(w, gen)
    elem = torch.empty((), dtype=w.dtype).element_size()
    per_seq = all_lens.to(torch.int64) * w.kv_heads * w.head_dim * 2 * elem
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


def run_reference(args):
    """--impl reference: the reference's CPU algorithm (C/OpenMP restatement) on host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = synth.WORKLOADS[args.workload]
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
        "config": config_of(w, {"sample": desc}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
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
        while not self._stop.wait(0.005):
            self.sample()

    def __enter__(self):
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
def run_b200(args):
    import torch.distributed as dist

    import attention_b200 as attn

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback)")
    if not attn.is_cuda_extension_loaded():
        raise RuntimeError("C-ABI library missing: python -m attention_b200.build")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    w = synth.WORKLOADS[args.workload]
    imbalance = None
    if args.scaling == "strong" and world > 1:
        # one global batch; this rank owns the sequences the longest-first assignment gives
        # it, in a page pool of its own with its own block table -- no data-path collective
        from attention_b200 import sharding
        all_lens = synth.draw_lengths(w, torch.Generator().manual_seed(args.seed))
        shards = sharding.lpt_assign(all_lens.tolist(), world)
        imbalance = sharding.load_imbalance(all_lens.tolist(), shards)
        mine = all_lens[torch.as_tensor(shards[rank], dtype=torch.int64)]
        w, (q, k, v, table, lens) = synth.make_workload_for_lengths(
            w, mine, seed=args.seed + rank, device=dev, kv_on_device=True)
    else:
        q, k, v, table, lens = synth.make_workload(w, seed=args.seed + rank, device=dev,
                                                   kv_on_device=True)
    my_bytes = workload_bytes(w, lens)
    kw = dict(kernel=args.kernel, chunk_tokens=args.chunk_tokens)
    K, W = args.steps, max(args.warmup, 3)

    # ---- value: inputs resident in HBM, the public call, K steps between two events ----
    for _ in range(W):
        attn.gqa_decode(q, k, v, table, lens, **kw)
    # keep the GPU busy for a moment more so the SM clock has left its idle state
    # (a 100 us kernel repeated W times is over before the clock ramps)
    t_spin = time.perf_counter()
    while time.perf_counter() - t_spin < args.spinup_seconds:
        for _ in range(20):
            attn.gqa_decode(q, k, v, table, lens, **kw)
        torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    barrier()
    with sampler:
        ev0.record()
        for _ in range(K):
            out = attn.gqa_decode(q, k, v, table, lens, **kw)
        ev1.record()
        sampler.sample()            # at least one sample while the queue is still draining
        torch.cuda.synchronize()
    barrier()
    ms_total = ev0.elapsed_time(ev1)

    # ---- roofline: the decode kernel alone, its own events on the launching stream ----
    ws = torch.empty(attn.workspace_bytes(w.batch, w.q_heads, w.kv_heads, w.head_dim, w.block_size,
                                          table.shape[1], args.chunk_tokens),
                     dtype=torch.uint8, device=dev)
    out2 = torch.empty_like(q)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
             for _ in range(K)]
    for a, b in pairs:
        attn.gqa_decode(q, k, v, table, lens, out=out2, workspace=ws, phases=1, **kw)
        a.record()
        attn.gqa_decode(q, k, v, table, lens, out=out2, workspace=ws, phases=2, **kw)
        b.record()
        attn.gqa_decode(q, k, v, table, lens, out=out2, workspace=ws, phases=4, **kw)
    torch.cuda.synchronize()
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in pairs)
    assert torch.equal(out, out2), "phased launches must reproduce the one-call result"

    # ---- e2e: a decode step through the public API with per-step inputs in pinned host
    #      memory: H2D of q, the new token's key/value, block table, lengths; kv_append;
    #      gqa_decode; D2H of the output.  The page pool is device-resident state. ----
    # All per-step host inputs live in ONE pinned staging buffer (as a serving engine packs
    # its step metadata), mirrored by one device buffer the operator's tensors are views of.
    def carve(specs, device, pin):
        offs, total = [], 0
        for shape, dtype in specs:
            total = (total + 255) // 256 * 256
            offs.append(total)
            total += int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        buf = torch.empty(total, dtype=torch.uint8, device=device)
        if pin:
            buf = buf.pin_memory()
        views = [buf[o:o + int(torch.Size(sh).numel()) * torch.empty((), dtype=dt).element_size()]
                 .view(dt).view(sh) for o, (sh, dt) in zip(offs, specs)]
        return buf, views

    kv_row = (w.batch, w.kv_heads, w.head_dim)
    specs = [(tuple(q.shape), q.dtype), (kv_row, w.dtype), (kv_row, w.dtype),
             (tuple(table.shape), torch.int32), (tuple(lens.shape), torch.int32)]
    hbuf, (hq, hkey, hval, ht, hl) = carve(specs, "cpu", True)
    dbuf, (dq, dkey, dval, dt_, dl) = carve(specs, dev, False)
    hq.copy_(q)
    hkey.copy_(torch.randn(kv_row).to(w.dtype))
    hval.copy_(torch.randn(kv_row).to(w.dtype))
    ht.copy_(table)
    hl.copy_(lens)
    hout = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    pos = (lens - 1).clamp_(min=0)

    def e2e_step():
        dbuf.copy_(hbuf, non_blocking=True)
        attn.kv_append(dkey, dval, k, v, dt_, pos)
        o = attn.gqa_decode(dq, k, v, dt_, dl, **kw)
        hout.copy_(o, non_blocking=True)

    for _ in range(W):
        e2e_step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(K):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    h2d = hbuf.numel()
    d2h = hout.numel() * hout.element_size()

    # ---- reductions over ranks: MAX time, SUM bytes ----
    stats = torch.tensor([ms_total, e2e_ms, kernel_ms], dtype=torch.float64, device=dev)
    total_bytes = torch.tensor([float(my_bytes)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    ms_total, e2e_ms, kernel_ms_max = (float(x) for x in stats.cpu())
    all_bytes = float(total_bytes.item())

    # ---- optional: everything from host, the page pools included (N = 1 only) ----
    cold = None
    if world == 1 and not args.no_cold_cache:
        pool_bytes = 2 * k.numel() * k.element_size()
        if pool_bytes < 8e9:
            hk, hv = k.cpu().pin_memory(), v.cpu().pin_memory()
            steps = min(K, 3)

            def cold_step():
                k.copy_(hk, non_blocking=True)
                v.copy_(hv, non_blocking=True)
                e2e_step()

            cold_step()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            c0.record()
            for _ in range(steps):
                cold_step()
            c1.record()
            torch.cuda.synchronize()
            cms = c0.elapsed_time(c1) / steps
            cold = {"value": my_bytes / (cms * 1e-3) / 1e9, "unit": UNIT, "steps": steps,
                    "h2d_bytes_per_step": h2d + pool_bytes, "d2h_bytes_per_step": d2h,
                    "note": "page pools copied from pinned host memory every step as well"}
            del hk, hv

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    value = all_bytes * K / (ms_total * 1e-3) / 1e9
    achieved = my_bytes / (kernel_ms * 1e-3) / 1e9
    ratio = NCU_TRAFFIC_RATIO.get(w.name)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_total / K, "us_per_call": ms_total / K * 1e3,
        "higher_is_better": True,
        "scaling": args.scaling if world > 1 else "weak", "vs_baseline": None,
        "dtype": DTYPE_NAME[w.dtype], "data": "synthetic",
        "config": config_of(synth.WORKLOADS[args.workload], {
            "lpt_load_imbalance": imbalance,
            "kernel": args.kernel, "chunk_tokens": args.chunk_tokens, "seed": args.seed,
            "l2": f"inputs {my_bytes / 1e6:.0f} MB per GPU, larger than the 126 MB L2; no flush",
            "bytes_per_step_per_gpu": my_bytes}),
        "pct_of_nominal_8TBps": 100.0 * value / world / NOMINAL_HBM_GBPS,
        "pct_of_measured_peak": 100.0 * value / world / peak,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": peak_src,
                     "kernel": "gqa_decode_mma_kernel" if w.dtype != torch.float32 and
                     args.kernel != "simt" else "gqa_decode_simt_kernel",
                     "kernel_us": kernel_ms * 1e3, "kernel_us_max_over_ranks": kernel_ms_max * 1e3,
                     "algorithmic_bytes": my_bytes,
                     "traffic": None if ratio is None else ratio * my_bytes},
        "e2e": {"value": all_bytes * K / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / K,
                "note": "per step: pinned-host q, new key/value row, block table and lengths "
                        "copied in (one packed buffer), kv_append + gqa_decode, output copied "
                        "back; the page pool is device-resident state"},
        "gpu_launches": 3 * K,
        "clocks": sampler.summary(),
    }
    if cold is not None:
        line["e2e_cold_cache"] = cold
    if world == 1 and not args.no_cpu_baseline:
        gbps, secs, threads, desc, _, _ = time_cpu_oracle(w, args.seed, args.cpu_seconds)
        line["cpu_baseline"] = {"value": gbps, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": desc, "seconds": secs}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- prefill (secondary)
def run_prefill(args):
    """Dense GQA prefill throughput: one JSON line with TFLOP/s of one ``gqa_prefill`` call on a
    full causal batch (4 * B * Hq * D * T^2 / 2 flops), the roofline against the measured dense
    bf16 tensor peak, and the CPU restatement of the reference timed on a bounded sample."""
    import attention_b200 as attn

    if not torch.cuda.is_available() or not attn.is_cuda_extension_loaded():
        raise RuntimeError("needs a CUDA device and the built C-ABI library (no CPU fallback)")
    dev = torch.device("cuda", 0)
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
    sampler = ClockSampler(physical_gpu_index(0))
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
    try:
        peak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
        src = "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except (OSError, KeyError, ValueError):
        peak, src = 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"
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
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- MLA decode (secondary)
def run_mla(args):
    """Paged latent (MLA) decode attention: one JSON line with the achieved GB/s over the
    algorithmic bytes (every visible cache row once, queries in, latent output back), the
    roofline against the measured HBM peak (and the tensor-core time beside it: at 128 heads
    the operator sits at the ridge), and the CPU restatement timed on a bounded sample."""
    import attention_b200 as attn
    from attention_b200.mla import mla_tc_status

    if not torch.cuda.is_available() or not attn.is_cuda_extension_loaded():
        raise RuntimeError("needs a CUDA device and the built C-ABI library (no CPU fallback)")
    dev = torch.device("cuda", 0)
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
    sampler = ClockSampler(physical_gpu_index(0))
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
    try:
        tpeak = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
    except (OSError, KeyError, ValueError):
        tpeak = 1590.0
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
    if not args.no_cpu_baseline:
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
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.op == "prefill":
        run_prefill(args)
        return
    if args.op == "mla":
        run_mla(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
