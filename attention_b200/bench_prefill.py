"""Throughput of the dense GQA prefill operator (secondary benchmark; the headline
benchmark of the repository is ``bench.py`` at the root, which measures decode).

    python -m attention_b200.bench_prefill [--batch 4] [--seq 4096] [--steps 20]

Prints one JSON line: achieved TFLOP/s of one ``gqa_prefill`` call on a full causal
batch (4 * B * Hq * D * T^2 / 2 floating-point operations), the roofline against the
measured dense bf16 tensor peak, and the CPU restatement of the reference timed on a
bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import attention_b200 as attn  # noqa: E402

FALLBACK_TFLOPS = 1590.0


def tensor_peak():
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(peaks["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except (OSError, KeyError, ValueError):
        return FALLBACK_TFLOPS, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    ap.add_argument("--non-causal", action="store_true")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--kernel", default="auto", choices=["auto", "simt", "mma"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if not torch.cuda.is_available() or not attn.is_cuda_extension_loaded():
        raise RuntimeError("needs a CUDA device and the built C-ABI library (no CPU fallback)")
    dev = torch.device("cuda", 0)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    gen = torch.Generator(device=dev).manual_seed(42)
    b, t, hq, hkv, d = args.batch, args.seq, args.q_heads, args.kv_heads, args.head_dim
    q = torch.empty(b, t, hq, d, device=dev, dtype=dtype).normal_(generator=gen)
    k = torch.empty(b, t, hkv, d, device=dev, dtype=dtype).normal_(generator=gen)
    v = torch.empty(b, t, hkv, d, device=dev, dtype=dtype).normal_(generator=gen)
    lens = torch.full((b,), t, dtype=torch.int32, device=dev)
    causal = not args.non_causal

    def step():
        return attn.gqa_prefill(q, k, v, lens, lens, causal=causal, kernel=args.kernel)

    for _ in range(max(args.warmup, 3)):
        step()
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < 0.3:
        step()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * b * hq * d * t * t * (0.5 if causal else 1.0)
    tflops = flops / ms / 1e9
    peak, src = tensor_peak()
    line = {
        "metric": "gqa_prefill_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"dense prefill B{b} T{t} {hq}/{hkv} heads D{d} "
                               f"{'causal' if causal else 'full'}", "kernel": args.kernel,
                   "flops_per_step": flops},
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s",
                     "frac": tflops / peak, "peak_source": src, "traffic": None},
        "gpu_launches": args.steps,
    }
    if not args.no_cpu_baseline:
        from oracle import gqa_oracle
        n = min(t, 512)     # a bounded sample: the first 512 query rows / keys of one sequence
        cq, ck, cv = q[:1, :n].cpu(), k[:1, :n].cpu(), v[:1, :n].cpu()
        cl = torch.tensor([n], dtype=torch.int32)
        threads = len(os.sched_getaffinity(0))
        torch.set_num_threads(threads)
        gqa_oracle.reference_gqa_prefill(cq, ck, cv, cl, cl, causal=causal)
        t0 = time.perf_counter()
        gqa_oracle.reference_gqa_prefill(cq, ck, cv, cl, cl, causal=causal)
        dt = time.perf_counter() - t0
        cflops = 4.0 * hq * d * n * n * (0.5 if causal else 1.0)
        line["cpu_baseline"] = {"value": cflops / dt / 1e12, "unit": "TFLOP/s", "cores": threads,
                                "kind": "port", "seconds": dt,
                                "sample": f"first {n} rows/keys of one sequence, torch fp32 "
                                          "restatement of the reference oracle"}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
