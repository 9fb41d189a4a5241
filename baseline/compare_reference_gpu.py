#!/usr/bin/env python
"""Side-by-side GPU timing of this library and the UNMODIFIED reference on one B200.

Context numbers, not the benchmark's reference arm (that one is the CPU oracle):
the reference's own CUDA decode kernel ("unoptimized CUDA baseline",
attention/core.py:26) and its Triton split kernel (attention/triton_decode.py),
installed untouched into ``baseline/_ref`` with

    TORCH_CUDA_ARCH_LIST=10.0 python -m pip install --no-index --no-build-isolation --no-deps \
        --target baseline/_ref <copy of the reference checkout>

Both run on the same seeded synthetic workloads as ``bench.py``; outputs are
compared with this library's before timing.  Usage:

    python baseline/compare_reference_gpu.py [workload ... | prefill | mla]
"""

from __future__ import annotations

import json
import statistics
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import attention_b200 as ours  # noqa: E402
from attention_b200 import synth  # noqa: E402

TOL = {torch.float32: 1e-4, torch.float16: 2e-3, torch.bfloat16: 1e-2}


def load_reference():
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "attention").is_dir():
        return None, "baseline/_ref is not installed"
    sys.path.insert(0, str(ref_dir))
    try:
        import attention as ref
    except Exception as exc:   # noqa: BLE001 - report whatever the import raised
        return None, f"import failed: {exc}"
    if not ref.is_cuda_extension_loaded():
        return None, "the reference's CUDA extension did not load"
    return ref, None


def time_call(fn, min_seconds=0.2, reps=20):
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < min_seconds:
        fn()
        torch.cuda.synchronize()
    samples = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        b.synchronize()
        samples.append(a.elapsed_time(b) * 1e3 / reps)
    return statistics.median(samples)


def compare_prefill(ref):
    """Dense prefill: this library vs the reference's CUDA kernels and its Triton backend."""
    for b, t in ((8, 1024), (4, 4096)):
        gen = torch.Generator(device="cuda").manual_seed(42)
        q = torch.empty(b, t, 32, 128, device="cuda", dtype=torch.bfloat16).normal_(generator=gen)
        k = torch.empty(b, t, 8, 128, device="cuda", dtype=torch.bfloat16).normal_(generator=gen)
        v = torch.empty(b, t, 8, 128, device="cuda", dtype=torch.bfloat16).normal_(generator=gen)
        lens = torch.full((b,), t, dtype=torch.int32, device="cuda")
        flops = 4.0 * b * 32 * 128 * t * t * 0.5
        mine = ours.gqa_prefill(q, k, v, lens, lens)
        row = {"workload": f"prefill B{b} T{t} 32/8 D128 bf16 causal"}
        legs = {
            "b200": lambda: ours.gqa_prefill(q, k, v, lens, lens),
            "ref_cuda": lambda: ref.gqa_prefill(q, k, v, lens, lens),
            "ref_triton_tensorcore": lambda: ref.gqa_prefill(q, k, v, lens, lens, backend="tensorcore"),
        }
        for leg, fn in legs.items():
            try:
                out = fn()
                torch.cuda.synchronize()
                close = torch.allclose(out.float(), mine.float(), atol=2e-2, rtol=2e-2)
                us = time_call(fn, reps=10 if leg == "b200" else 2)
                row[leg] = {"us": round(us, 1), "TFLOPs": round(flops / us / 1e6, 1),
                            "max_abs_diff_vs_b200": (out.float() - mine.float()).abs().max().item(),
                            "close": bool(close)}
            except Exception as exc:   # noqa: BLE001
                row[leg] = {"error": str(exc)[:200]}
        print(json.dumps(row), flush=True)


def compare_mla(ref):
    """Paged latent (MLA) decode: this library vs the reference's fused CUDA operator
    (attention/mla.py:43-53) on the synthetic MLA workloads."""
    # the shapes of the reference's own MLA decode timing (benchmarks/bench_tensorcore_followup.py:25-28:
    # one sequence, 4 heads, Dn 32, Dr 16, Dc 64, Dv 32, page 16, bf16, L = 512 / 1024 / 4096)
    small = {f"ref_bench_L{n}": synth.MlaWorkload(f"ref_bench_L{n}", 1, 1, 4, 32, 16, 64, 32, 16, torch.bfloat16, n, n)
             for n in (512, 1024, 4096)}
    for name in ("m2_deepseek_h128_bf16", "m3_deepseek_h16_bf16", *small):
        w = small.get(name) or synth.MLA_WORKLOADS[name]
        c = synth.make_mla_case(w, seed=42, device="cuda", cache_on_device=True)
        nbytes = synth.mla_algorithmic_bytes(c["lengths"].cpu(), w)
        args = (c["q_nope"], c["q_rope"], c["cache"], c["block_table"], c["lengths"], c["positions"],
                c["w_uk"], c["w_uv"])
        mine = ours.mla_decode(*args)
        row = {"workload": name, "algorithmic_MB": round(nbytes / 1e6, 1)}
        legs = {"b200_mla_decode": lambda: ours.mla_decode(*args),
                "ref_cuda_mla_decode": lambda: ref.mla_decode(*args)}
        for leg, fn in legs.items():
            try:
                out = fn()
                torch.cuda.synchronize()
                err = (out.float() - mine.float()).abs().max().item()
                close = torch.allclose(out.float(), mine.float(), atol=2e-2, rtol=2e-2)
                us = time_call(fn, reps=10 if leg.startswith("b200") else 1, min_seconds=0.05)
                row[leg] = {"us": round(us, 1), "GBps": round(nbytes / us / 1e3, 1),
                            "max_abs_diff_vs_b200": err, "close": bool(close)}
            except Exception as exc:   # noqa: BLE001
                row[leg] = {"error": str(exc)[:200]}
        print(json.dumps(row), flush=True)


def main():
    if "mla" in sys.argv[1:]:
        ref, why = load_reference()
        if ref is None:
            print(json.dumps({"unavailable": why}))
            return
        compare_mla(ref)
        return
    names = [a for a in sys.argv[1:] if a != "prefill"] or (
        [] if "prefill" in sys.argv[1:] else list(synth.WORKLOADS))
    ref, why = load_reference()
    if ref is None:
        print(json.dumps({"unavailable": why}))
        return
    if "prefill" in sys.argv[1:] or not sys.argv[1:]:
        compare_prefill(ref)
    for name in names:
        w = synth.WORKLOADS[name]
        q, k, v, table, lens = synth.make_workload(w, seed=42, device="cuda", kv_on_device=True)
        nbytes = synth.algorithmic_bytes(lens.cpu(), batch=w.batch, q_heads=w.q_heads,
                                         kv_heads=w.kv_heads, head_dim=w.head_dim,
                                         elem_size=q.element_size())
        mine = ours.gqa_decode(q, k, v, table, lens)
        tol = TOL[w.dtype]
        row = {"workload": name, "algorithmic_MB": round(nbytes / 1e6, 1)}
        legs = {
            "b200": lambda: ours.gqa_decode(q, k, v, table, lens),
            "ref_cuda": lambda: ref.gqa_decode(q, k, v, table, lens),
            "ref_triton_auto": lambda: ref.gqa_decode_auto(q, k, v, table, lens),
            "ref_triton_split16": lambda: ref.gqa_decode_split(q, k, v, table, lens, splits=16,
                                                               backend="triton"),
        }
        for leg, fn in legs.items():
            try:
                out = fn()
                torch.cuda.synchronize()
                err = (out.float() - mine.float()).abs().max().item()
                close = torch.allclose(out.float(), mine.float(), atol=2 * tol, rtol=2 * tol)
                reps = 20 if leg == "b200" else 3
                us = time_call(fn, reps=reps)
                row[leg] = {"us": round(us, 1), "GBps": round(nbytes / us / 1e3, 1),
                            "max_abs_diff_vs_b200": err, "close": bool(close)}
            except Exception as exc:   # noqa: BLE001 - a leg that cannot run is reported, not fatal
                row[leg] = {"error": str(exc)[:200]}
        # the reference's own Python/torch oracle on the host cores, on a bounded sample
        try:
            n = min(w.batch, 8)
            cq, ct, cl = q[:n].cpu(), table[:n].cpu(), lens[:n].cpu()
            ck, cv = k.cpu(), v.cpu()
            sample_bytes = synth.algorithmic_bytes(cl, batch=n, q_heads=w.q_heads,
                                                   kv_heads=w.kv_heads, head_dim=w.head_dim,
                                                   elem_size=q.element_size())
            ref.reference_gqa_decode(cq[:1], ck, cv, ct[:1], cl[:1])
            t0 = time.perf_counter()
            ref.reference_gqa_decode(cq, ck, cv, ct, cl)
            dt = time.perf_counter() - t0
            row["ref_python_oracle_cpu"] = {"seconds": round(dt, 3), "sequences": n,
                                            "GBps": round(sample_bytes / dt / 1e9, 3),
                                            "threads": torch.get_num_threads()}
        except Exception as exc:   # noqa: BLE001
            row["ref_python_oracle_cpu"] = {"error": str(exc)[:200]}
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
