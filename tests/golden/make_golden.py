"""Generate the golden fixtures by running the REFERENCE's own oracle.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports ``attention.reference_gqa_decode`` (attention/reference/gqa.py:7-44)
and the reference's fixture generator ``make_decode_case``
(benchmarks/data.py:8-43) from that checkout, and writes

  full_*.npz   small cases with every input stored next to the reference output
  prefill_*.npz dense prefill cases, inputs stored in full
  mla_*.npz    paged latent (MLA) decode cases, inputs stored in full
  seed_*.npz   larger cases: only the generator arguments, a sha256 of the
               regenerated inputs, and the reference output are stored; a test
               regenerates the inputs from the seed, checks the digest, then
               compares

The reference is only needed to (re)generate; the tests read the .npz files.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE.parents[1]))

from golden_io import digest, to_np  # noqa: E402

from attention_b200 import synth  # noqa: E402


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, str(Path(ref_root) / "benchmarks"))
    from attention import reference_gqa_decode  # the reference's oracle
    from data import make_decode_case           # the reference's fixture generator

    torch.set_num_threads(8)

    # ---- small cases, inputs stored in full (reference generator) ----------
    full_cases = [
        # name, lengths, q_heads, kv_heads, head_dim, block_size, dtype, seed, scale
        ("full_f32_g3_d32_bs4", [0, 1, 3, 4, 5, 9], 6, 2, 32, 4, torch.float32, 42, None),
        ("full_bf16_g4_d128_bs16", [40, 7, 64], 8, 2, 128, 16, torch.bfloat16, 7, None),
        ("full_f16_g7_d128_bs16", [33, 16, 1], 7, 1, 128, 16, torch.float16, 11, None),
        ("full_f16_mha_d64_bs8", [0, 17, 8, 23], 4, 4, 64, 8, torch.float16, 3, 0.2),
        ("full_f32_mqa_d80_bs5", [12, 5, 6], 5, 1, 80, 5, torch.float32, 5, None),
        ("full_bf16_g8_d256_bs32", [70, 32], 16, 2, 256, 32, torch.bfloat16, 9, None),
    ]
    for name, lengths, hq, hkv, d, bs, dtype, seed, scale in full_cases:
        q, k, v, table, lens = make_decode_case(lengths=lengths, q_heads=hq, kv_heads=hkv,
                                                head_dim=d, block_size=bs, dtype=dtype, seed=seed)
        out = reference_gqa_decode(q, k, v, table, lens, scale=scale)
        np.savez_compressed(
            HERE / f"{name}.npz", q=to_np(q), k=to_np(k), v=to_np(v), table=to_np(table),
            lens=to_np(lens), out=to_np(out), dtype=str(dtype).replace("torch.", ""),
            scale=np.float64(-1.0 if scale is None else scale))
        print(name, tuple(out.shape))

    # ---- seeded cases (this library's workload generator) ------------------
    seeded = [
        ("seed_c1_cpu_fp32", synth.WORKLOADS["c1_cpu_fp32"], 42),
        ("seed_c2_small_bf16", synth.scaled("c2_qwen3_8b_bf16", batch=3, len_lo=500, len_hi=1200), 42),
        ("seed_c3_small_fp16", synth.scaled("c3_qwen25_7b_fp16", batch=4, len_lo=100, len_hi=700), 42),
        ("seed_c4_small_bf16", synth.scaled("c4_longctx_bf16", batch=2, len_lo=3000, len_hi=5000), 42),
        ("seed_c5_small_bf16", synth.scaled("c5_skewed_bf16", batch=12, len_hi=4096), 42),
    ]
    for name, w, seed in seeded:
        q, k, v, table, lens = synth.make_workload(w, seed=seed)
        out = reference_gqa_decode(q, k, v, table, lens)
        np.savez_compressed(
            HERE / f"{name}.npz", out=to_np(out), lens=to_np(lens),
            dtype=str(w.dtype).replace("torch.", ""), seed=np.int64(seed),
            digest=digest(q, k, v, table, lens),
            workload=np.array([w.batch, w.q_heads, w.kv_heads, w.head_dim, w.block_size,
                               w.len_lo, w.len_hi, w.fixed_pool_blocks], dtype=np.int64),
            len_dist=w.len_dist)
        print(name, tuple(out.shape), lens.tolist()[:8])


def prefill_cases(ref_root: str) -> None:
    """Dense prefill fixtures from the reference's ``reference_gqa_prefill``
    (attention/reference/gqa.py:47-64): inputs stored in full."""
    sys.path.insert(0, ref_root)
    from attention.reference.gqa import reference_gqa_prefill

    cases = [
        # name, B, Tq, Tk, Hq, Hkv, D, dtype, q_lens, kv_lens, causal, scale, seed
        ("prefill_f32_causal_d32", 3, 9, 12, 6, 2, 32, torch.float32, [9, 4, 0], [12, 4, 7], True, None, 1),
        ("prefill_bf16_causal_d128", 2, 40, 40, 8, 2, 128, torch.bfloat16, [40, 17], [40, 17], True, None, 2),
        ("prefill_f16_noncausal_d64", 2, 20, 33, 4, 4, 64, torch.float16, [20, 5], [33, 30], False, 0.2, 3),
        ("prefill_bf16_qlonger_d128", 2, 70, 50, 7, 1, 128, torch.bfloat16, [70, 33], [50, 40], True, None, 4),
        ("prefill_f16_chunked_d128", 2, 16, 200, 8, 2, 128, torch.float16, [16, 9], [200, 137], True, None, 5),
        ("prefill_f32_mqa_d80", 2, 11, 11, 5, 1, 80, torch.float32, [11, 6], [11, 6], True, None, 6),
    ]
    for name, b, tq, tk, hq, hkv, d, dtype, ql, kl, causal, scale, seed in cases:
        gen = torch.Generator().manual_seed(seed)
        q = torch.randn(b, tq, hq, d, generator=gen).to(dtype)
        k = torch.randn(b, tk, hkv, d, generator=gen).to(dtype)
        v = torch.randn(b, tk, hkv, d, generator=gen).to(dtype)
        q_lens = torch.tensor(ql, dtype=torch.int32)
        kv_lens = torch.tensor(kl, dtype=torch.int32)
        out = reference_gqa_prefill(q, k, v, q_lens, kv_lens, causal=causal, scale=scale)
        np.savez_compressed(
            HERE / f"{name}.npz", q=to_np(q), k=to_np(k), v=to_np(v), q_lens=to_np(q_lens),
            kv_lens=to_np(kv_lens), out=to_np(out), dtype=str(dtype).replace("torch.", ""),
            causal=np.int64(1 if causal else 0), scale=np.float64(-1.0 if scale is None else scale))
        print(name, tuple(out.shape))


def mla_cases(ref_root: str) -> None:
    """Paged MLA decode fixtures.  The reference's oracle ``mla_reference``
    (attention/reference/mla.py:6-34, ``absorbed=True``) takes dense ``[B,L,*]`` latents, so the
    pages of each synthetic cache are gathered through the block table here before the call;
    the fixture stores the paged inputs and the reference output."""
    sys.path.insert(0, ref_root)
    from attention.reference.mla import mla_reference

    W = synth.MlaWorkload
    cases = [
        # name, workload, lengths, positions override, indices (K or None), all-visible positions, seed
        ("mla_f32_small", W("g", 2, 1, 4, 16, 8, 32, 16, 16, torch.float32, 0, 0), [64, 37], None, None, False, 11),
        ("mla_f16_multiquery", W("g", 3, 3, 4, 32, 16, 64, 32, 8, torch.float16, 0, 0), [50, 9, 0],
         [[47, 48, 49], [2, -1, 8], [0, 1, 2]], None, False, 12),
        ("mla_f32_sparse", W("g", 2, 2, 3, 16, 8, 32, 16, 4, torch.float32, 0, 0), [30, 21], None, 12, False, 13),
        ("mla_bf16_wide", W("g", 2, 1, 4, 32, 64, 512, 32, 32, torch.bfloat16, 0, 0), [100, 40], None, None, False, 14),
        ("mla_bf16_allvisible", W("g", 2, 2, 5, 16, 16, 128, 16, 16, torch.bfloat16, 0, 0), [33, 80], None, None, True, 15),
    ]
    for name, w, lens, pos, nk, all_visible, seed in cases:
        c = synth.make_mla_case(w, seed=seed, lengths=lens)
        if pos is not None:
            c["positions"] = torch.tensor(pos, dtype=torch.int32)
        cap = c["block_table"].shape[1] * w.page
        ref_pos = torch.full_like(c["positions"], cap) if all_visible else c["positions"]
        indices = None
        if nk is not None:
            gen = torch.Generator().manual_seed(seed + 100)
            rows = []
            for b in range(w.batch):
                for t in range(w.tq):
                    ix = torch.randperm(cap, generator=gen)[:nk].to(torch.int32)   # unique; some past len
                    ix[torch.randint(0, nk, (2,), generator=gen)] = -1             # ignored entries
                    rows.append(ix)
            indices = torch.stack(rows).view(w.batch, w.tq, nk)
        used = (c["lengths"].to(torch.int64) + w.page - 1) // w.page
        safe = torch.where(torch.arange(c["block_table"].shape[1])[None, :] < used[:, None],
                           c["block_table"].to(torch.int64), torch.zeros((), dtype=torch.int64))
        dense = c["cache"][safe.reshape(-1)].reshape(w.batch, cap, w.dc + w.dr)
        out = mla_reference(c["q_nope"], c["q_rope"], dense[..., :w.dc].contiguous(),
                            dense[..., w.dc:].contiguous(), c["w_uk"], c["w_uv"], ref_pos, c["lengths"],
                            absorbed=True, indices=indices)
        arrays = {k: to_np(v) for k, v in c.items()}
        if indices is not None:
            arrays["indices"] = to_np(indices)
        np.savez_compressed(HERE / f"{name}.npz", out=to_np(out), dtype=str(w.dtype).replace("torch.", ""),
                            causal=np.int64(0 if all_visible else 1), **arrays)
        print(name, tuple(out.shape))


if __name__ == "__main__":
    paths = [a for a in sys.argv[1:] if not a.startswith("--")]
    if not paths:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference [--mla-only | --prefill-only]")
    mla_cases(paths[0])
    if "--mla-only" in sys.argv:
        sys.exit(0)
    prefill_cases(paths[0])
    if "--prefill-only" in sys.argv:
        sys.exit(0)
    main(paths[0])
