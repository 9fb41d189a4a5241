"""Seeded synthetic decode workloads (page pools, block tables, lengths).

The layout conventions are those of the reference's fixture generator
(benchmarks/data.py:8-43): q/K/V drawn from N(0,1) in fp32 then cast, physical
pages handed out from a random permutation so that logical and physical page
order differ, and every table slot past a sequence's used pages set to -1.

Five named workloads mirror the benchmark configurations this library is
measured on.  "Qwen3-8B-shape" and "Qwen2.5-7B-shape" only borrow head counts;
no model weights, prompts or datasets are involved anywhere.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class DecodeWorkload:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int
    block_size: int
    dtype: torch.dtype
    len_lo: int
    len_hi: int
    len_dist: str = "uniform"          # "uniform" | "lognormal"
    lognormal_mu: float = 7.0
    lognormal_sigma: float = 1.2
    pool_factor: float = 1.25          # physical pool = ceil(factor * pages needed)
    fixed_pool_blocks: int = 0         # >0 overrides pool_factor


WORKLOADS = {
    "c1_cpu_fp32": DecodeWorkload("c1_cpu_fp32", 4, 32, 8, 128, 16, torch.float32, 64, 512,
                                  fixed_pool_blocks=128),
    "c2_qwen3_8b_bf16": DecodeWorkload("c2_qwen3_8b_bf16", 64, 32, 8, 128, 16, torch.bfloat16,
                                       1024, 4096),
    "c3_qwen25_7b_fp16": DecodeWorkload("c3_qwen25_7b_fp16", 128, 28, 4, 128, 16, torch.float16,
                                        256, 2048),
    "c4_longctx_bf16": DecodeWorkload("c4_longctx_bf16", 8, 64, 8, 128, 32, torch.bfloat16,
                                      32768, 131072),
    "c5_skewed_bf16": DecodeWorkload("c5_skewed_bf16", 256, 40, 8, 128, 16, torch.bfloat16,
                                     16, 32768, len_dist="lognormal"),
}


def draw_lengths(w: DecodeWorkload, gen: torch.Generator) -> torch.Tensor:
    """int32 [batch] context lengths from the workload's distribution (CPU generator)."""
    if w.len_dist == "uniform":
        lens = torch.randint(w.len_lo, w.len_hi + 1, (w.batch,), generator=gen)
    elif w.len_dist == "lognormal":
        x = torch.empty(w.batch, dtype=torch.float64).log_normal_(
            w.lognormal_mu, w.lognormal_sigma, generator=gen)
        lens = x.round().clamp_(w.len_lo, w.len_hi).to(torch.int64)
    else:
        raise ValueError(f"unknown length distribution {w.len_dist!r}")
    return lens.to(torch.int32)


def build_block_table(lens: torch.Tensor, block_size: int, pool_blocks: int,
                      gen: torch.Generator) -> torch.Tensor:
    """[B, max_pages] int32: used slots take distinct physical pages from a random
    permutation of the pool, unused slots are -1."""
    pages = [(int(n) + block_size - 1) // block_size for n in lens.tolist()]
    need = sum(pages)
    if pool_blocks < need:
        raise ValueError("pool smaller than the pages in use")
    max_pages = max(1, max(pages) if pages else 1)
    perm = torch.randperm(pool_blocks, generator=gen, dtype=torch.int64)[:need].to(torch.int32)
    table = torch.full((len(pages), max_pages), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages):
        table[b, :n] = perm[at:at + n]
        at += n
    return table


def pool_blocks_for(w: DecodeWorkload, lens: torch.Tensor) -> int:
    need = sum((int(n) + w.block_size - 1) // w.block_size for n in lens.tolist())
    if w.fixed_pool_blocks:
        return max(w.fixed_pool_blocks, need)
    return max(1, math.ceil(w.pool_factor * need))


def threaded_normal(shape, dtype: torch.dtype, seed: int, threads: int = 0) -> torch.Tensor:
    """A CPU tensor of N(0,1) draws filled by several threads, each with its own seeded
    generator over a fixed slice (deterministic for a given seed, whatever the thread count).
    One generator fills about 40 M elements a second; multi-GB page pools for the timed CPU
    baseline would otherwise take most of a minute to draw."""
    import os
    from concurrent.futures import ThreadPoolExecutor
    out = torch.empty(shape, dtype=dtype)
    flat = out.view(-1)
    n = flat.numel()
    step = 1 << 24
    threads = threads or len(os.sched_getaffinity(0))

    def fill(i):
        g = torch.Generator().manual_seed(seed * 1000003 + i)
        flat[i * step:(i + 1) * step].normal_(generator=g)

    with ThreadPoolExecutor(max(1, threads)) as ex:
        list(ex.map(fill, range((n + step - 1) // step)))
    return out


def _draw_tensors(w: DecodeWorkload, lens: torch.Tensor, gen: torch.Generator, seed: int, device,
                  kv_on_device: bool, kv_threaded: bool = False):
    """q, K, V and the page table for given lengths, drawn in that order from ``gen``."""
    q = torch.randn(w.batch, w.q_heads, w.head_dim, generator=gen, dtype=torch.float32)
    pool = pool_blocks_for(w, lens)
    shape = (pool, w.block_size, w.kv_heads, w.head_dim)
    if kv_on_device:
        dgen = torch.Generator(device=device).manual_seed(seed)
        k = torch.empty(shape, dtype=w.dtype, device=device).normal_(generator=dgen)
        v = torch.empty(shape, dtype=w.dtype, device=device).normal_(generator=dgen)
    elif kv_threaded:
        k = threaded_normal(shape, w.dtype, 2 * seed).to(device)
        v = threaded_normal(shape, w.dtype, 2 * seed + 1).to(device)
    else:
        k = torch.randn(shape, generator=gen, dtype=torch.float32).to(w.dtype).to(device)
        v = torch.randn(shape, generator=gen, dtype=torch.float32).to(w.dtype).to(device)
    table = build_block_table(lens, w.block_size, pool, gen)
    return (q.to(device=device, dtype=w.dtype).contiguous(), k.contiguous(), v.contiguous(),
            table.to(device).contiguous(), lens.to(device))


def make_workload(w: DecodeWorkload | str, *, seed: int = 42, device="cpu",
                  kv_on_device: bool = False):
    """Returns (q, k_cache, v_cache, block_table, context_lens) for a workload.

    Draw order with one CPU generator seeded with ``seed``: lengths, q, K, V,
    page permutation.  With ``kv_on_device`` the two page pools are drawn by a
    generator of the target device seeded with ``seed`` instead (multi-GB pools
    take tens of seconds to draw on a CPU); lengths, q and the table are the
    same either way.
    """
    if isinstance(w, str):
        w = WORKLOADS[w]
    gen = torch.Generator(device="cpu").manual_seed(seed)
    lens = draw_lengths(w, gen)
    return _draw_tensors(w, lens, gen, seed, device, kv_on_device)


def make_workload_for_lengths(w: DecodeWorkload | str, lens: torch.Tensor, *, seed: int = 42,
                              device="cpu", kv_on_device: bool = False, kv_threaded: bool = False):
    """Like ``make_workload`` but for given context lengths (e.g. one rank's share of a batch):
    batch = len(lens), a private page pool of ``pool_factor`` x the pages those lengths need.
    ``kv_threaded`` draws CPU page pools with ``threaded_normal`` (fast, for timing baselines).
    Returns (the resized workload, the five tensors)."""
    if isinstance(w, str):
        w = WORKLOADS[w]
    lens = lens.to(torch.int32).cpu()
    w = replace(w, batch=int(lens.numel()), fixed_pool_blocks=0)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return w, _draw_tensors(w, lens, gen, seed, device, kv_on_device, kv_threaded)


def scaled(w: DecodeWorkload | str, **changes) -> DecodeWorkload:
    """A copy of a workload with some fields replaced (smaller batch, shorter lengths...)."""
    if isinstance(w, str):
        w = WORKLOADS[w]
    return replace(w, **changes)


def algorithmic_bytes(context_lens: torch.Tensor, *, batch: int, q_heads: int, kv_heads: int,
                      head_dim: int, elem_size: int) -> int:
    """Bytes one decode call must move: every used K and V row once, q in, out back.

    sum(context_len) * kv_heads * head_dim * 2 * elem_size + 2 * B * Hq * D * elem_size.
    Block-table reads, split partials and page-tail padding are not counted.
    """
    tokens = int(context_lens.to(torch.int64).sum().item())
    return tokens * kv_heads * head_dim * 2 * elem_size + 2 * batch * q_heads * head_dim * elem_size


# ---------------------------------------------------------------------------
# paged latent (MLA) decode workloads
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class MlaWorkload:
    name: str
    batch: int
    tq: int                # query tokens per sequence (1 = plain decode)
    heads: int
    dn: int                # no-rope query width
    dr: int                # rotated width
    dc: int                # compressed latent width
    dv: int                # value width per head
    page: int
    dtype: torch.dtype
    len_lo: int
    len_hi: int
    pool_factor: float = 1.25


# "DeepSeek-shape" borrows only the published head geometry (128 heads, 512 + 64 wide
# latent rows); no weights, prompts or datasets are involved.
MLA_WORKLOADS = {
    "m1_small_fp32": MlaWorkload("m1_small_fp32", 2, 1, 4, 16, 8, 32, 16, 16, torch.float32, 20, 64),
    "m2_deepseek_h128_bf16": MlaWorkload("m2_deepseek_h128_bf16", 64, 1, 128, 128, 64, 512, 128, 64,
                                         torch.bfloat16, 1024, 4096),
    "m3_deepseek_h16_bf16": MlaWorkload("m3_deepseek_h16_bf16", 128, 1, 16, 128, 64, 512, 128, 64,
                                        torch.bfloat16, 1024, 8192),
    "m4_deepseek_h128_long_bf16": MlaWorkload("m4_deepseek_h128_long_bf16", 16, 1, 128, 128, 64, 512, 128, 64,
                                              torch.bfloat16, 16384, 65536),
}


def make_mla_case(w: MlaWorkload | str, *, seed: int = 42, device="cpu", lengths=None,
                  cache_on_device: bool = False):
    """A dict of tensors for one MLA decode call.

    Draw order with one CPU generator seeded with ``seed``: lengths (unless given), q_nope,
    q_rope, W_uk / sqrt(Dn), W_uv / sqrt(Dc), the page pool, the page permutation.  The weight
    scaling follows the reference's benchmark fixtures (benchmarks/bench_attention_primitives.py:52).
    positions[b, t] = len_b - tq + t, the last tq tokens of each sequence.
    """
    if isinstance(w, str):
        w = MLA_WORKLOADS[w]
    gen = torch.Generator(device="cpu").manual_seed(seed)
    if lengths is None:
        lens = torch.randint(w.len_lo, w.len_hi + 1, (w.batch,), generator=gen).to(torch.int32)
    else:
        lens = torch.as_tensor(lengths, dtype=torch.int32)
    q_nope = torch.randn(w.batch, w.tq, w.heads, w.dn, generator=gen)
    q_rope = torch.randn(w.batch, w.tq, w.heads, w.dr, generator=gen)
    w_uk = torch.randn(w.heads, w.dn, w.dc, generator=gen) / math.sqrt(w.dn)
    w_uv = torch.randn(w.heads, w.dv, w.dc, generator=gen) / math.sqrt(w.dc)
    need = sum((int(n) + w.page - 1) // w.page for n in lens.tolist())
    pool = max(1, math.ceil(w.pool_factor * need))
    shape = (pool, w.page, w.dc + w.dr)
    if cache_on_device:
        dgen = torch.Generator(device=device).manual_seed(seed)
        cache = torch.empty(shape, dtype=w.dtype, device=device).normal_(generator=dgen)
    else:
        cache = torch.randn(shape, generator=gen).to(w.dtype).to(device)
    table = build_block_table(lens, w.page, pool, gen)
    positions = (lens[:, None].to(torch.int64) - w.tq + torch.arange(w.tq)[None, :]).to(torch.int32)
    to = lambda t: t.to(device=device, dtype=w.dtype).contiguous()   # noqa: E731
    return {
        "q_nope": to(q_nope), "q_rope": to(q_rope), "w_uk": to(w_uk), "w_uv": to(w_uv),
        "cache": cache.contiguous(), "block_table": table.to(device).contiguous(),
        "lengths": lens.to(device), "positions": positions.to(device).contiguous(),
    }


def mla_algorithmic_bytes(lengths: torch.Tensor, w: MlaWorkload) -> int:
    """Bytes one latent-attention call must move: every visible cache row once, the absorbed
    and rotated queries in, the latent output back.  Page tables and split partials are not counted."""
    es = torch.empty((), dtype=w.dtype).element_size()
    tokens = int(lengths.to(torch.int64).sum().item())
    rows = w.batch * w.tq * w.heads
    return tokens * (w.dc + w.dr) * es + rows * (w.dc + w.dr) * es + rows * w.dc * es


def scaled_mla(w: MlaWorkload | str, **changes) -> MlaWorkload:
    """A copy of an MLA workload with some fields replaced."""
    if isinstance(w, str):
        w = MLA_WORKLOADS[w]
    return replace(w, **changes)
