"""Batch sharding of a paged decode workload across the GPUs of one box.

Sequences are independent (each output row depends only on its own q row, pages
and length), so the batch is partitioned and every rank owns its own page pool
with locally renumbered block ids and its own block table / lengths.  The
forward pass needs no collective; only a harness gathers outputs afterwards.
"""

from __future__ import annotations

import heapq

import torch


def lpt_assign(lengths, world_size: int) -> list[list[int]]:
    """Greedy longest-processing-time-first: sequence ids per rank.

    Deterministic (ties broken by sequence id, then by rank id); every rank's list is
    sorted by sequence id.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    heap = [(0, r) for r in range(world_size)]
    heapq.heapify(heap)
    shards: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        load, r = heapq.heappop(heap)
        shards[r].append(i)
        heapq.heappush(heap, (load + int(lengths[i]), r))
    return [sorted(s) for s in shards]


def load_imbalance(lengths, shards) -> float:
    """max over ranks of assigned tokens divided by the mean (1.0 = perfect)."""
    loads = [sum(int(lengths[i]) for i in s) for s in shards]
    mean = sum(loads) / max(1, len(loads))
    return max(loads) / mean if mean > 0 else 1.0


def extract_shard(q, k_cache, v_cache, block_table, context_lens, seq_ids, *, device=None):
    """The rank-local workload for ``seq_ids``: (q, k_pool, v_pool, table, lens).

    The local pool holds exactly the pages those sequences use, renumbered 0..n-1 in
    (sequence, logical page) order; unused table slots stay -1.  ``device`` moves the result.
    """
    ids = torch.as_tensor(seq_ids, dtype=torch.int64)
    block_size = k_cache.shape[1]
    lens = context_lens.cpu()[ids]
    table = block_table.cpu()[ids]
    used = (lens.to(torch.int64) + block_size - 1) // block_size
    max_pages = max(1, int(used.max()) if used.numel() else 1)
    local_table = torch.full((len(ids), max_pages), -1, dtype=torch.int32)
    src_pages = []
    at = 0
    for row, n in enumerate(used.tolist()):
        src_pages.append(table[row, :n].to(torch.int64))
        local_table[row, :n] = torch.arange(at, at + n, dtype=torch.int32)
        at += n
    if src_pages and at > 0:
        src = torch.cat(src_pages).to(k_cache.device)
        k_local = k_cache.index_select(0, src)
        v_local = v_cache.index_select(0, src)
    else:   # a rank with no tokens still needs a non-empty pool for the operator's checks
        k_local = torch.zeros((1,) + tuple(k_cache.shape[1:]), dtype=k_cache.dtype, device=k_cache.device)
        v_local = torch.zeros_like(k_local)
    q_local = q[ids.to(q.device)]
    outs = (q_local.contiguous(), k_local.contiguous(), v_local.contiguous(), local_table, lens.to(torch.int32))
    if device is not None:
        outs = tuple(t.to(device) for t in outs)
    return outs


def scatter_outputs(parts, shards, batch: int) -> torch.Tensor:
    """Reassemble per-rank outputs ([len(shard), Hq, D] each) into [batch, Hq, D]."""
    ref = next(p for p in parts if p.numel() or True)
    out = torch.zeros((batch,) + tuple(ref.shape[1:]), dtype=ref.dtype, device=ref.device)
    for part, ids in zip(parts, shards):
        if len(ids):
            out[torch.as_tensor(ids, dtype=torch.int64, device=out.device)] = part.to(out.device)
    return out
