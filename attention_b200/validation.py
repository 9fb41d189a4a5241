"""Opt-in, synchronising checks of caller-owned paging metadata (debugging aid).

Mirrors the reference's ``validate_paged_metadata`` (attention/validation.py:5-39):
the decode and append operators trust the block table, lengths and positions
they are given; this function is how a caller checks them, at the price of a
device-to-host copy.
"""

from __future__ import annotations

import torch


def validate_paged_metadata(block_table, context_lens, *, block_size, num_blocks, positions=None):
    """Raise ValueError on the first inconsistency.

    * shapes [B, max_pages] / [B], both int32
    * 0 <= context_len <= max_pages * block_size
    * every page a sequence uses is in [0, num_blocks) (unused slots are not looked at)
    * with ``positions`` (int32 [B]): each append position is inside the table, lands on a
      valid page, and no two sequences write the same (page, slot)
    """
    if block_size <= 0 or num_blocks <= 0:
        raise ValueError("block_size and num_blocks must be positive")
    if block_table.ndim != 2 or context_lens.ndim != 1 or block_table.shape[0] != context_lens.numel():
        raise ValueError("metadata shapes must be [B,MaxPages] and [B]")
    if block_table.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise ValueError("metadata must be int32")
    if positions is not None and (positions.shape != context_lens.shape
                                  or positions.dtype != torch.int32):
        raise ValueError("positions must be int32 [B]")
    table = block_table.detach().cpu()
    lens = context_lens.detach().cpu().to(torch.int64)
    max_pages = table.shape[1]
    cap = max_pages * block_size
    bad = ((lens < 0) | (lens > cap)).nonzero()
    if bad.numel():
        raise ValueError(f"invalid length at batch {int(bad[0])}")
    used = (lens + block_size - 1) // block_size
    cols = torch.arange(max_pages).unsqueeze(0)
    in_use = cols < used.unsqueeze(1)
    wrong = in_use & ((table < 0) | (table >= num_blocks))
    if wrong.any():
        b, p = (int(x) for x in wrong.nonzero()[0])
        raise ValueError(f"invalid block at batch {b}, page {p}")
    if positions is not None:
        pos = positions.detach().cpu().to(torch.int64)
        off = ((pos < 0) | (pos >= cap)).nonzero()
        if off.numel():
            raise ValueError(f"invalid append position at batch {int(off[0])}")
        page = table.gather(1, (pos // block_size).unsqueeze(1)).squeeze(1).to(torch.int64)
        badpage = ((page < 0) | (page >= num_blocks)).nonzero()
        if badpage.numel():
            raise ValueError(f"invalid append page at batch {int(badpage[0])}")
        dest = page * block_size + pos % block_size
        if dest.unique().numel() != dest.numel():
            raise ValueError("conflicting append destinations")
