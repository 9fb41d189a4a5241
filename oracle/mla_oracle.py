"""CPU oracle for paged multi-head latent attention (MLA) decode.  TEST INFRASTRUCTURE ONLY.

Restates, on the CPU, the arithmetic of the reference library's slow oracle
``mla_reference`` (attention/reference/mla.py:6-34) plus the page gather that
the reference's CUDA operators do on the fly (csrc/cuda/mla/mla.cu:34-56).
Nothing in the shipped package imports this module; the tests, the smoke check
and the CPU leg of the benchmark use it as the checker only.

Parity pin: ``tests/golden/mla_*.npz`` hold outputs of the reference's own
``mla_reference`` produced by importing the reference
(``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` compares
the functions below against them.

Conventions (attention/mla.py:1-6): the paged cache is ``[blocks, page, Dc+Dr]``
with the compressed latent in the first Dc columns and the rotated key part in
the last Dr; ``positions`` are absolute int32 ``[B,T]``; a query row attends to
logical tokens ``s < end`` with ``end = min(len, max(0, pos+1))`` when causal
and ``end = len`` otherwise (mla.cu:38); with ``indices`` (int32 ``[B,T,K]``)
only the listed tokens that satisfy ``0 <= s < end`` count (mla.cu:45-46);
rows that see no token are zero (mla.cu:55).
"""

from __future__ import annotations

import math

import numpy as np
import torch


def gather_pages(cache: torch.Tensor, block_table: torch.Tensor, lengths: torch.Tensor):
    """Dense ``latent [B,L,Dc+Dr]`` view of a paged cache, L = max_pages * page.

    Table slots past a sequence's used pages may hold any value (the reference
    never reads them); they are gathered from page 0 here and masked later.
    """
    blocks, page, width = cache.shape
    batch, max_pages = block_table.shape
    used = (lengths.to(torch.int64) + page - 1) // page
    slot = torch.arange(max_pages)[None, :]
    safe = torch.where(slot < used[:, None].cpu(), block_table.cpu().to(torch.int64),
                       torch.zeros((), dtype=torch.int64))
    dense = cache.cpu()[safe.reshape(-1)].reshape(batch, max_pages * page, width)
    return dense


def visible_mask(lengths, positions, total, *, causal=True, indices=None):
    """bool ``[B,T,total]``: which logical tokens each query row may attend to."""
    batch, tq = positions.shape
    ids = torch.arange(total).view(1, 1, total)
    mask = ids < lengths.view(batch, 1, 1).to(torch.int64)
    if causal:
        mask = mask & (ids <= positions.view(batch, tq, 1).to(torch.int64))
    if indices is not None:
        chosen = torch.zeros(batch, tq, total, dtype=torch.bool)
        for b in range(batch):
            for t in range(tq):
                ix = indices[b, t].to(torch.int64)
                ix = ix[(ix >= 0) & (ix < total)]
                chosen[b, t, ix] = True
        mask = mask & chosen
    return mask


def _latent_attention_fp32(q_absorbed, q_rope, cache, block_table, lengths, positions, scale, causal, indices):
    dc = q_absorbed.shape[-1]
    dense = gather_pages(cache, block_table, lengths).float()
    lat, rope = dense[..., :dc], dense[..., dc:]
    qa, qr = q_absorbed.cpu().float(), q_rope.cpu().float()
    scores = (torch.einsum("bthc,bsc->bths", qa, lat) + torch.einsum("bthr,bsr->bths", qr, rope)) * scale
    idx = None if indices is None else indices.cpu()
    mask = visible_mask(lengths.cpu(), positions.cpu(), dense.shape[1], causal=causal, indices=idx)[:, :, None, :]
    scores = scores.masked_fill(~mask, float("-inf"))
    seen = mask.any(dim=-1, keepdim=True)
    weights = torch.softmax(torch.where(seen, scores, torch.zeros_like(scores)), dim=-1)
    weights = torch.where(seen, weights, torch.zeros_like(weights))
    return torch.einsum("bths,bsc->bthc", weights, lat)


def reference_mla_latent_attention(q_absorbed, q_rope, cache, block_table, lengths, positions, *,
                                   scale, causal=True, indices=None):
    """Latent output ``[B,T,H,Dc]`` of paged latent attention, fp32 arithmetic.

    score = (q_absorbed . c + q_rope . k_rope) * scale, dense softmax over the
    visible tokens, output = weights . c, rounded once to the input dtype
    (attention/reference/mla.py:13-33 with ``absorbed=True``, before the value
    projection).
    """
    u = _latent_attention_fp32(q_absorbed, q_rope, cache, block_table, lengths, positions, scale, causal,
                               indices)
    return u.to(q_absorbed.dtype)


def reference_mla_decode(q_nope, q_rope, cache, block_table, lengths, positions, w_uk, w_uv, *,
                         scale=None, causal=True, indices=None, round_intermediates=False):
    """Absorbed MLA over a paged cache: ``[B,T,H,Dv]`` in the input dtype.

    q_absorbed = q_nope . W_uk, latent attention as above, out = u . W_uv^T
    (attention/reference/mla.py:10-12,29-31).  The reference oracle keeps the two
    intermediates in fp32; its CUDA operators round both to the input dtype
    (mla.cu:90,105).  ``round_intermediates`` selects the latter.
    """
    if scale is None:
        scale = 1.0 / math.sqrt(q_nope.shape[-1] + q_rope.shape[-1])
    dtype = q_nope.dtype
    qa = torch.einsum("bthd,hdc->bthc", q_nope.cpu().float(), w_uk.cpu().float())
    if round_intermediates:
        qa = qa.to(dtype).float()
    u = _latent_attention_fp32(qa, q_rope, cache, block_table, lengths, positions, scale, causal, indices)
    if round_intermediates:
        u = u.to(dtype).float()
    return torch.einsum("bthc,hvc->bthv", u, w_uv.cpu().float()).to(dtype)


def reference_mla_project(x, w, absorb: bool):
    """Per-head projection (mla.cu:17-27): ``absorb`` contracts x ``[B,T,H,Dn]`` with
    W_uk ``[H,Dn,Dc]``; otherwise x ``[B,T,H,Dc]`` with W_uv ``[H,Dv,Dc]``.  fp32 sum, one rounding."""
    eq = "bthd,hdc->bthc" if absorb else "bthc,hvc->bthv"
    return torch.einsum(eq, x.cpu().float(), w.cpu().float()).to(x.dtype)


def reference_latent_kv_write(latent, rope_key, cache, slot_mapping):
    """Returns a copy of ``cache`` with row ``slot`` = latent ++ rope_key (mla.cu:29-32)."""
    out = cache.clone()
    flat = out.view(-1, out.shape[-1])
    flat[slot_mapping.to(torch.int64)] = torch.cat((latent, rope_key), dim=1)
    return out


def mla_latent_attention_f64(q_absorbed, q_rope, cache, block_table, lengths, positions, *, scale,
                             causal=True, indices=None):
    """Independent float64 formulation (streaming log-sum-exp, token by token through the page
    table, the order the CUDA kernels walk) returning float64 ``[B,T,H,Dc]`` unrounded."""
    qa = q_absorbed.cpu().to(torch.float64).numpy()
    qr = q_rope.cpu().to(torch.float64).numpy()
    cch = cache.cpu().to(torch.float64).numpy()
    table = block_table.cpu().numpy()
    lens = lengths.cpu().numpy()
    pos = positions.cpu().numpy()
    idx = None if indices is None else indices.cpu().numpy()
    batch, tq, heads, dc = qa.shape
    page = cch.shape[1]
    out = np.zeros((batch, tq, heads, dc))
    for b in range(batch):
        for t in range(tq):
            end = int(lens[b])
            if causal:
                end = min(end, max(0, int(pos[b, t]) + 1))
            toks = range(end) if idx is None else [int(s) for s in idx[b, t] if 0 <= int(s) < end]
            m = np.full(heads, -np.inf)
            l = np.zeros(heads)
            acc = np.zeros((heads, dc))
            for s in toks:
                row = cch[int(table[b, s // page]), s % page]
                sc = (qa[b, t] @ row[:dc] + qr[b, t] @ row[dc:]) * scale
                mn = np.maximum(m, sc)
                a = np.where(np.isinf(m), 0.0, np.exp(m - mn))
                p = np.exp(sc - mn)
                l = l * a + p
                acc = acc * a[:, None] + p[:, None] * row[None, :dc]
                m = mn
            ok = l > 0
            out[b, t][ok] = acc[ok] / l[ok][:, None]
    return out
