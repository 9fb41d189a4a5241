"""The five benchmark configurations at full size on the GPU: parity against the
torch oracle run on the same device tensors, plus size-independent properties
(page relabelling, sharding) that must hold bit for bit."""

import pytest
import torch

from conftest import TOL
from oracle import gqa_oracle

import attention_b200 as attn
from attention_b200 import sharding, synth

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", params=list(synth.WORKLOADS))
def workload(request):
    w = synth.WORKLOADS[request.param]
    inputs = synth.make_workload(w, seed=42, device=DEV, kv_on_device=True)
    yield w, inputs
    del inputs
    torch.cuda.empty_cache()


def test_full_size_parity(workload):
    w, (q, k, v, table, lens) = workload
    torch.backends.cuda.matmul.allow_tf32 = False
    want = gqa_oracle.reference_gqa_decode(q, k, v, table, lens)
    got = attn.gqa_decode(q, k, v, table, lens)
    tol = TOL[w.dtype]
    torch.testing.assert_close(got.float(), want.float(), atol=tol, rtol=tol)
    assert torch.isfinite(got.float()).all()


def test_full_size_split_front_door(workload):
    w, (q, k, v, table, lens) = workload
    want = attn.gqa_decode(q, k, v, table, lens)
    got = attn.gqa_decode_split(q, k, v, table, lens, splits=4)
    tol = TOL[w.dtype]
    torch.testing.assert_close(got.float(), want.float(), atol=tol, rtol=tol)


def test_page_relabelling_is_bit_exact(workload):
    """Moving every page to a new physical slot (and rewriting the table) changes nothing."""
    w, (q, k, v, table, lens) = workload
    base = attn.gqa_decode(q, k, v, table, lens).clone()
    n = k.shape[0]
    gen = torch.Generator(device=DEV).manual_seed(1)
    perm = torch.randperm(n, device=DEV, generator=gen)          # new slot -> old page
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(n, device=DEV)                       # old page -> new slot
    k2, v2 = k[perm].contiguous(), v[perm].contiguous()
    t2 = torch.where(table >= 0, inv[table.clamp(min=0).long()].to(torch.int32), table)
    again = attn.gqa_decode(q, k2, v2, t2, lens)
    assert torch.equal(base, again)


@pytest.mark.parametrize("world", [2, 8])
def test_sharded_equals_unsharded_bit_for_bit(workload, world):
    """Each rank's local pool + table gives exactly the rows of the single-GPU run.

    With one base chunk length a sequence is cut the same way wherever it lands, so the
    rows agree bit for bit.  (chunk_tokens=0 derives the base from the local batch shape, so
    there the rows agree only to rounding -- checked at the end.)"""
    w, (q, k, v, table, lens) = workload
    whole = attn.gqa_decode(q, k, v, table, lens, chunk_tokens=512)
    auto_parts = []
    shards = sharding.lpt_assign(lens.tolist(), world)
    parts = []
    for ids in shards:
        if not ids:
            parts.append(torch.empty((0,) + tuple(q.shape[1:]), dtype=q.dtype, device=DEV))
            continue
        local = sharding.extract_shard(q, k, v, table, lens, ids, device=DEV)
        parts.append(attn.gqa_decode(*local, chunk_tokens=512))
        auto_parts.append(attn.gqa_decode(*local))
    again = sharding.scatter_outputs(parts, shards, q.shape[0])
    assert torch.equal(whole, again)
    if all(len(s) for s in shards):
        auto = sharding.scatter_outputs(auto_parts, shards, q.shape[0])
        tol = TOL[w.dtype]
        torch.testing.assert_close(auto.float(), whole.float(), atol=tol, rtol=tol)
