"""Paged latent-attention (MLA) decode: the CUDA path through the C ABI against the oracle and
against fixtures produced by the reference's own ``mla_reference``."""

import math

import pytest
import torch

import attention_b200 as attn
from attention_b200 import synth
from conftest import TOL, load_mla, mla_cases
from oracle import mla_oracle

gpu = pytest.mark.gpu
DEV = "cuda:0"


def _dev(c):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in c.items()}


def _close(got, want, dtype, scale=1.0):
    tol = TOL[dtype] * scale
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), atol=tol, rtol=tol)


def _decode(c, **kw):
    return attn.mla_decode(c["q_nope"], c["q_rope"], c["cache"], c["block_table"], c["lengths"],
                           c["positions"], c["w_uk"], c["w_uv"], indices=c.get("indices"), **kw)


# --------------------------------------------------------------------------- CPU
def test_mla_front_doors_reject_cpu_tensors():
    c = synth.make_mla_case("m1_small_fp32")
    with pytest.raises(RuntimeError, match="CUDA"):
        _decode(c)
    with pytest.raises(RuntimeError, match="CUDA"):
        attn.mla_query_absorb(c["q_nope"], c["w_uk"])
    with pytest.raises(RuntimeError, match="CUDA"):
        attn.latent_kv_write(torch.zeros(1, 32), torch.zeros(1, 8), c["cache"], torch.zeros(1, dtype=torch.int64))


def test_mla_workspace_sizes_and_status_codes():
    from attention_b200 import _cabi
    lib = _cabi.load()
    assert lib.mla_b200_attend_workspace_bytes(64, 1, 128, 512, 64, 64, 64, 0) >= 256
    assert lib.mla_b200_attend_workspace_bytes(64, 1, 128, 513, 64, 64, 64, 0) == 0     # dc > 512
    assert lib.mla_b200_attend_workspace_bytes(1, 1, 0, 512, 64, 64, 64, 0) == 0        # no heads
    small = lib.mla_b200_attend_workspace_bytes(1, 1, 4, 32, 8, 16, 256, 0)
    assert small >= 4 * 2 * (32 + 2) * 4          # one row of 4 heads is split at this capacity
    assert lib.mla_b200_decode_workspace_bytes(2, 1, 4, 32, 8, 16, 4, 0) > 2 * 2 * 4 * 32 * 4
    # invalid arguments are refused before any launch (no GPU needed)
    assert lib.mla_b200_attend(None, None, None, None, None, None, None, None, 7, 1, 1, 1, 32, 8, 1, 16, 1, 0,
                               1.0, 1, None, 0, None) == -2
    assert lib.mla_b200_attend(None, None, None, None, None, None, None, None, 0, 1, 1, 1, 600, 8, 1, 16, 1, 0,
                               1.0, 1, None, 0, None) == -33
    assert lib.mla_b200_attend(None, None, None, None, None, None, None, None, 0, 1, 1, 1, 32, 8, 1, 16, 1, 0,
                               1.0, 1, None, 0, None) == -1
    assert lib.mla_b200_attend(None, None, None, None, None, None, None, None, 0, 1, 1, 1, 32, 8, 1, 16, 1, 0,
                               float("nan"), 1, None, 0, None) == -7
    assert lib.mla_b200_project(None, None, None, 0, 4, 0, 8, 8, 1, None) == -32
    assert "MLA" in _cabi.strerror(-32) and "512" in _cabi.strerror(-33)


# --------------------------------------------------------------------------- GPU
@gpu
@pytest.mark.parametrize("name", mla_cases())
def test_mla_decode_matches_reference_fixture(name):
    c, causal, want = load_mla(name)
    got = _decode(_dev(c), causal=causal)
    assert got.dtype == want.dtype and got.shape == want.shape
    # two extra roundings (absorbed query, latent output) relative to the fp32 oracle
    _close(got, want, want.dtype, scale=2.0)


@gpu
@pytest.mark.parametrize("name", mla_cases())
def test_mla_stages_match_oracle(name):
    c, causal, _ = load_mla(name)
    d = _dev(c)
    scale = 1.0 / math.sqrt(c["q_nope"].shape[-1] + c["q_rope"].shape[-1])
    qa = attn.mla_query_absorb(d["q_nope"], d["w_uk"])
    _close(qa, mla_oracle.reference_mla_project(c["q_nope"], c["w_uk"], True), qa.dtype)
    u = attn.mla_latent_attention(qa, d["q_rope"], d["cache"], d["block_table"], d["lengths"],
                                  d["positions"], scale=scale, causal=causal, indices=d["indices"])
    want_u = mla_oracle.reference_mla_latent_attention(qa.cpu(), c["q_rope"], c["cache"], c["block_table"],
                                                       c["lengths"], c["positions"], scale=scale,
                                                       causal=causal, indices=c["indices"])
    _close(u, want_u, u.dtype)
    out = attn.mla_value_project(u, d["w_uv"])
    _close(out, mla_oracle.reference_mla_project(u.cpu(), c["w_uv"], False), out.dtype)
    # the one-call path equals the three operators bit for bit
    assert torch.equal(out, _decode(d, causal=causal))


@gpu
@pytest.mark.parametrize("splits", [1, 2, 5, 32])
def test_mla_split_counts_agree(splits):
    c, causal, _ = load_mla("mla_bf16_wide")
    d = _dev(c)
    scale = 0.07
    qa = attn.mla_query_absorb(d["q_nope"], d["w_uk"])
    args = (qa, d["q_rope"], d["cache"], d["block_table"], d["lengths"], d["positions"])
    want = mla_oracle.reference_mla_latent_attention(qa.cpu(), c["q_rope"], c["cache"], c["block_table"],
                                                     c["lengths"], c["positions"], scale=scale)
    got = attn.mla_latent_attention(*args, scale=scale, kernel="simt", splits=splits)
    _close(got, want, got.dtype)


@gpu
def test_mla_sparse_more_splits_than_indices():
    c, causal, _ = load_mla("mla_f32_sparse")
    d = _dev(c)
    scale = 0.2
    qa = attn.mla_query_absorb(d["q_nope"], d["w_uk"])
    got = attn.mla_latent_attention(qa, d["q_rope"], d["cache"], d["block_table"], d["lengths"],
                                    d["positions"], scale=scale, indices=d["indices"], splits=20)
    want = mla_oracle.mla_latent_attention_f64(qa.cpu(), c["q_rope"], c["cache"], c["block_table"],
                                               c["lengths"], c["positions"], scale=scale, indices=c["indices"])
    _close(got, torch.from_numpy(want).float(), torch.float32)


@gpu
def test_latent_kv_write_then_decode_sees_the_new_token():
    w = synth.MLA_WORKLOADS["m1_small_fp32"]
    c = _dev(synth.make_mla_case(w, lengths=[30, 17]))
    cache0 = c["cache"].clone()
    lens = c["lengths"]
    # append one token per sequence at position len (its page is already in the table here)
    page = w.page
    slots = torch.stack([c["block_table"][b, int(lens[b]) // page].long() * page + int(lens[b]) % page
                         for b in range(2)])
    lat = torch.randn(2, w.dc, device=DEV)
    rope = torch.randn(2, w.dr, device=DEV)
    attn.latent_kv_write(lat, rope, c["cache"], slots)
    want_cache = mla_oracle.reference_latent_kv_write(lat.cpu(), rope.cpu(), cache0.cpu(), slots.cpu())
    assert torch.equal(c["cache"].cpu(), want_cache)
    c["lengths"] = lens + 1
    c["positions"] = c["positions"] + 1
    got = _decode(c)
    cc = {k: v.cpu() for k, v in c.items()}
    want = mla_oracle.reference_mla_decode(cc["q_nope"], cc["q_rope"], cc["cache"], cc["block_table"],
                                           cc["lengths"], cc["positions"], cc["w_uk"], cc["w_uv"])
    _close(got, want, torch.float32, scale=2.0)


@gpu
def test_mla_empty_batch_and_zero_rows():
    w = synth.MLA_WORKLOADS["m1_small_fp32"]
    c = _dev(synth.make_mla_case(w, lengths=[0, 5]))
    out = _decode(c)
    assert torch.count_nonzero(out[0]) == 0 and torch.count_nonzero(out[1]) > 0
    e = {k: (v[:0].contiguous() if k in ("q_nope", "q_rope", "block_table", "lengths", "positions") else v)
         for k, v in c.items()}
    assert _decode(e).shape == (0, 1, w.heads, w.dv)


@gpu
def test_mla_invalid_arguments_raise():
    c = _dev(synth.make_mla_case("m1_small_fp32"))
    with pytest.raises(RuntimeError, match="scale"):
        _decode(c, scale=-1.0)
    bad = dict(c)
    bad["lengths"] = c["lengths"].long()
    with pytest.raises(RuntimeError, match="int32"):
        _decode(bad)
    bad = dict(c)
    bad["w_uk"] = c["w_uk"].half()
    with pytest.raises(RuntimeError, match="dtype"):
        _decode(bad)
    bad = dict(c)
    bad["cache"] = c["cache"][..., :-1].contiguous()
    with pytest.raises(RuntimeError, match="dimensions"):
        _decode(bad)


@gpu
def test_mla_deepseek_shape_small_batch():
    """128 heads, 512 + 64 wide rows, ragged lengths: the shape the tensor-core kernel is built for."""
    w = synth.scaled_mla("m2_deepseek_h128_bf16", batch=3)
    c = synth.make_mla_case(w, lengths=[700, 64, 1], seed=3)
    got = _decode(_dev(c))
    want = mla_oracle.reference_mla_decode(c["q_nope"], c["q_rope"], c["cache"], c["block_table"],
                                           c["lengths"], c["positions"], c["w_uk"], c["w_uv"],
                                           round_intermediates=True)
    _close(got, want, torch.bfloat16)


# ------------------------------------------------------------- tensor-core kernel (CTA pair)
def _tc_case(heads, tq, page, lengths, dtype=torch.bfloat16, seed=5):
    w = synth.MlaWorkload("t", len(lengths), tq, heads, 32, 64, 512, 32, page, dtype, 0, 0)
    return w, synth.make_mla_case(w, lengths=lengths, seed=seed)


def _latent(c, d, kernel, splits=0, causal=True):
    scale = 0.06
    qa = attn.mla_query_absorb(d["q_nope"], d["w_uk"])
    got = attn.mla_latent_attention(qa, d["q_rope"], d["cache"], d["block_table"], d["lengths"],
                                    d["positions"], scale=scale, causal=causal, kernel=kernel, splits=splits)
    want = mla_oracle.reference_mla_latent_attention(qa.cpu(), c["q_rope"], c["cache"], c["block_table"],
                                                     c["lengths"], c["positions"], scale=scale, causal=causal)
    return got, want


@gpu
@pytest.mark.parametrize("heads,tq,page,lengths,dtype", [
    (128, 1, 64, [700, 64, 1, 0, 33], torch.bfloat16),
    (16, 1, 64, [300, 31, 32, 257], torch.bfloat16),
    (128, 2, 16, [130, 5], torch.float16),            # two row tiles per sequence
    (24, 3, 48, [100, 49, 200], torch.bfloat16),      # rows of several query tokens share a tile; odd page size
    (5, 1, 8, [1000], torch.float16),
])
def test_mla_tensor_core_kernel_matches_oracle(heads, tq, page, lengths, dtype):
    from attention_b200.mla import mla_tc_status
    mla_tc_status(reset=True)
    w, c = _tc_case(heads, tq, page, lengths, dtype)
    d = _dev(c)
    for splits in (0, 1, 3):
        got, want = _latent(c, d, "tcgen05", splits=splits)
        _close(got, want, dtype)
    simt, _ = _latent(c, d, "simt")
    _close(got, simt, dtype)
    assert mla_tc_status() == 0


@gpu
def test_mla_tensor_core_kernel_non_causal_and_early_positions():
    from attention_b200.mla import mla_tc_status
    w, c = _tc_case(32, 2, 32, [90, 40])
    c["positions"] = torch.tensor([[10, 80], [-1, 39]], dtype=torch.int32)
    d = _dev(c)
    got, want = _latent(c, d, "tcgen05")
    _close(got, want, torch.bfloat16)
    assert torch.count_nonzero(got[1, 0]) == 0
    got, want = _latent(c, d, "tcgen05", causal=False)
    _close(got, want, torch.bfloat16)
    assert mla_tc_status() == 0


@gpu
def test_mla_tensor_core_kernel_refuses_other_shapes():
    w = synth.MLA_WORKLOADS["m1_small_fp32"]
    d = _dev(synth.make_mla_case(w))
    qa = attn.mla_query_absorb(d["q_nope"], d["w_uk"])
    with pytest.raises(RuntimeError, match="kernel"):
        attn.mla_latent_attention(qa, d["q_rope"], d["cache"], d["block_table"], d["lengths"], d["positions"],
                                  scale=0.1, kernel="tcgen05")


@gpu
def test_mla_tensor_core_kernel_many_ragged_sequences():
    """More sequences than SM pairs, ragged lengths: ranges of the tile schedule start and end
    inside sequences, several work items per CTA pair, whole-unit and partial items mixed."""
    from attention_b200.mla import mla_tc_status
    gen = torch.Generator().manual_seed(11)
    lengths = torch.randint(1, 1400, (90,), generator=gen).tolist()
    lengths[3] = 0
    lengths[17] = 4000                                  # one long sequence spanning several ranges
    w, c = _tc_case(16, 1, 64, lengths, torch.bfloat16, seed=12)
    d = _dev(c)
    got, want = _latent(c, d, "tcgen05")
    _close(got, want, torch.bfloat16)
    assert torch.count_nonzero(got[3]) == 0
    again, _ = _latent(c, d, "tcgen05")
    assert torch.equal(got, again)                      # same schedule, same order of sums: repeatable
    assert mla_tc_status() == 0


@gpu
@pytest.mark.parametrize("rows,heads,d_in,d_out,dtype", [
    (3, 5, 128, 512, torch.bfloat16),      # W_uk-like, one partial row tile
    (70, 2, 64, 64, torch.float16),        # two row tiles, the second ragged
    (64, 3, 512, 128, torch.bfloat16),     # W_uv-like
    (130, 1, 192, 192, torch.float16),
])
def test_mla_projections_tensor_core_path(rows, heads, d_in, d_out, dtype):
    """Widths that are multiples of 64 take the mma.sync projection kernel; both directions."""
    gen = torch.Generator().manual_seed(rows + d_in)
    x = (torch.randn(rows, 1, heads, d_in, generator=gen)).to(dtype)
    w_absorb = (torch.randn(heads, d_in, d_out, generator=gen) / math.sqrt(d_in)).to(dtype)
    w_value = (torch.randn(heads, d_out, d_in, generator=gen) / math.sqrt(d_in)).to(dtype)
    got = attn.mla_query_absorb(x.to(DEV), w_absorb.to(DEV))
    _close(got, mla_oracle.reference_mla_project(x, w_absorb, True), dtype)
    got = attn.mla_value_project(x.to(DEV), w_value.to(DEV))
    _close(got, mla_oracle.reference_mla_project(x, w_value, False), dtype)
