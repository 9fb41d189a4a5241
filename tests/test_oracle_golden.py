"""The oracle restatements against outputs of the reference itself (CPU only)."""

import numpy as np
import pytest
import torch

from conftest import TOL, full_cases, load_full, load_seeded, seed_cases
from oracle import gqa_oracle


def _close(got, want, dtype):
    tol = TOL[dtype]
    torch.testing.assert_close(got.float(), want.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("name", full_cases())
def test_torch_restatement_matches_reference_full(name):
    q, k, v, table, lens, scale, want = load_full(name)
    got = gqa_oracle.reference_gqa_decode(q, k, v, table, lens, scale=scale)
    assert got.dtype == q.dtype and got.shape == q.shape
    _close(got, want, q.dtype)


@pytest.mark.parametrize("name", full_cases())
def test_c_restatement_matches_reference_full(name):
    q, k, v, table, lens, scale, want = load_full(name)
    got = gqa_oracle.gqa_decode_c(q, k, v, table, lens, scale=scale)
    _close(got, want, q.dtype)


@pytest.mark.parametrize("name", full_cases())
def test_f64_restatement_matches_reference_full(name):
    q, k, v, table, lens, scale, want = load_full(name)
    got = gqa_oracle.gqa_decode_f64(q, k, v, table, lens, scale=scale)
    _close(torch.from_numpy(got).to(q.dtype), want, q.dtype)


@pytest.mark.parametrize("name", seed_cases())
def test_restatements_match_reference_seeded(name):
    (q, k, v, table, lens), want = load_seeded(name)
    _close(gqa_oracle.reference_gqa_decode(q, k, v, table, lens), want, q.dtype)
    _close(gqa_oracle.gqa_decode_c(q, k, v, table, lens), want, q.dtype)


def test_zero_length_rows_are_zero():
    q, k, v, table, lens, scale, want = load_full("full_f32_g3_d32_bs4")
    assert int(lens[0]) == 0
    for fn in (gqa_oracle.reference_gqa_decode, gqa_oracle.gqa_decode_c):
        assert torch.count_nonzero(fn(q, k, v, table, lens)[0]) == 0


def test_c_oracle_thread_count_does_not_change_result():
    q, k, v, table, lens, scale, _ = load_full("full_bf16_g4_d128_bs16")
    a = gqa_oracle.gqa_decode_c(q, k, v, table, lens, threads=1)
    b = gqa_oracle.gqa_decode_c(q, k, v, table, lens, threads=4)
    assert torch.equal(a, b)


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 40])
def test_split_merge_algebra_equals_unsplit(splits):
    """Reference split ranges + left-to-right merge reproduce the unsplit result,
    including splits > tokens (empty partials are skipped)."""
    q, k, v, table, lens, scale, _ = load_full("full_f32_g3_d32_bs4")
    mx, sm, acc = gqa_oracle.split_partials_f64(q, k, v, table, lens, splits, scale=scale)
    merged = gqa_oracle.merge_partials_f64(mx, sm, acc)
    whole = gqa_oracle.gqa_decode_f64(q, k, v, table, lens, scale=scale)
    np.testing.assert_allclose(merged, whole, rtol=1e-12, atol=1e-12)


def test_kv_append_restatement_roundtrip():
    q, k, v, table, lens, scale, _ = load_full("full_f32_g3_d32_bs4")
    k2, v2 = k.clone(), v.clone()
    pos = torch.tensor([0, 0, 2, 3, 4, 8], dtype=torch.int32)
    key = torch.randn(q.shape[0], k.shape[2], k.shape[3])
    val = torch.randn_like(key)
    table = table.clone()
    # sequence 0 has no page yet: give it a fresh distinct one
    used = set(table[table >= 0].tolist())
    table[0, 0] = next(i for i in range(k.shape[0]) if i not in used)
    gqa_oracle.reference_kv_append(key, val, k2, v2, table, pos)
    bs = k.shape[1]
    for b, t in enumerate(pos.tolist()):
        phys = int(table[b, t // bs])
        assert torch.equal(k2[phys, t % bs], key[b]) and torch.equal(v2[phys, t % bs], val[b])
    changed = (k2 != k).any(dim=(2, 3)).sum()
    assert changed <= q.shape[0]


# ---------------------------------------------------------------------------
# paged latent (MLA) decode restatements against the reference's mla_reference
# ---------------------------------------------------------------------------
from conftest import load_mla, mla_cases  # noqa: E402
from oracle import mla_oracle  # noqa: E402


@pytest.mark.parametrize("name", mla_cases())
def test_mla_restatement_matches_reference(name):
    c, causal, want = load_mla(name)
    got = mla_oracle.reference_mla_decode(c["q_nope"], c["q_rope"], c["cache"], c["block_table"],
                                          c["lengths"], c["positions"], c["w_uk"], c["w_uv"],
                                          causal=causal, indices=c["indices"])
    assert got.dtype == want.dtype and got.shape == want.shape
    _close(got, want, want.dtype)


@pytest.mark.parametrize("name", mla_cases())
def test_mla_f64_stream_matches_dense_restatement(name):
    c, causal, _ = load_mla(name)
    scale = 1.0 / (c["q_nope"].shape[-1] + c["q_rope"].shape[-1]) ** 0.5
    qa = mla_oracle.reference_mla_project(c["q_nope"], c["w_uk"], True)
    dense = mla_oracle.reference_mla_latent_attention(qa, c["q_rope"], c["cache"], c["block_table"],
                                                      c["lengths"], c["positions"], scale=scale,
                                                      causal=causal, indices=c["indices"])
    stream = mla_oracle.mla_latent_attention_f64(qa, c["q_rope"], c["cache"], c["block_table"], c["lengths"],
                                                 c["positions"], scale=scale, causal=causal,
                                                 indices=c["indices"])
    _close(torch.from_numpy(stream).to(dense.dtype), dense, dense.dtype)


def test_mla_rows_without_visible_tokens_are_zero():
    c, causal, want = load_mla("mla_f16_multiquery")
    assert int(c["lengths"][2]) == 0 and int(c["positions"][1, 1]) == -1
    assert torch.count_nonzero(want[2]) == 0 and torch.count_nonzero(want[1, 1]) == 0
    got = mla_oracle.reference_mla_decode(c["q_nope"], c["q_rope"], c["cache"], c["block_table"],
                                          c["lengths"], c["positions"], c["w_uk"], c["w_uv"])
    assert torch.count_nonzero(got[2]) == 0 and torch.count_nonzero(got[1, 1]) == 0


def test_latent_kv_write_restatement():
    c, _, _ = load_mla("mla_f32_small")
    cache = c["cache"]
    dc = c["w_uk"].shape[-1]
    slots = torch.tensor([5, 0, 17], dtype=torch.int64)
    lat = torch.randn(3, dc)
    rope = torch.randn(3, cache.shape[-1] - dc)
    out = mla_oracle.reference_latent_kv_write(lat, rope, cache, slots)
    flat = out.view(-1, cache.shape[-1])
    assert torch.equal(flat[slots, :dc], lat) and torch.equal(flat[slots, dc:], rope)
    keep = torch.ones(flat.shape[0], dtype=torch.bool)
    keep[slots] = False
    assert torch.equal(flat[keep], cache.view(-1, cache.shape[-1])[keep])
