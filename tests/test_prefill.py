"""Dense GQA prefill: the oracle against the reference's outputs (CPU), and the CUDA
kernels (through the C ABI) against the oracle (GPU)."""

import pytest
import torch

from conftest import TOL, load_prefill, prefill_cases
from oracle import gqa_oracle

import attention_b200 as attn

DEV = "cuda"


def _close(got, want, dtype, what=""):
    tol = TOL[dtype]
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), atol=tol, rtol=tol,
                               msg=lambda m: f"{what}: {m}")


# --------------------------------------------------------------------------- CPU: oracle pin
@pytest.mark.parametrize("name", prefill_cases())
def test_prefill_oracle_matches_reference(name):
    q, k, v, ql, kl, causal, scale, want = load_prefill(name)
    got = gqa_oracle.reference_gqa_prefill(q, k, v, ql, kl, causal=causal, scale=scale)
    assert got.shape == q.shape and got.dtype == q.dtype
    _close(got, want, q.dtype, name)


def test_prefill_oracle_padding_rows_are_zero():
    q, k, v, ql, kl, causal, scale, _ = load_prefill("prefill_bf16_qlonger_d128")
    out = gqa_oracle.reference_gqa_prefill(q, k, v, ql, kl, causal=causal, scale=scale)
    # sequence 0: 70 queries over 50 keys, right aligned: the first 20 rows see nothing
    assert torch.count_nonzero(out[0, :20]) == 0 and torch.count_nonzero(out[0, 20]) > 0
    assert torch.count_nonzero(out[1, int(ql[1]):]) == 0


def test_prefill_front_door_rejects_cpu_tensors():
    q, k, v, ql, kl, causal, scale, _ = load_prefill("prefill_f32_causal_d32")
    with pytest.raises(RuntimeError, match="CUDA"):
        attn.gqa_prefill(q, k, v, ql, kl)
    with pytest.raises(ValueError):
        attn.gqa_prefill(q, k, v, ql, kl, backend="triton")


# --------------------------------------------------------------------------- GPU parity
def _case(b, tq, tk, hq, hkv, d, dtype, q_lens, kv_lens, seed=0):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(b, tq, hq, d, generator=gen).to(dtype)
    k = torch.randn(b, tk, hkv, d, generator=gen).to(dtype)
    v = torch.randn(b, tk, hkv, d, generator=gen).to(dtype)
    return (q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(q_lens, dtype=torch.int32, device=DEV),
            torch.tensor(kv_lens, dtype=torch.int32, device=DEV))


def _tc_ok(dtype, d):
    """Shapes the tensor-core kernels (mma.sync and tcgen05) take."""
    return dtype in (torch.float16, torch.bfloat16) and d in (64, 128)


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["auto", "simt", "mma", "tcgen05"])
@pytest.mark.parametrize("name", prefill_cases())
def test_prefill_golden(name, kernel):
    q, k, v, ql, kl, causal, scale, want = load_prefill(name)
    if kernel in ("mma", "tcgen05") and not _tc_ok(q.dtype, q.shape[-1]):
        pytest.skip("shape not covered by the tensor-core kernels")
    got = attn.gqa_prefill(q.to(DEV), k.to(DEV), v.to(DEV), ql.to(DEV), kl.to(DEV), causal=causal,
                           scale=scale, kernel=kernel)
    _close(got, want, q.dtype, f"{name} {kernel}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_ragged_batches(dtype, causal):
    """Lengths around the 64-row / 64-key tile edges, q shorter, equal and longer than kv,
    empty sequences, chunked prefill (few queries over a long prefix)."""
    q_lens = [0, 1, 63, 64, 65, 130, 200, 16, 7, 200]
    kv_lens = [5, 1, 63, 64, 65, 300, 150, 300, 0, 200]
    args = _case(10, 200, 300, 8, 2, 128, dtype, q_lens, kv_lens, seed=3)
    want = gqa_oracle.reference_gqa_prefill(*args, causal=causal)
    kernels = ("auto", "simt", "mma", "tcgen05") if _tc_ok(dtype, 128) else ("auto", "simt")
    for kernel in kernels:
        got = attn.gqa_prefill(*args, causal=causal, kernel=kernel)
        _close(got, want, dtype, f"{dtype} causal={causal} {kernel}")
        assert torch.count_nonzero(got[0]) == 0 and torch.count_nonzero(got[8]) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("hq,hkv,d", [(4, 4, 128), (8, 1, 128), (28, 4, 128), (6, 2, 64), (5, 1, 64),
                                       (8, 2, 256), (4, 2, 96), (3, 3, 40)])
def test_prefill_head_layouts_and_sizes(hq, hkv, d):
    args = _case(2, 150, 150, hq, hkv, d, torch.bfloat16, [150, 77], [150, 77], seed=hq + d)
    want = gqa_oracle.reference_gqa_prefill(*args)
    _close(attn.gqa_prefill(*args), want, torch.bfloat16, f"{hq}/{hkv} D={d}")
    _close(attn.gqa_prefill(*args, backend="tensorcore"), want, torch.bfloat16)
    if _tc_ok(torch.bfloat16, d):
        for kernel in ("mma", "tcgen05"):
            _close(attn.gqa_prefill(*args, kernel=kernel), want, torch.bfloat16, f"{kernel} D={d}")
    else:
        with pytest.raises(RuntimeError, match="kernel"):
            attn.gqa_prefill(*args, kernel="tcgen05")


@pytest.mark.gpu
def test_prefill_long_sequence_and_scale():
    args = _case(1, 2048, 2048, 8, 2, 128, torch.bfloat16, [2048], [2048], seed=9)
    want = gqa_oracle.reference_gqa_prefill(*args, scale=0.05)
    for kernel in ("mma", "tcgen05"):
        _close(attn.gqa_prefill(*args, scale=0.05, kernel=kernel), want, torch.bfloat16,
               f"2k causal {kernel}")
    args = _case(2, 33, 4096, 8, 2, 128, torch.float16, [33, 20], [4096, 3000], seed=10)
    want = gqa_oracle.reference_gqa_prefill(*args)
    for kernel in ("mma", "tcgen05"):
        _close(attn.gqa_prefill(*args, kernel=kernel), want, torch.float16,
               f"chunked over 4k prefix {kernel}")


@pytest.mark.gpu
def test_prefill_tcgen05_status_word_stays_clear():
    """The tcgen05 kernel's bounded waits never ran out in the calls above (or here)."""
    from attention_b200 import _cabi
    args = _case(2, 260, 260, 8, 2, 128, torch.bfloat16, [260, 100], [260, 100], seed=12)
    attn.gqa_prefill(*args, kernel="tcgen05")
    assert _cabi.load().gqa_b200_prefill_tc_status(0) == 0


@pytest.mark.gpu
def test_prefill_argument_checks():
    q, k, v, ql, kl = _case(2, 8, 8, 4, 2, 64, torch.float16, [8, 3], [8, 3])
    bad = [
        (dict(q=q[0]), r"\[B,T,H,D\]"),
        (dict(v=v[:, :4].contiguous()), r"\[B,T,H,D\]"),
        (dict(k=k[:1], v=v[:1]), "batch or head_dim"),
        (dict(q=q[:, :, :3].contiguous()), "head mapping"),
        (dict(ql=ql[:1]), r"lengths must be \[B\]"),
        (dict(ql=ql.long()), "int32"),
        (dict(q=q.float()), "dtype mismatch"),
        (dict(q=q.double(), k=k.double(), v=v.double()), "unsupported dtype"),
        (dict(scale=0.0), "scale"),
        (dict(q=q.transpose(1, 2)), "contiguous"),
    ]
    for change, pattern in bad:
        a = dict(q=q, k=k, v=v, ql=ql, kl=kl, scale=None)
        a.update(change)
        with pytest.raises(RuntimeError, match=pattern):
            attn.gqa_prefill(a["q"], a["k"], a["v"], a["ql"], a["kl"], scale=a["scale"])
    with pytest.raises(ValueError, match="tensorcore"):
        attn.gqa_prefill(q.float(), k.float(), v.float(), ql, kl, backend="tensorcore")
    empty = attn.gqa_prefill(q[:0], k[:0], v[:0], ql[:0], kl[:0])
    assert empty.shape == (0, 8, 4, 64)


@pytest.mark.gpu
def test_prefill_degenerate_shapes():
    """No keys at all, a single query row, and query tiles that end inside a 128-row tile."""
    q, k, v, ql, kl = _case(2, 5, 7, 4, 2, 128, torch.bfloat16, [5, 2], [7, 0])
    empty_kv = torch.empty(2, 0, 2, 128, dtype=torch.bfloat16, device=DEV)
    out = attn.gqa_prefill(q, empty_kv, empty_kv, ql, torch.zeros_like(kl))
    assert out.shape == q.shape and torch.count_nonzero(out) == 0
    for kernel in ("auto", "mma", "tcgen05", "simt"):
        got = attn.gqa_prefill(q, k, v, ql, kl, kernel=kernel)
        _close(got, gqa_oracle.reference_gqa_prefill(q, k, v, ql, kl), torch.bfloat16, kernel)
        assert torch.count_nonzero(got[1]) == 0          # sequence 1 has no keys
    args = _case(3, 129, 257, 8, 4, 64, torch.float16, [129, 1, 128], [257, 200, 128], seed=4)
    want = gqa_oracle.reference_gqa_prefill(*args)
    for kernel in ("mma", "tcgen05"):
        _close(attn.gqa_prefill(*args, kernel=kernel), want, torch.float16, kernel)


@pytest.mark.gpu
def test_prefill_kernels_agree_on_a_large_ragged_batch():
    """tcgen05, mma.sync and the oracle on 16 ragged sequences up to 3000 tokens."""
    gen = torch.Generator().manual_seed(77)
    q_lens = torch.randint(1, 3001, (16,), generator=gen).tolist()
    kv_lens = [n + int(torch.randint(0, 500, (1,), generator=gen)) for n in q_lens]
    args = _case(16, 3000, 3500, 16, 4, 128, torch.bfloat16, q_lens, kv_lens, seed=78)
    want = gqa_oracle.reference_gqa_prefill(*args)
    for kernel in ("tcgen05", "mma"):
        _close(attn.gqa_prefill(*args, kernel=kernel), want, torch.bfloat16, kernel)


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_two_tile_item_edges(causal):
    """The tcgen05 kernel works on items of two 128-row query tiles: query lengths around 128,
    256 and 384 rows (second tile empty, one row, full), keys shorter than queries (the first
    rows of a causal sequence see nothing), keys around the 64-key half tiles, and enough
    (sequence, head) pairs that a CTA walks several items in both directions of the hand-out."""
    q_lens = [255, 256, 257, 128, 129, 384, 385, 512, 1, 300, 200, 400]
    kv_lens = [255, 300, 257, 64, 65, 127, 500, 129, 193, 100, 200, 40]
    args = _case(12, 512, 500, 16, 4, 128, torch.bfloat16, q_lens, kv_lens, seed=21)
    want = gqa_oracle.reference_gqa_prefill(*args, causal=causal)
    for kernel in ("tcgen05", "mma"):
        got = attn.gqa_prefill(*args, causal=causal, kernel=kernel)
        _close(got, want, torch.bfloat16, f"causal={causal} {kernel}")
        for b, n in enumerate(q_lens):
            assert torch.count_nonzero(got[b, n:]) == 0, f"rows past q_len of sequence {b} ({kernel})"
    from attention_b200 import _cabi
    assert _cabi.load().gqa_b200_prefill_tc_status(0) == 0


@pytest.mark.gpu
def test_prefill_random_shapes_tcgen05_against_mma_and_itself():
    """Forty random shapes (head layouts, D 64 / 128, both dtypes, ragged lengths down to zero,
    causal or not): the tcgen05 kernel agrees with the mma.sync kernel, gives the same bits when
    called twice, and its bounded waits never run out."""
    import random
    from attention_b200 import _cabi
    rng = random.Random(5)
    for it in range(40):
        b = rng.randint(1, 5)
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 4, 8])
        hq = hkv * rng.choice([1, 2, 4, 7, 8])
        tq, tk = rng.randint(1, 700), rng.randint(1, 1100)
        dtype = rng.choice([torch.bfloat16, torch.float16])
        causal = rng.random() < 0.7
        q_lens = [rng.randint(0, tq) for _ in range(b)]
        kv_lens = [rng.randint(0, tk) for _ in range(b)]
        args = _case(b, tq, tk, hq, hkv, d, dtype, q_lens, kv_lens, seed=100 + it)
        got = attn.gqa_prefill(*args, causal=causal, kernel="tcgen05")
        again = attn.gqa_prefill(*args, causal=causal, kernel="tcgen05")
        want = attn.gqa_prefill(*args, causal=causal, kernel="mma")
        what = f"case {it}: B{b} tq{tq} tk{tk} {hq}/{hkv} D{d} {dtype} causal={causal}"
        _close(got, want, dtype, what)
        assert torch.equal(got, again), what
    assert _cabi.load().gqa_b200_prefill_tc_status(0) == 0
