"""GPU parity of the CUDA path (through the C ABI) against the CPU/torch oracle."""

import math

import pytest
import torch

from conftest import TOL, full_cases, load_full, load_seeded, seed_cases
from oracle import gqa_oracle

import attention_b200 as attn
from attention_b200 import _cabi, synth

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _cuda(*ts):
    return tuple(t.to(DEV) for t in ts)


def _assert_close(got, want, dtype, what=""):
    tol = TOL[dtype]
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), atol=tol, rtol=tol, msg=lambda m: f"{what}: {m}")


def _make_case(lengths, hq, hkv, d, bs, dtype, seed=0, pool_extra=3):
    """Inputs in the reference fixture's layout: permuted pages, -1 in unused slots."""
    gen = torch.Generator().manual_seed(seed)
    lens = torch.tensor(lengths, dtype=torch.int32)
    pages = [(n + bs - 1) // bs for n in lengths]
    pool = max(1, sum(pages) + pool_extra)
    q = torch.randn(len(lengths), hq, d, generator=gen).to(dtype)
    k = torch.randn(pool, bs, hkv, d, generator=gen).to(dtype)
    v = torch.randn(pool, bs, hkv, d, generator=gen).to(dtype)
    table = synth.build_block_table(lens, bs, pool, gen)
    return q, k, v, table, lens


def _oracle(q, k, v, table, lens, scale=None):
    """torch fp32 oracle on the GPU copies (the checker, never the product)."""
    return gqa_oracle.reference_gqa_decode(q, k, v, table, lens, scale=scale)


# --------------------------------------------------------------------------- golden
@pytest.mark.parametrize("kernel", ["auto", "simt"])
@pytest.mark.parametrize("name", full_cases())
def test_golden_full(name, kernel):
    q, k, v, table, lens, scale, want = load_full(name)
    got = attn.gqa_decode(*_cuda(q, k, v, table, lens), scale=scale, kernel=kernel)
    assert got.dtype == q.dtype and got.shape == q.shape
    _assert_close(got, want, q.dtype, name)


@pytest.mark.parametrize("kernel", ["auto", "simt"])
@pytest.mark.parametrize("name", seed_cases())
def test_golden_seeded(name, kernel):
    (q, k, v, table, lens), want = load_seeded(name)
    got = attn.gqa_decode(*_cuda(q, k, v, table, lens), kernel=kernel)
    _assert_close(got, want, q.dtype, name)


@pytest.mark.parametrize("chunk", [16, 48, 512])
@pytest.mark.parametrize("name", ["seed_c2_small_bf16", "seed_c3_small_fp16", "seed_c1_cpu_fp32"])
def test_golden_seeded_forced_chunks(name, chunk):
    """Many small KV chunks (down to one tile) exercise plan + partials + merge."""
    (q, k, v, table, lens), want = load_seeded(name)
    got = attn.gqa_decode(*_cuda(q, k, v, table, lens), chunk_tokens=chunk)
    _assert_close(got, want, q.dtype, f"{name} chunk={chunk}")


def test_reference_import_name_runs_the_same_kernels():
    """The reference's callers write `import attention; attention.gqa_decode(*tensors)`
    positionally (benchmarks/bench_gqa_decode.py:43)."""
    import attention
    (q, k, v, table, lens), want = load_seeded("seed_c2_small_bf16")
    tensors = _cuda(q, k, v, table, lens)
    got = attention.gqa_decode(*tensors)
    _assert_close(got, want, q.dtype, "import attention")
    assert torch.equal(got, attn.gqa_decode(*tensors))
    assert attention.is_cuda_extension_loaded()


# --------------------------------------------------------------------------- edge grid
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bs", [1, 8, 16, 32, 64, 5, 24])
def test_lengths_around_page_edges(dtype, bs):
    lengths = [0, 1, max(1, bs - 1), bs, bs + 1, 3 * bs, 3 * bs + 1, 0, 7 * bs - 1]
    q, k, v, table, lens = _make_case(lengths, 8, 2, 128, bs, dtype, seed=bs)
    dq, dk, dv, dt, dl = _cuda(q, k, v, table, lens)
    want = _oracle(dq, dk, dv, dt, dl)
    for kernel in ("auto", "simt"):
        for chunk in (0, 16):
            got = attn.gqa_decode(dq, dk, dv, dt, dl, kernel=kernel, chunk_tokens=chunk)
            _assert_close(got, want, dtype, f"bs={bs} {kernel} chunk={chunk}")
            assert torch.count_nonzero(got[0]) == 0 and torch.count_nonzero(got[7]) == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 1), (8, 2), (10, 2), (28, 4), (64, 8), (32, 1),
                                     (40, 2), (3, 3)])
def test_head_groupings(dtype, hq, hkv):
    """MHA, MQA, groups 4/5/7/8, and groups of 20 and 32 (more than one head group per item)."""
    q, k, v, table, lens = _make_case([70, 33, 129], hq, hkv, 128, 16, dtype, seed=hq * 100 + hkv)
    args = _cuda(q, k, v, table, lens)
    want = _oracle(*args)
    for kernel in ("auto", "simt"):
        _assert_close(attn.gqa_decode(*args, kernel=kernel), want, dtype, f"{hq}/{hkv} {kernel}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d", [1, 8, 32, 64, 80, 96, 128, 192, 256])
def test_head_dims(dtype, d):
    q, k, v, table, lens = _make_case([45, 16, 100], 8, 2, d, 16, dtype, seed=d)
    args = _cuda(q, k, v, table, lens)
    want = _oracle(*args)
    _assert_close(attn.gqa_decode(*args), want, dtype, f"D={d} auto")
    _assert_close(attn.gqa_decode(*args, kernel="simt", chunk_tokens=32), want, dtype, f"D={d} simt")


def test_exact_capacity_and_poisoned_slots():
    bs, pages = 16, 6
    lengths = [bs * pages, 5, bs * pages - 1]
    q, k, v, table, lens = _make_case(lengths, 8, 2, 128, bs, torch.bfloat16, seed=4)
    assert table.shape[1] == pages and (table[1, 1:] == -1).all()
    args = _cuda(q, k, v, table, lens)
    _assert_close(attn.gqa_decode(*args), _oracle(*args), torch.bfloat16)


@pytest.mark.parametrize("scale", [0.03, 1.0, 2.5])
def test_custom_scale(scale):
    q, k, v, table, lens = _make_case([90, 17], 8, 2, 64, 16, torch.float16, seed=1)
    args = _cuda(q, k, v, table, lens)
    _assert_close(attn.gqa_decode(*args, scale=scale), _oracle(*args, scale=scale), torch.float16)
    _assert_close(attn.gqa_decode(*args, scale=scale, kernel="simt"), _oracle(*args, scale=scale),
                  torch.float16)


def test_unaligned_views_take_the_generic_kernel():
    """A q whose storage offset is not 16-byte aligned is still a valid contiguous input."""
    q, k, v, table, lens = _make_case([50, 20], 8, 2, 128, 16, torch.bfloat16, seed=2)
    dq, dk, dv, dt, dl = _cuda(q, k, v, table, lens)
    flat = torch.empty(dq.numel() + 1, dtype=dq.dtype, device=DEV)
    q_off = flat[1:].view_as(dq)
    q_off.copy_(dq)
    assert q_off.data_ptr() % 16 != 0 and q_off.is_contiguous()
    _assert_close(attn.gqa_decode(q_off, dk, dv, dt, dl), _oracle(dq, dk, dv, dt, dl), torch.bfloat16)
    with pytest.raises(RuntimeError):
        attn.gqa_decode(q_off, dk, dv, dt, dl, kernel="mma")


def test_out_and_workspace_arguments():
    q, k, v, table, lens = _make_case([300, 40, 1000], 8, 2, 128, 16, torch.bfloat16, seed=3)
    args = _cuda(q, k, v, table, lens)
    want = _oracle(*args)
    out = torch.full_like(args[0], float("nan"))
    need = attn.workspace_bytes(3, 8, 2, 128, 16, table.shape[1], 64)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)      # control words start at zero
    res = attn.gqa_decode(*args, out=out, workspace=ws, chunk_tokens=64)
    assert res is out
    _assert_close(out, want, torch.bfloat16)
    hdr = ws[:20].view(torch.int32).cpu()
    assert int(hdr[2]) == 0 and int(hdr[1]) == sum(-(-n // 64) for n in (300, 40, 1000))
    assert int(hdr[0]) == 0 and int(hdr[4]) == 0               # counters back at zero
    # the three-launch path on the same workspace, and the one- and two-launch paths after it
    out3 = attn.gqa_decode(*args, workspace=ws, chunk_tokens=64, phases=7)
    assert torch.equal(out3, out)
    assert torch.equal(attn.gqa_decode(*args, workspace=ws, chunk_tokens=64, phases=8), out)
    assert torch.equal(attn.gqa_decode(*args, workspace=ws, chunk_tokens=64, phases=16), out)
    small = torch.empty(need - 256, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="workspace"):
        attn.gqa_decode(*args, workspace=small, chunk_tokens=64)


def test_batch_zero_returns_empty():
    q, k, v, table, lens = _make_case([5], 8, 2, 128, 16, torch.float16)
    dq, dk, dv, dt, dl = _cuda(q, k, v, table, lens)
    out = attn.gqa_decode(dq[:0], dk, dv, dt[:0], dl[:0])
    assert out.shape == (0, 8, 128)


def test_persistent_grid_smaller_than_work():
    """Few CTAs pulling many items from the device-side counter."""
    q, k, v, table, lens = _make_case([700, 33, 512, 1, 64], 8, 4, 128, 16, torch.bfloat16, seed=8)
    args = _cuda(q, k, v, table, lens)
    want = _oracle(*args)
    for kernel in ("mma", "simt"):
        got = attn.gqa_decode(*args, chunk_tokens=32, max_ctas=3, kernel=kernel)
        _assert_close(got, want, torch.bfloat16, kernel)


def test_repeated_calls_are_bit_identical():
    q, k, v, table, lens = _make_case([2000, 900, 4500], 32, 8, 128, 16, torch.bfloat16, seed=5)
    args = _cuda(q, k, v, table, lens)
    a = attn.gqa_decode(*args).clone()
    for _ in range(3):
        assert torch.equal(a, attn.gqa_decode(*args))


# --------------------------------------------------------------------------- split front door
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits", [1, 2, 3, 8, 64])
def test_split_matches_oracle_and_reference_partial_layout(dtype, splits):
    lengths = [0, 5, 130, 47]       # 5 tokens < 8 splits: empty partitions
    q, k, v, table, lens = _make_case(lengths, 8, 2, 128, 16, dtype, seed=splits)
    args = _cuda(q, k, v, table, lens)
    want = _oracle(*args)
    got = attn.gqa_decode_split(*args, splits=splits)
    _assert_close(got, want, dtype, f"splits={splits}")
    if splits > 1:
        ws = torch.full((4, 8, splits, 130), float("nan"), dtype=torch.float32, device=DEV)
        got = attn.gqa_decode_split(*args, splits=splits, workspace=ws)
        _assert_close(got, want, dtype)
        mx, sm, acc = gqa_oracle.split_partials_f64(q, k, v, table, lens, splits)
        ws = ws.cpu().double()
        live = torch.from_numpy(sm) > 0
        tol = 1e-3 if dtype == torch.float32 else 3e-2
        assert torch.equal(ws[..., 1] > 0, live)
        assert (ws[..., 0][~live] == -math.inf).all() and (ws[..., 2:][~live] == 0).all()
        # partials are relative to each partition's own max: compare max, and acc/sum
        torch.testing.assert_close(ws[..., 0][live], torch.from_numpy(mx)[live], atol=tol, rtol=tol)
        ratio = ws[..., 2:][live] / ws[..., 1][live].unsqueeze(-1)
        ref = torch.from_numpy(acc)[live] / torch.from_numpy(sm)[live].unsqueeze(-1)
        torch.testing.assert_close(ratio, ref, atol=tol, rtol=tol)


def test_split_argument_errors():
    q, k, v, table, lens = _make_case([40], 8, 2, 128, 16, torch.float16)
    args = _cuda(q, k, v, table, lens)
    with pytest.raises(RuntimeError, match="splits"):
        attn.gqa_decode_split(*args, splits=0)
    with pytest.raises(RuntimeError, match="workspace requires"):
        attn.gqa_decode_split(*args, splits=1, workspace=torch.empty(1, 8, 1, 130, device=DEV))
    with pytest.raises(RuntimeError, match="workspace shape"):
        attn.gqa_decode_split(*args, splits=2, workspace=torch.empty(1, 8, 3, 130, device=DEV))
    with pytest.raises(ValueError):
        attn.gqa_decode_split(*args, backend="triton")


def test_auto_front_door():
    q, k, v, table, lens = _make_case([900, 40], 8, 2, 128, 16, torch.bfloat16, seed=6)
    args = _cuda(q, k, v, table, lens)
    _assert_close(attn.gqa_decode_auto(*args), _oracle(*args), torch.bfloat16)
    with pytest.raises(ValueError):
        attn.gqa_decode_auto(args[0][0], *args[1:])


# --------------------------------------------------------------------------- argument checks
def test_every_reference_check_raises_runtime_error():
    q, k, v, table, lens = _cuda(*_make_case([40, 9], 8, 2, 128, 16, torch.float16))
    bad = [
        (dict(q=q.cpu()), "CUDA tensor"),
        (dict(q=q.transpose(0, 1)), "contiguous"),
        (dict(q=q[0]), r"q must be \[B, Hq, D\]"),
        (dict(k=k[0]), "k_cache must be"),
        (dict(v=v[:1]), "v_cache shape mismatch"),
        (dict(table=table[0]), "block_table must be"),
        (dict(lens=lens.view(2, 1)), "context_lens must be"),
        (dict(q=q.float()), "dtype must match"),
        (dict(q=q.double(), k=k.double(), v=v.double()), "float32/float16/bfloat16"),
        (dict(table=table.long()), "int32"),
        (dict(lens=lens[:1]), "batch sizes must match"),
        (dict(q=q[:, :, :64].contiguous()), "head_dim must match"),
        (dict(q=q[:, :7].contiguous()), "divisible"),
        (dict(scale=0.0), "scale"),
        (dict(scale=float("inf")), "scale"),
        (dict(scale=-1.0), "scale"),
    ]
    for change, pattern in bad:
        a = dict(q=q, k=k, v=v, table=table, lens=lens, scale=None)
        a.update(change)
        with pytest.raises(RuntimeError, match=pattern):
            attn.gqa_decode(a["q"], a["k"], a["v"], a["table"], a["lens"], scale=a["scale"])
    big = torch.empty(2, 8, 512, dtype=torch.float16, device=DEV)
    kk = torch.empty(4, 16, 2, 512, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="head_dim"):
        attn.gqa_decode(big, kk, kk, table, lens)


# --------------------------------------------------------------------------- kv_append
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("d", [128, 5])
def test_kv_append_matches_oracle_then_decode(dtype, d):
    lengths = [40, 9, 64, 1]
    q, k, v, table, lens = _make_case(lengths, 8, 2, d, 16, dtype, seed=d, pool_extra=0)
    # appending at position == length may need a fresh page for sequences at a page edge
    table = torch.cat([table, torch.full((4, 1), -1, dtype=torch.int32)], dim=1)
    pool = k.shape[0]
    k = torch.cat([k, torch.zeros(4, *k.shape[1:], dtype=dtype)])
    v = torch.cat([v, torch.zeros(4, *v.shape[1:], dtype=dtype)])
    for b, n in enumerate(lengths):
        if n % 16 == 0:
            table[b, n // 16] = pool + b
    pos = lens.clone()
    key = torch.randn(4, 2, d).to(dtype)
    val = torch.randn(4, 2, d).to(dtype)
    attn.validate_paged_metadata(table, lens, block_size=16, num_blocks=k.shape[0], positions=pos)
    k_ref, v_ref = k.clone(), v.clone()
    gqa_oracle.reference_kv_append(key, val, k_ref, v_ref, table, pos)
    dk, dv = k.to(DEV), v.to(DEV)
    attn.kv_append(key.to(DEV), val.to(DEV), dk, dv, table.to(DEV), pos.to(DEV))
    assert torch.equal(dk.cpu(), k_ref) and torch.equal(dv.cpu(), v_ref)
    new_lens = (lens + 1).to(DEV)
    got = attn.gqa_decode(q.to(DEV), dk, dv, table.to(DEV), new_lens)
    want = _oracle(q.to(DEV), k_ref.to(DEV), v_ref.to(DEV), table.to(DEV), new_lens)
    _assert_close(got, want, dtype)


def test_kv_append_skips_out_of_range_positions():
    q, k, v, table, lens = _make_case([10, 10], 8, 2, 64, 16, torch.float16, seed=9)
    dk, dv = k.to(DEV), v.to(DEV)
    key = torch.randn(2, 2, 64).half().to(DEV)
    pos = torch.tensor([-1, 16 * table.shape[1]], dtype=torch.int32, device=DEV)
    attn.kv_append(key, key, dk, dv, table.to(DEV), pos)
    assert torch.equal(dk.cpu(), k) and torch.equal(dv.cpu(), v)


# --------------------------------------------------------------------------- randomized shapes
def test_randomized_shapes_against_oracle():
    """Seeded sweep over dtypes, head layouts, head sizes, page sizes, chunk lengths and
    ragged batches (with empty and one-token sequences mixed in)."""
    rng = torch.Generator().manual_seed(1234)

    def pick(options):
        return options[int(torch.randint(len(options), (1,), generator=rng))]

    for case in range(40):
        dtype = pick([torch.float32, torch.float16, torch.bfloat16])
        hkv = pick([1, 2, 3, 4, 8])
        group = pick([1, 2, 4, 5, 7, 8, 16, 20])
        d = pick([64, 128, 128, 128, 256, 32, 80, 100])
        bs = pick([1, 4, 8, 16, 16, 32, 64, 128, 12])
        batch = pick([1, 2, 5, 17])
        top = pick([1, 40, 300, 1500])
        lengths = torch.randint(0, top + 1, (batch,), generator=rng).tolist()
        if case % 4 == 0:
            lengths[0] = 0
        chunk = pick([0, 0, 16, 64, 512])
        kernel = pick(["auto", "auto", "simt"])
        q, k, v, table, lens = _make_case(lengths, hkv * group, hkv, d, bs, dtype, seed=case)
        args = _cuda(q, k, v, table, lens)
        got = attn.gqa_decode(*args, chunk_tokens=chunk, kernel=kernel)
        _assert_close(got, _oracle(*args), dtype,
                      f"case {case}: {dtype} Hkv={hkv} G={group} D={d} bs={bs} L={lengths} "
                      f"chunk={chunk} {kernel}")


# --------------------------------------------------------------------------- one, two, three launches
ONE_LAUNCH, TWO_LAUNCH, THREE_LAUNCH = 8, 16, 7     # `phases` values that force a path


@pytest.mark.parametrize("kernel", ["auto", "simt"])
@pytest.mark.parametrize("chunk", [0, 16, 64, 512])
def test_one_two_and_three_launch_paths_agree(kernel, chunk):
    """Same chunk list, same partial slots, same merge arithmetic: with an explicit chunk length
    the three paths give identical bits; with the automatic one (the plan kernel and the
    self-planning decode kernel may pick different bases) they agree within the tolerance."""
    lengths = [0, 1, 15, 16, 17, 300, 0, 1000, 64, 2500, 33, 4097, 5]
    for dtype, hq, hkv in ((torch.bfloat16, 32, 8), (torch.float16, 28, 4), (torch.float32, 8, 2)):
        q, k, v, table, lens = _make_case(lengths, hq, hkv, 128, 16, dtype, seed=chunk + hq)
        args = _cuda(q, k, v, table, lens)
        one = attn.gqa_decode(*args, kernel=kernel, chunk_tokens=chunk, phases=ONE_LAUNCH)
        two = attn.gqa_decode(*args, kernel=kernel, chunk_tokens=chunk, phases=TWO_LAUNCH)
        three = attn.gqa_decode(*args, kernel=kernel, chunk_tokens=chunk, phases=THREE_LAUNCH)
        default = attn.gqa_decode(*args, kernel=kernel, chunk_tokens=chunk)
        assert torch.equal(one, two), f"{dtype} {kernel} chunk={chunk}"
        assert torch.equal(default, two), f"{dtype} {kernel} chunk={chunk}"
        if chunk:
            assert torch.equal(one, three), f"{dtype} {kernel} chunk={chunk}"
        _assert_close(one, three, dtype)
        _assert_close(one, _oracle(*args), dtype, f"{dtype} {kernel} chunk={chunk}")
        assert torch.count_nonzero(one[0]) == 0 and torch.count_nonzero(one[6]) == 0


def test_default_path_follows_the_static_shape():
    """A batch whose every possible work item fits a CTA of its own takes one launch (the
    workspace's plan words are written, no merge launch is needed); a larger table takes two."""
    q, k, v, table, lens = _make_case([300, 40, 500], 8, 2, 128, 16, torch.bfloat16, seed=8)
    args = _cuda(q, k, v, table, lens)
    want = _oracle(*args)
    _assert_close(attn.gqa_decode(*args), want, torch.bfloat16, "small table")
    wide = torch.full((3, 4096), -1, dtype=torch.int32)
    wide[:, : table.shape[1]] = table
    args_wide = _cuda(q, k, v, wide, lens)
    _assert_close(attn.gqa_decode(*args_wide), want, torch.bfloat16, "wide table")


def test_one_launch_path_leaves_the_workspace_clean():
    """After any call the work counter, the exit counter and every ticket are zero again, so the
    next call (other lengths, other shape) can use the same workspace without clearing it."""
    lib_need = attn.workspace_bytes(6, 32, 8, 128, 16, 400, 0)
    ws = torch.zeros(lib_need, dtype=torch.uint8, device=DEV)
    control = int(_cabi.load().gqa_b200_workspace_control_bytes())   # header + tickets
    for seed, lengths in enumerate(([3000, 70, 0, 6000, 1, 999], [16, 16, 16, 16, 16, 16],
                                    [6400, 6400, 6400, 1, 0, 0])):
        q, k, v, table, lens = _make_case(lengths, 32, 8, 128, 16, torch.bfloat16, seed=seed)
        wide = torch.full((6, 400), -1, dtype=torch.int32)
        wide[:, : table.shape[1]] = table
        args = _cuda(q, k, v, wide, lens)
        for chunk in (0, 64):
            if attn.workspace_bytes(6, 32, 8, 128, 16, 400, chunk) > lib_need:
                continue
            got = attn.gqa_decode(*args, workspace=ws, chunk_tokens=chunk, phases=ONE_LAUNCH)
            _assert_close(got, _oracle(*args), torch.bfloat16, f"{lengths} chunk={chunk}")
            words = ws[:control].view(torch.int32).cpu()
            assert int(words[0]) == 0 and int(words[4]) == 0, "counters not released"
            assert int(words[64:].abs().sum()) == 0, "a ticket was left behind"


def test_calls_of_different_shapes_share_one_workspace():
    """The control words sit at a fixed place, so the partials a small-shape call writes can
    never be what a later, larger call reads as its arrival counters."""
    big = attn.workspace_bytes(40, 128, 8, 256, 16, 100, 0)
    ws = torch.zeros(big, dtype=torch.uint8, device=DEV)
    shapes = [(3, 8, 2, 128, torch.bfloat16), (40, 128, 8, 256, torch.float32),
              (7, 28, 4, 128, torch.float16), (40, 128, 8, 256, torch.float32)]
    gen = torch.Generator().manual_seed(3)
    for i, (batch, hq, hkv, d, dtype) in enumerate(shapes):
        lengths = torch.randint(1, 1500, (batch,), generator=gen).tolist()
        q, k, v, table, lens = _make_case(lengths, hq, hkv, d, 16, dtype, seed=i)
        args = _cuda(q, k, v, table, lens)
        for kernel in ("auto", "simt"):
            for phases in (0, ONE_LAUNCH, TWO_LAUNCH, THREE_LAUNCH):
                got = attn.gqa_decode(*args, workspace=ws, kernel=kernel, phases=phases)
                _assert_close(got, _oracle(*args), dtype, f"shape {i} {kernel} phases={phases}")


def test_batches_beyond_the_self_planning_limit_take_three_launches():
    """More than 2048 sequences: the prefix array no longer fits the decode CTA's shared memory,
    the call falls back to plan + decode + merge."""
    gen = torch.Generator().manual_seed(11)
    lengths = torch.randint(0, 90, (2100,), generator=gen).tolist()
    q, k, v, table, lens = _make_case(lengths, 8, 2, 64, 16, torch.float16, seed=12)
    args = _cuda(q, k, v, table, lens)
    _assert_close(attn.gqa_decode(*args), _oracle(*args), torch.float16)


# --------------------------------------------------------------------------- stream capture
def test_decode_can_be_captured_in_a_cuda_graph_and_replayed():
    """No allocation, no host read of the lengths, no synchronisation inside the call: the
    launch can be recorded once and replayed on new contents of the same buffers (every run
    leaves the workspace's control words at zero for the next)."""
    q, k, v, table, lens = _make_case([900, 40, 2500, 0, 64], 32, 8, 128, 16, torch.bfloat16, seed=21)
    dq, dk, dv, dt, dl = _cuda(q, k, v, table, lens)
    out = torch.empty_like(dq)
    ws = torch.zeros(attn.workspace_bytes(5, 32, 8, 128, 16, table.shape[1]), dtype=torch.uint8,
                     device=DEV)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        attn.gqa_decode(dq, dk, dv, dt, dl, out=out, workspace=ws)     # warm-up outside capture
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        attn.gqa_decode(dq, dk, dv, dt, dl, out=out, workspace=ws)
    graph.replay()
    torch.cuda.synchronize()
    _assert_close(out, _oracle(dq, dk, dv, dt, dl), torch.bfloat16, "first replay")
    # new query, shorter/longer lengths within the same table, same buffers
    dq.copy_(torch.randn_like(dq))
    dl.copy_(torch.tensor([17, 33, 1200, 0, 5], dtype=torch.int32))   # within each row's pages
    graph.replay()
    torch.cuda.synchronize()
    _assert_close(out, _oracle(dq, dk, dv, dt, dl), torch.bfloat16, "second replay")


def test_batches_larger_than_the_plan_kernels_block():
    """More sequences than the plan kernel has threads (its scan runs in several rounds), with
    empty, one-chunk and many-chunk sequences mixed."""
    gen = torch.Generator().manual_seed(5)
    lengths = torch.randint(0, 120, (2500,), generator=gen).tolist()
    lengths[7] = 700
    lengths[1999] = 0
    q, k, v, table, lens = _make_case(lengths, 4, 2, 64, 16, torch.float16, seed=31)
    args = _cuda(q, k, v, table, lens)
    want = _oracle(*args)
    for chunk in (0, 16, 64):
        _assert_close(attn.gqa_decode(*args, chunk_tokens=chunk), want, torch.float16, f"chunk={chunk}")
    _assert_close(attn.gqa_decode(*args, kernel="simt", chunk_tokens=32), want, torch.float16, "simt")
