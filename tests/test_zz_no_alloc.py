"""gqa_b200_decode_static: the entry point for callers that cannot allocate.

Some users of the C ABI have no scratch to give: all free HBM already belongs to
their KV page pool, or they sit in a decode loop where cudaMalloc's device-wide
synchronisation is not acceptable, or their host runtime owns device memory.
For them the library carries an 8 MiB scratch array of its own.  This test calls
that entry point directly through the C ABI, twice in a row on different inputs
(the array is shared and keeps the previous call's contents), and checks each
result against the ordinary entry point, which gets a workspace from the caller:
both run the same plan, decode and merge on the same inputs, so the results must
be equal bit for bit.  It also checks that the free device memory does not move
across a call, and that the size limit is enforced from both sides: a shape whose
scratch need is just inside the built-in array runs, one just outside is refused.

The file name sorts last on purpose: with ``-x`` every other test has already
run when this one does.  It does not depend on them and passes on its own.
"""

import pytest
import torch

from attention_b200 import _cabi, synth

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
STATIC_LIMIT = -14


def _args(q, k, v, table, lens, out):
    return (q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), lens.data_ptr(),
            out.data_ptr(), DTYPE_CODE[q.dtype], q.size(0), q.size(1), k.size(2), q.size(2),
            k.size(0), k.size(1), table.size(1), 1.0 / q.size(2) ** 0.5)


def _decode_with_caller_workspace(lib, q, k, v, table, lens):
    out = torch.empty_like(q)
    need = lib.gqa_b200_workspace_bytes(q.size(0), q.size(1), k.size(2), q.size(2), k.size(1),
                                        table.size(1), 0)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    # a fresh workspace: its control words are zeroed once, through the C ABI
    rc = lib.gqa_b200_workspace_init(ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, _cabi.strerror(rc)
    rc = lib.gqa_b200_decode(*_args(q, k, v, table, lens, out), ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, _cabi.strerror(rc)
    return out


def _decode_static(lib, q, k, v, table, lens):
    out = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.gqa_b200_decode_static(*_args(q, k, v, table, lens, out), stream)
    return rc, out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = _cabi.load()
    cases = [
        synth.scaled("c2_qwen3_8b_bf16", batch=6, len_lo=200, len_hi=3000),   # several chunks each
        synth.scaled("c3_qwen25_7b_fp16", batch=9, len_lo=1, len_hi=700),     # different shape next
        synth.scaled("c1_cpu_fp32", batch=3, len_lo=64, len_hi=400, fixed_pool_blocks=0),
    ]
    for i, w in enumerate(cases):
        inputs = synth.make_workload(w, seed=100 + i, device=DEV, kv_on_device=True)
        want = _decode_with_caller_workspace(lib, *inputs)
        rc, got = _decode_static(lib, *inputs)
        assert rc == 0, _cabi.strerror(rc)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        # same inputs again straight away: stale scratch from the call before must not matter,
        # and the call must leave the amount of free device memory where it was
        out = torch.full_like(inputs[0], float("nan"))
        stream = torch.cuda.current_stream().cuda_stream
        args = _args(*inputs, out)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.gqa_b200_decode_static(*args, stream)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert rc == 0
        assert free_after == free_before, "the static entry point must not allocate device memory"
        assert torch.equal(out, want)


def test_static_scratch_limit_from_both_sides():
    """The widest block table whose worst-case scratch still fits the built-in array is
    accepted (and gives the ordinary entry point's bits); one page more is refused."""
    lib = _cabi.load()
    w = synth.scaled("c2_qwen3_8b_bf16", batch=8, len_lo=100, len_hi=900)
    q, k, v, table, lens = synth.make_workload(w, seed=5, device=DEV, kv_on_device=True)
    limit = 8 << 20

    def need(pages):
        return lib.gqa_b200_workspace_bytes(w.batch, w.q_heads, w.kv_heads, w.head_dim, w.block_size,
                                            pages, 0)

    lo, hi = table.size(1), 1 << 22            # need(lo) fits, need(hi) does not
    assert need(lo) <= limit < need(hi)
    while hi - lo > 1:                         # need() is monotone in the table width
        mid = (lo + hi) // 2
        if need(mid) <= limit:
            lo = mid
        else:
            hi = mid
    assert need(lo) <= limit < need(lo + 1)

    def widened(pages):
        t = torch.full((w.batch, pages), -1, dtype=torch.int32, device=DEV)
        t[:, : table.size(1)] = table
        return t

    inside, outside = widened(lo), widened(lo + 1)
    want = _decode_with_caller_workspace(lib, q, k, v, inside, lens)
    rc, got = _decode_static(lib, q, k, v, inside, lens)
    assert rc == 0, _cabi.strerror(rc)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    rc, out = _decode_static(lib, q, k, v, outside, lens)
    assert rc == STATIC_LIMIT
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()          # nothing was launched


def test_static_scratch_entry_point_refuses_shapes_beyond_its_limit():
    lib = _cabi.load()
    w = synth.scaled("c2_qwen3_8b_bf16", batch=2, len_lo=20, len_hi=40)
    q, k, v, table, lens = synth.make_workload(w, seed=1, device=DEV, kv_on_device=True)
    # a wide table: the worst-case scratch for 2 x 4M-token tables is far beyond 8 MiB
    wide = torch.full((2, 1 << 18), -1, dtype=torch.int32, device=DEV)
    wide[:, : table.size(1)] = table
    need = lib.gqa_b200_workspace_bytes(2, w.q_heads, w.kv_heads, w.head_dim, w.block_size,
                                        wide.size(1), 0)
    assert need > (8 << 20)
    rc, out = _decode_static(lib, q, k, v, wide, lens)
    assert rc == STATIC_LIMIT
    assert "GQA_B200_STATIC_SCRATCH_BYTES" in _cabi.strerror(rc)
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()          # nothing was launched
    # the same sequences through a table of ordinary width are accepted
    rc, out = _decode_static(lib, q, k, v, table, lens)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
