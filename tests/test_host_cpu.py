"""CPU-only checks: the C ABI loads and exports what the header declares, the
host-side policy/validation/sharding logic, and the no-fallback rule."""

import re
from pathlib import Path

import pytest
import torch

import attention_b200 as attn
from attention_b200 import _cabi, sharding, synth
from attention_b200._paths import HEADER, MLA_HEADER

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = HEADER.read_text() + MLA_HEADER.read_text()
    return re.findall(r"GQA_B200_API\s+[\w\s\*]+?\b((?:gqa|mla)_b200_\w+)\s*\(", text)


def test_library_loads_and_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 9 and len(set(names)) == len(names)
    lib = _cabi.load()
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(_cabi.SIGNATURES), "ctypes table and header disagree"
    assert lib.gqa_b200_abi_version() == 2
    assert attn.is_cuda_extension_loaded()


def test_strerror_covers_every_status_code():
    text = HEADER.read_text() + MLA_HEADER.read_text()
    codes = [int(c) for c in re.findall(r"#define (?:GQA|MLA)_B200_ERR_\w+\s+\((-\d+)\)", text)]
    assert codes and len(set(codes)) == len(codes)
    for c in codes:
        assert "unknown" not in _cabi.strerror(c)
    assert _cabi.strerror(0) == "ok"
    assert "unknown" in _cabi.strerror(-999)


def test_chunk_policy_depends_only_on_length():
    lib = _cabi.load()
    f = lib.gqa_b200_chunk_tokens
    assert f(1, 512) == 512 and f(16384, 512) == 512 and f(16385, 512) == 1024
    assert f(65536, 512) == 1024 and f(65537, 512) == 2048 and f(131072, 512) == 2048
    assert f(100, 64) == 64 and f(64 * 32 + 1, 64) == 128
    assert f(5, 8) < 0 and f(5, 1 << 20) < 0 and f(5, 0) < 0      # out-of-range base
    auto = lib.gqa_b200_auto_chunk_tokens
    assert auto(64, 32, 8, 16, 254) == 1024         # big batch: long chunks
    assert auto(128, 28, 4, 16, 128) == 1024
    assert auto(1, 32, 8, 16, 512) == 256           # one 8k sequence: one wave of 256 items
    assert auto(8, 32, 8, 16, 32) == 128
    assert auto(1, 32, 8, 16, 16) == 64             # one short sequence: cut as finely as allowed
    assert auto(1, 64, 8, 32, 4096) == 1024
    assert auto(2, 7, 2, 16, 4) < 0                 # heads not divisible


def test_max_chunks_bound_is_a_true_upper_bound():
    lib = _cabi.load()
    for base in (16, 64, 512):
        for bs, pages in ((16, 3), (16, 254), (32, 4028), (1, 700), (5, 9000)):
            cap = bs * pages
            bound = lib.gqa_b200_max_chunks_per_seq(pages, bs, base)
            probes = {cap, 1, 32 * base, 32 * base + 1, 128 * base, 128 * base + 1, cap // 2}
            worst = 0
            for n in probes:
                if 0 < n <= cap:
                    ct = lib.gqa_b200_chunk_tokens(n, base)
                    worst = max(worst, -(-n // ct))
            assert bound >= worst >= 1


def test_workspace_bytes_grows_with_shape_and_is_aligned():
    a = attn.workspace_bytes(64, 32, 8, 128, 16, 254)
    b = attn.workspace_bytes(128, 32, 8, 128, 16, 254)
    assert a % 256 == 0 and b > a > 0
    assert attn.workspace_bytes(4, 8, 2, 128, 16, 4, 16) > attn.workspace_bytes(4, 8, 2, 128, 16, 4, 512)


def test_compute_entry_points_reject_bad_arguments_without_a_gpu():
    """Argument errors are reported before any CUDA call, so they are checkable here."""
    lib = _cabi.load()
    one = 1   # any non-null pointer value; never dereferenced on these paths
    base = dict(dtype=2, batch=2, hq=8, hkv=2, d=128, blocks=4, bs=16, pages=2, scale=0.1)

    def call(**kw):
        a = {**base, **kw}
        return lib.gqa_b200_decode(one, one, one, one, one, one, a["dtype"], a["batch"], a["hq"],
                                   a["hkv"], a["d"], a["blocks"], a["bs"], a["pages"], a["scale"],
                                   None, 0, None)

    assert call(dtype=7) == -2
    assert call(batch=-1) == -8
    assert call(hq=7) == -3
    assert call(d=0) == -4 and call(d=257) == -4
    assert call(blocks=0) == -5 and call(bs=0) == -5
    assert call(pages=0) == -6
    assert call(scale=0.0) == -7 and call(scale=float("nan")) == -7
    assert call() == -9                      # no workspace
    assert call(batch=0) == 0                # empty batch: ok, nothing launched
    rc = lib.gqa_b200_decode_split(one, one, one, one, one, one, 2, 2, 8, 2, 128, 4, 16, 2, 0.1,
                                   0, None, None)
    assert rc == -10
    rc = lib.gqa_b200_decode_split(one, one, one, one, one, one, 2, 2, 8, 2, 128, 4, 16, 2, 0.1,
                                   2, None, None)
    assert rc == -9


def test_python_front_door_rejects_cpu_tensors_no_fallback():
    q, k, v, table, lens = synth.make_workload(
        synth.scaled("c1_cpu_fp32", batch=2, len_lo=8, len_hi=20), seed=1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        attn.gqa_decode(q, k, v, table, lens)
    with pytest.raises(RuntimeError, match="CUDA"):
        attn.kv_append(q[:, :8], q[:, :8], k, v, table, lens)


def test_product_never_imports_the_oracle():
    for path in list((ROOT / "attention_b200").rglob("*.py")) + list((ROOT / "attention_b200").rglob("*.cu*")):
        text = path.read_text()
        assert "oracle" not in text.lower() or path.name == "synth.py", path
    text = (ROOT / "attention" / "__init__.py").read_text()
    assert "import oracle" not in text and "from oracle" not in text


def test_reference_import_name_exposes_the_rebuilt_path():
    """`import attention; attention.gqa_decode(...)` is the reference's entry point
    (attention/__init__.py:2-19); here the name resolves to the B200 library."""
    import attention
    assert attention.gqa_decode is attn.gqa_decode
    for name in ("gqa_decode", "gqa_decode_split", "gqa_decode_auto", "gqa_prefill", "kv_append",
                 "is_cuda_extension_loaded", "latent_kv_write", "mla_query_absorb",
                 "mla_value_project", "mla_latent_attention", "mla_decode", "sparse_mla"):
        assert callable(getattr(attention, name)), name
        assert name in attention.__all__
    assert not hasattr(attention, "reference_gqa_decode")     # the checker is not shipped
    q, k, v, table, lens = synth.make_workload(
        synth.scaled("c1_cpu_fp32", batch=2, len_lo=8, len_hi=20), seed=1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):    # still no CPU fallback
        attention.gqa_decode(q, k, v, table, lens)


def test_validate_paged_metadata():
    table = torch.tensor([[0, 1, -1], [2, -1, -1]], dtype=torch.int32)
    lens = torch.tensor([20, 3], dtype=torch.int32)
    attn.validate_paged_metadata(table, lens, block_size=16, num_blocks=3)
    with pytest.raises(ValueError, match="invalid length"):
        attn.validate_paged_metadata(table, torch.tensor([49, 3], dtype=torch.int32),
                                     block_size=16, num_blocks=3)
    with pytest.raises(ValueError, match="invalid block at batch 0, page 1"):
        attn.validate_paged_metadata(torch.tensor([[0, 7, -1], [2, -1, -1]], dtype=torch.int32),
                                     lens, block_size=16, num_blocks=3)
    with pytest.raises(ValueError, match="int32"):
        attn.validate_paged_metadata(table.long(), lens, block_size=16, num_blocks=3)
    pos = torch.tensor([20, 3], dtype=torch.int32)
    attn.validate_paged_metadata(table, lens, block_size=16, num_blocks=3, positions=pos)
    with pytest.raises(ValueError, match="append page"):
        attn.validate_paged_metadata(table, lens, block_size=16, num_blocks=3,
                                     positions=torch.tensor([20, 16], dtype=torch.int32))
    with pytest.raises(ValueError, match="append position"):
        attn.validate_paged_metadata(table, lens, block_size=16, num_blocks=3,
                                     positions=torch.tensor([48, 3], dtype=torch.int32))
    dup = torch.tensor([[0, 1, -1], [1, -1, -1]], dtype=torch.int32)
    with pytest.raises(ValueError, match="conflicting"):
        attn.validate_paged_metadata(dup, lens, block_size=16, num_blocks=3,
                                     positions=torch.tensor([19, 3], dtype=torch.int32))


def test_synthetic_workloads_follow_the_fixture_conventions():
    for name, w in synth.WORKLOADS.items():
        small = synth.scaled(w, batch=min(w.batch, 6), len_lo=min(w.len_lo, 40),
                             len_hi=min(w.len_hi, 200), fixed_pool_blocks=0)
        q, k, v, table, lens = synth.make_workload(small, seed=3)
        assert q.dtype == k.dtype == v.dtype == w.dtype and table.dtype == lens.dtype == torch.int32
        used = (lens.long() + w.block_size - 1) // w.block_size
        cols = torch.arange(table.shape[1]).unsqueeze(0)
        in_use = cols < used.unsqueeze(1)
        assert (table[~in_use] == -1).all()
        pages = table[in_use]
        assert pages.unique().numel() == pages.numel() and pages.min() >= 0 and pages.max() < k.shape[0]
        assert k.shape[0] >= pages.numel()
        attn.validate_paged_metadata(table, lens, block_size=w.block_size, num_blocks=k.shape[0])
    lens = synth.draw_lengths(synth.WORKLOADS["c5_skewed_bf16"], torch.Generator().manual_seed(42))
    assert lens.min() >= 16 and lens.max() <= 32768
    again = synth.make_workload(synth.scaled("c2_qwen3_8b_bf16", batch=2, len_lo=10, len_hi=30), seed=5)
    once = synth.make_workload(synth.scaled("c2_qwen3_8b_bf16", batch=2, len_lo=10, len_hi=30), seed=5)
    assert all(torch.equal(a, b) for a, b in zip(again, once))


def test_algorithmic_bytes_formula():
    lens = torch.tensor([10, 0, 5], dtype=torch.int32)
    got = synth.algorithmic_bytes(lens, batch=3, q_heads=8, kv_heads=2, head_dim=128, elem_size=2)
    assert got == 15 * 2 * 128 * 2 * 2 + 2 * 3 * 8 * 128 * 2


def test_lpt_sharding_balances_the_skewed_batch():
    lens = synth.draw_lengths(synth.WORKLOADS["c5_skewed_bf16"], torch.Generator().manual_seed(42)).tolist()
    shards = sharding.lpt_assign(lens, 8)
    assert sorted(i for s in shards for i in s) == list(range(len(lens)))
    assert sharding.load_imbalance(lens, shards) < 1.01
    contiguous = [list(range(r * 32, (r + 1) * 32)) for r in range(8)]
    assert sharding.load_imbalance(lens, contiguous) > 1.2
    assert sharding.lpt_assign(lens, 8) == shards            # deterministic
    assert sharding.lpt_assign([5, 5], 4) == [[0], [1], [], []]
