"""pytest configuration: the ``gpu`` marker and shared fixture loaders."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
for p in (ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

from golden_io import GOLDEN_DIR, digest, dtype_of, from_np  # noqa: E402

from attention_b200 import synth  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# fp32 follows the reference's own fp32 convention; fp16/bf16 are the stated bars.
TOL = {torch.float32: 1e-4, torch.float16: 2e-3, torch.bfloat16: 1e-2}


def full_cases():
    return sorted(p.stem for p in GOLDEN_DIR.glob("full_*.npz"))   # decode, inputs stored


def seed_cases():
    return sorted(p.stem for p in GOLDEN_DIR.glob("seed_*.npz"))


def load_full(name):
    """-> (q, k, v, table, lens, scale_or_None, reference_out)"""
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    dn = str(z["dtype"])
    scale = float(z["scale"])
    return (from_np(z["q"], dn), from_np(z["k"], dn), from_np(z["v"], dn),
            torch.from_numpy(z["table"].copy()), torch.from_numpy(z["lens"].copy()),
            None if scale < 0 else scale, from_np(z["out"], dn))


def load_seeded(name):
    """Regenerate a seeded case and return (inputs tuple, reference_out).

    Fails loudly if the regenerated inputs do not hash to the stored digest (a
    random-number-generator drift would otherwise look like a parity failure).
    """
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    dn = str(z["dtype"])
    b, hq, hkv, d, bs, lo, hi, fixed = (int(x) for x in z["workload"])
    w = synth.DecodeWorkload(name, b, hq, hkv, d, bs, dtype_of(dn), lo, hi,
                             len_dist=str(z["len_dist"]), fixed_pool_blocks=fixed)
    inputs = synth.make_workload(w, seed=int(z["seed"]))
    assert digest(*inputs) == str(z["digest"]), "regenerated inputs differ from the fixture's"
    return inputs, from_np(z["out"], dn)


def prefill_cases():
    return sorted(p.stem for p in GOLDEN_DIR.glob("prefill_*.npz"))


def load_prefill(name):
    """-> (q, k, v, q_lens, kv_lens, causal, scale_or_None, reference_out)"""
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    dn = str(z["dtype"])
    scale = float(z["scale"])
    return (from_np(z["q"], dn), from_np(z["k"], dn), from_np(z["v"], dn),
            torch.from_numpy(z["q_lens"].copy()), torch.from_numpy(z["kv_lens"].copy()),
            bool(int(z["causal"])), None if scale < 0 else scale, from_np(z["out"], dn))


def mla_cases():
    return sorted(p.stem for p in GOLDEN_DIR.glob("mla_*.npz"))


def load_mla(name):
    """-> (dict of input tensors incl. optional 'indices', causal, reference_out [B,T,H,Dv])"""
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    dn = str(z["dtype"])
    c = {k: from_np(z[k], dn) for k in ("q_nope", "q_rope", "w_uk", "w_uv", "cache")}
    for k in ("block_table", "lengths", "positions"):
        c[k] = torch.from_numpy(z[k].copy())
    c["indices"] = torch.from_numpy(z["indices"].copy()) if "indices" in z.files else None
    return c, bool(int(z["causal"])), from_np(z["out"], dn)
