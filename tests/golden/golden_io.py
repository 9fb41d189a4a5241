"""Read/write helpers for the golden fixtures (npz files; bf16 kept as raw uint16)."""

from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import torch

GOLDEN_DIR = Path(__file__).resolve().parent
_DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def from_np(a: np.ndarray, dtype_name: str) -> torch.Tensor:
    if dtype_name == "bfloat16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(a.copy())


def dtype_of(name: str) -> torch.dtype:
    return _DT[name]


def digest(*tensors: torch.Tensor) -> str:
    """sha256 over the raw bytes of the tensors, in order."""
    h = hashlib.sha256()
    for t in tensors:
        h.update(to_np(t).tobytes())
    return h.hexdigest()
