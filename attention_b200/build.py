"""Build recipe of the C-ABI library (plain nvcc, sm_100a only, in-tree output).

    python -m attention_b200.build          # build if sources are newer than the .so
    python -m attention_b200.build --force
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

from ._paths import CSRC, HEADER, LIB_DIR, LIB_PATH, MLA_HEADER

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-cudart", "static", "-diag-suppress", "1886",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HEADER, MLA_HEADER]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into one shared library for sm_100a."""
    if not force and not _stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    cmd = ["nvcc", *NVCC_FLAGS, "-o", str(LIB_PATH), *map(str, sources())]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
