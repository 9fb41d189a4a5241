"""Where the sources and the built library live."""

from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB_PATH = LIB_DIR / "libgqa_decode_b200.so"
HEADER = PKG.parent / "include" / "gqa_decode_b200.h"
MLA_HEADER = PKG.parent / "include" / "mla_decode_b200.h"
