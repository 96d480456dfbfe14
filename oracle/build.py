"""Build recipe for the plain-C oracle (test infrastructure, not product code).

``python -m oracle.build`` compiles oracle/tacvq_oracle.c into
oracle/libtacvq_oracle.so with gcc.  ``-ffp-contract=off`` keeps every
multiply and add separately rounded (the source spells out the fused ones with
``fmaf``); ``-mfma -mf16c`` make ``fmaf`` and the fp16 conversions single
hardware instructions with IEEE rounding.  No ``-march=native``: the library is
built on one machine and loaded on another.

The reference project is pure Python, so there is nothing of it to compile here
(no ``oracle/_ref`` binary); the reference is pinned through the golden vectors
written by tests/golden/make_golden.py instead.
"""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "tacvq_oracle.c"
TARGET = HERE / "libtacvq_oracle.so"


def build(force: bool = False) -> Path:
    if not force and TARGET.exists() and TARGET.stat().st_mtime >= SOURCE.stat().st_mtime:
        return TARGET
    cmd = [
        "gcc", "-O2", "-std=gnu11", "-fPIC", "-shared", "-fopenmp", "-mfma", "-mf16c", "-ffp-contract=off",
        "-Wall", "-Wextra", str(SOURCE), "-o", str(TARGET), "-lm",
    ]
    subprocess.run(cmd, check=True)
    return TARGET


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
