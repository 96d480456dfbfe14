"""In-tree build of libtacvq.so (hand-written sm_100a kernels behind a C ABI).

``python -m tac_vq_kv_cache_b200.build`` compiles every ``csrc/*.cu`` with nvcc for
``sm_100a`` only and links them into ``tac_vq_kv_cache_b200/libtacvq.so``.  nvcc
cross-compiles without a GPU, so this also runs on a CPU-only machine.  Object
files are cached under ``csrc/build/`` and rebuilt when their source, a header
or the flags change.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
TARGET = PKG / "libtacvq.so"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-I", str(INCLUDE),
    "-I", str(CSRC),
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; libtacvq.so cannot be built")
    return found


def _stamp(src: Path, extra: list[str]) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for header in sorted(list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))):
        h.update(header.read_bytes())
    h.update(" ".join(NVCC_FLAGS + extra).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    objdir = CSRC / "build"
    objdir.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    jobs = []
    objects = []
    for src in sources:
        obj = objdir / (src.stem + ".o")
        tag = objdir / (src.stem + ".stamp")
        objects.append(obj)
        stamp = _stamp(src, extra)
        if not force and obj.exists() and tag.exists() and tag.read_text() == stamp:
            continue
        jobs.append((src, obj, tag, stamp))

    def compile_one(job):
        src, obj, tag, stamp = job
        cmd = [nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose or ptxas_info:
            sys.stderr.write(res.stderr)
        tag.write_text(stamp)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(compile_one, jobs))
    if jobs or not TARGET.exists():
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
               *map(str, objects), "-o", str(TARGET)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return TARGET


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
