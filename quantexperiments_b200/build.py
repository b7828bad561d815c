"""In-tree build of libcbl.so (hand-written CUDA for sm_100a behind a C ABI).

    python -m quantexperiments_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU; the shared object is written next to this file so that it
travels with the source tree. Nothing is cached outside the tree."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libcbl.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "cbl.h"]
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel for sm_100a into libcbl.so; returns its path."""
    if not force and not _stale():
        return LIB
    cmd = ["nvcc", *ARCH, "-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC", "--threads", "0",
           "-I", str(PKG.parent / "include"), *(["-Xptxas", "-v"] if verbose else []),
           *[str(s) for s in sources()], "-o", str(LIB)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError(f"nvcc failed ({r.returncode}): {' '.join(cmd)}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
