"""Build libturboquant.so (sm_100a only) in-tree with nvcc.

    python -m turborag_b200.build [--force] [--verbose]

Output: turborag_b200/lib/libturboquant.so.  The same file is what the
reference's ctypes wrapper expects at build/libturboquant.so; pass its path as
`lib_path` (or copy/symlink it there) to use it as a drop-in.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libturboquant.so"
SOURCES = ["tq_capi.cpp", "tq_pack.cu", "tq_dequant.cu", "tq_decode.cu",
           "tq_prefill_tc.cu", "tq_peer.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*")) + [ROOT / "include" / "turboquant.h"]
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    objs = []
    for src in _sources():
        obj = LIB_DIR / (src.stem + ".o")
        cmd = [NVCC, "-O3", "-std=c++17", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC",
               "-I", str(ROOT / "include"), "-I", str(CSRC), "-x", "cu", "-c", str(src),
               "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        objs.append(str(obj))
    cmd = [NVCC, "-shared", *ARCH, "-o", str(LIB_PATH), *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
