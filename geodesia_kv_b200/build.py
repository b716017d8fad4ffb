"""In-tree build of the CUDA library (sm_100a only).

``python -m geodesia_kv_b200.build`` compiles ``csrc/*.cu`` with nvcc into
``geodesia_kv_b200/libgeodesia_kv_b200.so``.  The library exposes only the C ABI
declared in ``include/geodesia_kv_b200.h`` and links nothing but the CUDA
runtime, so a build takes seconds and needs no GPU.  Fast-math is never used:
the packer and the allocator must reproduce the reference's IEEE arithmetic.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libgeodesia_kv_b200.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return str(Path(cand) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: set CUDA_HOME")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "geodesia_kv_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines: tuple = (), out: Path = LIB) -> Path:
    if not force and not is_stale() and out == LIB:
        return LIB
    cmd = [nvcc_path(), *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-O3", "-shared",
           "-Xptxas", "-v" if verbose else "-O3", *[f"-D{d}" for d in defines], "-o", str(out), *map(str, sources())]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
