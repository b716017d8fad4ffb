"""In-tree build of the CUDA library (sm_100a only).

``python -m geodesia_kv_b200.build`` compiles ``csrc/*.cu`` with nvcc into
``geodesia_kv_b200/libgeodesia_kv_b200.so``.  The library exposes only the C ABI
declared in ``include/geodesia_kv_b200.h`` and links nothing but the CUDA
runtime, so a build takes seconds and needs no GPU.  Fast-math is never used:
the packer and the allocator must reproduce the reference's IEEE arithmetic.
"""
from __future__ import annotations

import hashlib
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


def source_hash(defines: tuple = ()) -> str:
    """Digest of everything the library is compiled from (file contents, not time stamps: a copied
    tree keeps its library valid whatever order its files were written in)."""
    h = hashlib.sha256(repr(sorted(defines)).encode())
    deps = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "geodesia_kv_b200.h"]
    for d in deps:
        h.update(d.name.encode())
        h.update(d.read_bytes())
    return h.hexdigest()


def _stamp(out: Path) -> Path:
    return out.with_name(out.name + ".hash")


def is_stale(out: Path = LIB, defines: tuple = ()) -> bool:
    stamp = _stamp(out)
    return not out.exists() or not stamp.exists() or stamp.read_text().strip() != source_hash(defines)


# A second build of the same sources for ONE test: every wait of the decode kernel gives up after a
# few milliseconds instead of a second, and the producer withholds the bytes of one block, so that the
# kernel's give-up path (status word, NaN output) can be exercised without ever hanging a GPU.
WAIT_TEST_LIB = PKG / "libgeodesia_kv_b200_waittest.so"
WAIT_TEST_DEFINES = ("GKV_WAIT_LIMIT_NS=3000000ull", "GKV_TEST_WITHHOLD_BLOCK=1", "GKV_FAST_BUILD=1")   # D = 128, g = 32 only


def build(force: bool = False, verbose: bool = False, defines: tuple = (), out: Path = LIB) -> Path:
    if not force and not is_stale(out, defines):
        return out
    cmd = [nvcc_path(), *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-O3", "-shared",
           "-Xptxas", "-v" if verbose else "-O3", *[f"-D{d}" for d in defines], "-o", str(out), *map(str, sources())]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    _stamp(out).write_text(source_hash(defines) + "\n")
    if verbose:
        print(res.stderr)
    return out


def build_wait_test(force: bool = False) -> Path:
    return build(force=force, defines=WAIT_TEST_DEFINES, out=WAIT_TEST_LIB)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--wait-test" in sys.argv:
        print(build_wait_test(force="--force" in sys.argv))
