"""Compile the REFERENCE's own CUDA extension, unmodified, for sm_100a.  TEST INFRASTRUCTURE ONLY.

Sources are compiled where they lie in a checkout of geodesia-ai/geodesia-kv
(``geodesia_kv_cuda/binding.cpp`` and ``geodesia_kv_cuda/mixed_attn.cu``); nothing is copied
into this repository and the output goes to ``oracle/_ref/`` (git-ignored).  The result is a
torch extension module ``geodesia_kv_ref_ext`` exposing the reference's ``mixed_attn_decode``;
the GPU tests use it as a second oracle and the benchmark's CPU-baseline leg times it beside
the CPU port.  Flags are the reference's own (geodesia_kv/cuda_ext.py:77) plus the sm_100a target.

    python oracle/build_ref.py [--reference /path/to/checkout]      (default: $GEODESIA_REFERENCE)
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NAME = "geodesia_kv_ref_ext"


def reference_checkout() -> Path | None:
    """Where the reference's sources are: $GEODESIA_REFERENCE, else a directory named ``reference``
    beside this repository; None when neither holds the CUDA sources."""
    cands = [os.environ.get("GEODESIA_REFERENCE"), HERE.parent.parent / "reference"]
    for c in cands:
        if c and (Path(c) / "geodesia_kv_cuda" / "mixed_attn.cu").exists():
            return Path(c)
    return None


def build(reference: Path, force: bool = False) -> Path | None:
    src = reference / "geodesia_kv_cuda"
    if not (src / "mixed_attn.cu").exists():
        return None
    so = OUT / f"{NAME}.so"
    if so.exists() and not force:
        return so
    import torch
    from torch.utils import cpp_extension as ce
    OUT.mkdir(exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    common = ["-O3", "-std=c++17", f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    objs = []
    jobs = [
        (["g++", "-fPIC", "-c", str(src / "binding.cpp"), "-o", str(OUT / "binding.o")] + common + inc, OUT / "binding.o"),
        (["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "--use_fast_math", "-lineinfo", "-Xcompiler", "-fPIC",
          "-c", str(src / "mixed_attn.cu"), "-o", str(OUT / "mixed_attn.o")] + common + inc, OUT / "mixed_attn.o"),
    ]
    procs = [(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True), obj) for cmd, obj in jobs]
    for p, obj in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"compiling {obj.name} failed:\n{out[-4000:]}")
        objs.append(str(obj))
    libdir = Path(torch.__file__).parent / "lib"
    link = ["g++", "-shared", "-o", str(so), *objs, f"-L{libdir}", "-L/usr/local/cuda/lib64", "-lc10", "-lc10_cuda",
            "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart", f"-Wl,-rpath,{libdir}"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stderr[-4000:])
    for o in objs:
        Path(o).unlink()
    return so


def load():
    """Import the built module, or return None when it has not been built."""
    so = OUT / f"{NAME}.so"
    if not so.exists():
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    where = Path(a.reference) if a.reference else reference_checkout()
    if where is None:
        raise SystemExit("no checkout of the reference: pass --reference or set GEODESIA_REFERENCE")
    print(build(where, a.force))
