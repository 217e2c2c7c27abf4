"""Builds the native library in-tree: ``mintccl_b200/_C/libmintccl_b200.so``.

Every ``.cu`` / ``.cpp`` under ``csrc/`` is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into one shared object with a C interface
(``csrc/mintccl.h``) that ``mintccl_b200._native`` loads with ctypes.  nvcc cross-compiles, so the build
needs no GPU.  Usage: ``python -m mintccl_b200.build [--force] [--verbose]``.

The reference has no build step at all (README.md:38 "no custom build or bindings"): its device code
is PTX text inside Triton kernels compiled at run time.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT_DIR = ROOT / "_C"
OBJ_DIR = OUT_DIR / "obj"
LIB = OUT_DIR / "libmintccl_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=default", "-cudart", "static"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[Path]:
    out = []
    for sub in ("host", "kernels", "sim"):
        for ext in ("*.cu", "*.cpp"):
            out += sorted((CSRC / sub).glob(ext))
    return out


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".hpp"):
            h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(src: Path, verbose: bool, extra: list[str]) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".stamp")
    key = hashlib.sha256(src.read_bytes() + _headers_digest().encode() + " ".join(extra).encode()).hexdigest()
    if obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj
    if src.suffix == ".cu":
        cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *CXX_FLAGS, "-I", str(CSRC), "-I", "/usr/local/cuda/include", "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src.name} failed:\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)
    stamp.write_text(key)
    return obj


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for p in OBJ_DIR.glob("*"):
            p.unlink()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose or ptxas_info, extra), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if LIB.exists() and LIB.stat().st_mtime >= newest and not force:
        return LIB
    cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-cudart", "static", "-Xcompiler", "-fPIC", "-o", str(LIB),
           *[str(o) for o in objs], "-lpthread", "-ldl", "-lrt"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="pass -Xptxas -v (registers, spills, shared memory)")
    a = ap.parse_args()
    lib = build(a.force, a.verbose, a.ptxas_info)
    print(lib)


if __name__ == "__main__":
    sys.exit(main())
