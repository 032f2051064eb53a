"""Builds `libtlm_b200.so` in-tree from `csrc/*.cu` with nvcc for sm_100a.

    python -m train_large_model_from_scratch_b200.build_ext [--force] [--verbose]

Each source is compiled to an object under `build/` (in parallel, skipped when
the object is newer than the source and the headers) and the objects are
linked into one shared library next to the package. The kernels expose a C ABI
(see `ops/native.py`), so no Python or torch headers are involved and the
cross-compile needs no GPU.
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "libtlm_b200.so")
OBJ_DIR = os.path.join(os.path.dirname(PKG), "build", "tlm_b200")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources(exclude: tuple[str, ...] = ()) -> list[str]:
    return [s for s in sorted(glob.glob(os.path.join(SRC, "*.cu"))) if os.path.basename(s) not in exclude]


def _stale(obj: str, src: str, headers: list[str]) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(f) > t for f in [src] + headers)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = glob.glob(os.path.join(SRC, "*.cuh")) + glob.glob(os.path.join(SRC, "*.h"))
    srcs = sources()
    objs = [os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o") for s in srcs]
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(pair):
        src, obj = pair
        if not force and not ptxas_info and not _stale(obj, src, headers):
            return None
        cmd = [_nvcc()] + flags + ["-I", SRC, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        logs = list(ex.map(compile_one, zip(srcs, objs)))
    if verbose or ptxas_info:
        for s, log in zip(srcs, logs):
            if log:
                print(f"== {os.path.basename(s)}\n{log}")
    if force or any(l is not None for l in logs) or not os.path.exists(OUT):
        cmd = [_nvcc(), "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.ptxas))
