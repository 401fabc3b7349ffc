"""Compile the CUDA sources into ``libpermuto_b200.so`` next to this file (sm_100a only).

nvcc cross-compiles without a GPU.  One object per pos_dim is built in parallel, then linked
with the C-ABI translation unit.  Usage: ``python -m permutohedral_encoding_b200.build [--force]``.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libpermuto_b200.so")
DIMS = (2, 3, 4, 5, 6, 7)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc() -> str:
    return os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def _sources():
    names = ["permuto_dim.cu", "permuto_cabi.cu", "permuto_probe.cu", "permuto_adam.cu", "permuto_geometry.cuh",
             "permuto_internal.h"]
    paths = [os.path.join(CSRC, n) for n in names if os.path.isfile(os.path.join(CSRC, n))]
    paths.append(os.path.join(INCLUDE, "permuto_b200.h"))
    return paths


def _stale() -> bool:
    if not os.path.isfile(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in _sources())


def _run(cmd, verbose):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + res.stdout)
    if verbose and res.stdout.strip():
        print(res.stdout)
    return res.stdout


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, defines=(), out: str | None = None) -> str:
    """Build if sources are newer than the library; returns the library path.  ``defines`` adds
    -D macros (tuning experiments) and ``out`` writes the library elsewhere."""
    global OBJ_DIR, LIB_PATH
    if out:
        LIB_PATH = os.path.abspath(out)
        OBJ_DIR = LIB_PATH + ".obj"
        force = True
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"] + ["-I", INCLUDE, "-I", CSRC]
    flags += [f"-D{d}" for d in defines]
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    jobs = []
    for d in DIMS:
        obj = os.path.join(OBJ_DIR, f"permuto_dim{d}.o")
        jobs.append(([_nvcc(), *flags, f"-DPERMUTO_DIM={d}", "-c", os.path.join(CSRC, "permuto_dim.cu"), "-o", obj], obj))
    for name in ("permuto_cabi", "permuto_probe", "permuto_adam"):
        src = os.path.join(CSRC, name + ".cu")
        if os.path.isfile(src):
            obj = os.path.join(OBJ_DIR, name + ".o")
            jobs.append(([_nvcc(), *flags, "-c", src, "-o", obj], obj))
    objs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        futs = {ex.submit(_run, cmd, verbose or ptxas_info): obj for cmd, obj in jobs}
        for fut in cf.as_completed(futs):
            out = fut.result()
            if ptxas_info:
                print(out)
            objs.append(futs[fut])
    _run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *sorted(objs), "-o", LIB_PATH], verbose)
    return LIB_PATH


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills per kernel")
    ap.add_argument("-D", dest="defines", action="append", default=[], help="extra macro, e.g. -D PERMUTO_THREADS=128")
    ap.add_argument("--out", default=None, help="write the library to this path instead")
    args = ap.parse_args()
    print(build(force=args.force, verbose=True, ptxas_info=args.ptxas_info, defines=args.defines, out=args.out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
