"""Build the UNMODIFIED reference CUDA extension for sm_100 into ``oracle/_ref/``.

Test infrastructure only: nothing in the product package imports this file or its output.

The reference (RaduAlexandru/permutohedral_encoding) has no CPU path, so the strongest
parity check is its own extension rebuilt for Blackwell and run beside the new kernels on
the same seeded inputs.  Its shipped ``setup.py`` cannot produce that build (it clamps the
architecture to compute capability 90 and forces ``-std=c++14``, which the installed torch
headers reject), so this recipe compiles the two reference translation units where they lie
(``src/Encoding.cu`` and ``src/PyBridge.cxx``) with the flags the reference uses otherwise
(``--extended-lambda --expt-relaxed-constexpr --generate-line-info``, default ``-fmad``) and
links them into one pybind11 module named ``permuto_ref_C``.  No reference source is copied:
the only outputs are object files and the shared library under ``oracle/_ref/``.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MODULE = "permuto_ref_C"


def _torch_paths():
    import torch  # noqa: F401
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    lib = ce.library_paths("cuda")
    return inc, lib


def so_path() -> str:
    return os.path.join(OUT_DIR, MODULE + ".so")


def build(reference: str, force: bool = False, verbose: bool = True) -> str | None:
    """Compile and link; returns the path of the module or None if the sources are absent."""
    src_cu = os.path.join(reference, "src", "Encoding.cu")
    src_cx = os.path.join(reference, "src", "PyBridge.cxx")
    if not (os.path.isfile(src_cu) and os.path.isfile(src_cx)):
        return so_path() if os.path.isfile(so_path()) else None
    out = so_path()
    if os.path.isfile(out) and not force:
        newest = max(os.path.getmtime(src_cu), os.path.getmtime(src_cx))
        if os.path.getmtime(out) >= newest:
            return out
    os.makedirs(OUT_DIR, exist_ok=True)
    inc, lib = _torch_paths()
    incs = [f"-I{os.path.join(reference, 'include')}", f"-I{os.path.join(reference, 'kernels')}"]
    incs += [f"-I{p}" for p in inc]
    defs = [f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=1"]
    obj_cu = os.path.join(OUT_DIR, "Encoding.o")
    obj_cx = os.path.join(OUT_DIR, "PyBridge.o")
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmds = [
        [nvcc, "-std=c++17", "--extended-lambda", "--expt-relaxed-constexpr",
         "--generate-line-info", "-O3", "-Xcompiler", "-fPIC",
         "-gencode=arch=compute_100,code=sm_100", *defs, *incs, "-c", src_cu, "-o", obj_cu],
        ["g++", "-std=c++17", "-O3", "-fPIC", *defs, *incs, "-c", src_cx, "-o", obj_cx],
        ["g++", "-shared", obj_cu, obj_cx, "-o", out,
         *[f"-L{p}" for p in lib], *[f"-Wl,-rpath,{p}" for p in lib],
         "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
         "-lcudart"],
    ]
    for cmd in cmds:
        t0 = time.time()
        if verbose:
            print("[build_ref]", " ".join(cmd[:4]), "...", flush=True)
        subprocess.run(cmd, check=True)
        if verbose:
            print(f"[build_ref]   done in {time.time() - t0:.0f} s", flush=True)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("PERMUTO_REFERENCE_DIR", "/root/reference"))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    out = build(args.reference, args.force)
    if out is None:
        print("[build_ref] reference sources not found and no prebuilt module present")
        return 1
    print("[build_ref] module:", out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
