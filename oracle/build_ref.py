"""Compile the reference's own prebuilt-kernel extension (`scorch_ops`) for use as a checker.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product path; only the
test-suite, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may load it.

The reference ships one translation unit for this path (``csrc/ops.cpp``, which includes
``csrc/spmm.h`` and ``csrc/kernels.h``; built by ``setup.py:57-66`` of the reference as a torch
C++ extension with ``-O3 -march=native -ffast-math -funroll-loops -fopenmp``).  This recipe
runs ``g++`` on that file where it lies (no source is copied) with the same flags, except
that ``-march=native`` is replaced by two portable levels, because the binary is built on one
machine and run on another:

* ``x86-64-v3``  (AVX2 + FMA)      -> ``oracle/_ref/x86-64-v3/scorch_ops.so``
* ``x86-64-v4``  (AVX-512 F/BW/..) -> ``oracle/_ref/x86-64-v4/scorch_ops.so``

``oracle/ref_loader.py`` picks the widest level the running host supports.
Outputs go only into ``oracle/_ref/`` (git-ignored).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LEVELS = ("x86-64-v3", "x86-64-v4")


def reference_root() -> str:
    return os.environ.get("SCORCH_REFERENCE_ROOT", "/root/reference")


def build(force: bool = False, verbose: bool = True) -> list[str]:
    src = os.path.join(reference_root(), "csrc", "ops.cpp")
    if not os.path.exists(src):
        if verbose:
            print(f"[oracle/_ref] reference source not found at {src}: keeping prebuilt files")
        return []
    import torch
    from torch.utils import cpp_extension as cx
    import pybind11

    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = cx.include_paths() + [sysconfig.get_paths()["include"], pybind11.get_include()]
    gomp = glob.glob(os.path.join(tlib, "libgomp*.so*"))
    built = []
    procs = []
    for lvl in LEVELS:
        d = os.path.join(OUT, lvl)
        os.makedirs(d, exist_ok=True)
        so = os.path.join(d, "scorch_ops.so")
        if not force and os.path.exists(so) and os.path.getmtime(so) >= os.path.getmtime(src):
            built.append(so)
            continue
        cmd = ["g++", "-shared", "-fPIC", "-std=c++17", "-O3", f"-march={lvl}", "-ffast-math",
               "-funroll-loops", "-fopenmp", "-w",
               "-DTORCH_EXTENSION_NAME=scorch_ops", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
        cmd += [f"-I{p}" for p in inc]
        cmd += [src, "-o", so, f"-L{tlib}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python",
                f"-Wl,-rpath,{tlib}"]
        cmd += [gomp[0]] if gomp else ["-fopenmp"]
        if verbose:
            print("[oracle/_ref]", " ".join(cmd))
        procs.append((so, subprocess.Popen(cmd)))
    for so, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"building {so} failed")
        built.append(so)
    return built


if __name__ == "__main__":
    build(force="--force" in sys.argv)
