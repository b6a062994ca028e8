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

The reference's Python package (``src/scorch``, pure Python) is staged beside the binaries as
``oracle/_ref/pkg/src/scorch`` so that tests can run the reference's own ``scorch.matmul`` /
``scorch.einsum`` front end — once over the reference's kernels (the stock CPU path) and once
over this repository's drop-in ``scorch_ops`` module.
Outputs go only into ``oracle/_ref/`` (git-ignored).

The reference checkout is found through ``SCORCH_REFERENCE_ROOT``; without it a directory
named ``reference`` beside this repository is tried.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LEVELS = ("x86-64-v3", "x86-64-v4")


def reference_root() -> str:
    env = os.environ.get("SCORCH_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def stage_python_package(root: str, verbose: bool = True) -> str | None:
    """Copy the reference's pure-Python package (and the C++ headers its JIT path prepends) to
    oracle/_ref/pkg, laid out like the reference project: the package finds its project root by
    walking up to the first directory that holds a ``setup.py``."""
    pkg = os.path.join(root, "src", "scorch")
    if not os.path.isdir(pkg):
        return None
    base = os.path.join(OUT, "pkg")
    dst = os.path.join(base, "src", "scorch")
    newest = max(os.path.getmtime(os.path.join(d, f)) for d, _, fs in os.walk(pkg) for f in fs
                 if f.endswith(".py"))
    stamp = os.path.join(base, ".staged")
    if os.path.exists(stamp) and os.path.getmtime(stamp) >= newest and os.path.isdir(dst):
        return dst
    shutil.rmtree(base, ignore_errors=True)
    shutil.copytree(pkg, dst, ignore=shutil.ignore_patterns("__pycache__", "*.so", "*.pyc"))
    if os.path.isdir(os.path.join(root, "csrc")):
        shutil.copytree(os.path.join(root, "csrc"), os.path.join(base, "csrc"))
    with open(os.path.join(base, "setup.py"), "w") as f:
        f.write("# marks the project root for the staged package (it walks up to a setup.py)\n")
    open(stamp, "w").close()
    if verbose:
        print(f"[oracle/_ref] staged the reference's Python package at {dst}")
    return dst


def build(force: bool = False, verbose: bool = True) -> list[str]:
    src = os.path.join(reference_root(), "csrc", "ops.cpp")
    if not os.path.exists(src):
        if verbose:
            print(f"[oracle/_ref] reference source not found at {src}: keeping prebuilt files")
        return []
    stage_python_package(reference_root(), verbose)
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
