"""Ahead-of-time build of ``libscorch_b200.so`` (the C-ABI library) with nvcc for sm_100a.

    python -m scorch_b200.build [--force] [--verbose]

The library is built in-tree (``scorch_b200/libscorch_b200.so``); nvcc cross-compiles without a
GPU.  ``-Xptxas -v`` output (registers, spills, shared memory per kernel) is written to
``scorch_b200/csrc/build/ptxas.log``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJDIR = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libscorch_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _host_cxx() -> str:
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJDIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    headers.append(os.path.abspath(__file__))
    nvcc = _nvcc()
    procs, objs = [], []
    for src in sources():
        obj = os.path.join(OBJDIR, src[:-3] + ".o")
        objs.append(obj)
        path = os.path.join(CSRC, src)
        if not force and not _stale(obj, [path] + headers):
            continue
        cmd = [nvcc, *ARCH, "-lineinfo", "-O3", "-std=c++17", "-ccbin", _host_cxx(),
               "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
               f"-I{INCLUDE}", f"-I{CSRC}", "-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        log = open(os.path.join(OBJDIR, src[:-3] + ".ptxas.log"), "w")
        procs.append((src, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), log))
    failed = []
    for src, p, log in procs:
        rc = p.wait()
        log.close()
        if rc != 0:
            failed.append(src)
            sys.stderr.write(open(log.name).read())
    if failed:
        raise RuntimeError(f"nvcc failed for {failed}")
    if procs or force or _stale(LIB, objs):
        cmd = [nvcc, *ARCH, "-shared", "-ccbin", _host_cxx(), "-o", LIB, *objs, "-cudart", "static"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    with open(os.path.join(OBJDIR, "ptxas.log"), "w") as out:
        for src in sources():
            p = os.path.join(OBJDIR, src[:-3] + ".ptxas.log")
            if os.path.exists(p):
                out.write(f"==== {src}\n" + open(p).read())
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
