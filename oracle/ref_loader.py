"""Load the compiled reference extension from ``oracle/_ref`` (checker only).

TEST INFRASTRUCTURE ONLY: the product never imports this module.  ``load()`` returns the
reference's own ``scorch_ops`` pybind module (bound in the reference at ``csrc/ops.cpp:219-237``)
built by ``oracle/build_ref.py``, or ``None`` when no prebuilt binary is present.
"""
from __future__ import annotations

import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_mod = None
_level = None


def _host_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def pick_level() -> str | None:
    """Widest ISA level both built and supported by this host."""
    flags = _host_flags()
    v3 = {"avx2", "fma", "bmi2", "f16c", "movbe"} <= flags
    v4 = v3 and {"avx512f", "avx512bw", "avx512cd", "avx512dq", "avx512vl"} <= flags
    for lvl, ok in (("x86-64-v4", v4), ("x86-64-v3", v3)):
        if ok and os.path.exists(os.path.join(_HERE, "_ref", lvl, "scorch_ops.so")):
            return lvl
    return None


def load():
    global _mod, _level
    if _mod is not None:
        return _mod
    lvl = pick_level()
    if lvl is None:
        return None
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    path = os.path.join(_HERE, "_ref", lvl, "scorch_ops.so")
    spec = importlib.util.spec_from_file_location("scorch_ops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _mod, _level = mod, lvl
    return mod


def level() -> str | None:
    return _level


def reference_package_dir() -> str | None:
    """Directory to put on sys.path to import the reference's own Python package ``scorch``
    (staged by ``oracle/build_ref.py``), or None when it has not been staged."""
    d = os.path.join(_HERE, "_ref", "pkg", "src")
    return d if os.path.isdir(os.path.join(d, "scorch")) else None
