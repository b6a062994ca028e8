"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on CPU.

The CPU oracle (``oracle/``) and, when its binary exists, the compiled reference extension
(``oracle/_ref``) are CHECKERS: tests compare the CUDA path against them, never the reverse.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "hotpath_golden.npz")
    data = np.load(path)

    class G:
        def case(self, prefix):
            pre = prefix + "."
            return {k[len(pre):]: data[k] for k in data.files if k.startswith(pre)}

        files = data.files
    return G()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def ref_ops():
    """The reference's own compiled extension, or skip when the binary was not built."""
    from oracle import ref_loader
    mod = ref_loader.load()
    if mod is None:
        pytest.skip("oracle/_ref is not built on this machine")
    return mod


@pytest.fixture(scope="session")
def sb_lib():
    """The C-ABI library; built on demand where nvcc exists (cross-compiles without a GPU)."""
    from scorch_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.lib()
