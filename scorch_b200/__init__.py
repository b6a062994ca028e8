"""scorch_b200 — B200 (sm_100a) CUDA kernels for the sparse hot path of Scorch (CSR SpMM with
bias/ReLU epilogues, SDDMM, CSR row softmax, SpMV, two-phase SpGEMM) behind the reference's own
operator boundary.

``import scorch_b200 as scorch`` gives ``scorch.matmul`` / ``scorch.einsum`` / ``scorch.STensor``
with the reference's calling conventions; ``scorch_b200.scorch_ops`` is the drop-in for the
reference's ``scorch_ops`` extension module; ``include/scorch_b200.h`` is the C ABI underneath.
Like the reference (src/scorch/__init__.py:14-18) unknown attributes fall through to ``torch``.
"""
from __future__ import annotations

from .stensor import STensor, TensorFormat, TensorIndex, TensorStorage, parse_format
from .ops import add, einsum, elementwise, matmul, spmm_bias_act
from . import scorch_ops

__all__ = ["STensor", "TensorFormat", "TensorIndex", "TensorStorage", "parse_format", "add", "einsum",
           "elementwise", "matmul", "spmm_bias_act", "scorch_ops"]


def __getattr__(name):
    import torch
    return getattr(torch, name)
