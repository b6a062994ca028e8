"""Drop-in for the reference's ``scorch_ops`` extension module (reference: csrc/ops.cpp:91-237).

Same function names, argument order, keyword names and result shape as the pybind module the
reference builds, so ``scorch.prebuilt_kernels`` / ``scorch.ops`` / ``scorch.trace`` can look the
symbols up by name (reference: src/scorch/prebuilt_kernels.py:96-101, src/scorch/ops.py:405-415,
src/scorch/trace.py:269-299) and run them on a B200 instead of the OpenMP kernels.

Argument encoding is the reference's (src/scorch/prebuilt_kernels.py:211-218):
``*_shape`` sequences of ints, ``*_mode_indices`` a list per storage level of lists of int32
tensors, ``*_values`` a 1-D tensor.  Tensors may live on the host (like the reference's) or on
the GPU.  Host tensors are copied to the current CUDA device, the kernel runs there, and the
result comes back as a host tensor; CUDA tensors are used in place and the result stays on the
device.  There is no CPU compute path: without a CUDA device every call raises.

Results are ``Tensor`` objects exposing ``.storage.value`` and ``.storage.index.mode_indices``
(reference: csrc/header.h:4-16, bound at csrc/ops.cpp:227-236).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import kernels as K


class TensorIndex:
    def __init__(self, mode_indices=None):
        self.mode_indices = [] if mode_indices is None else mode_indices


class TensorStorage:
    def __init__(self, value=None, index=None):
        self.value = value
        self.index = index if index is not None else TensorIndex()


class Tensor:
    def __init__(self, value=None, mode_indices=None, shape=None):
        self.storage = TensorStorage(value, TensorIndex(mode_indices))
        self.shape = list(shape) if shape is not None else []


# ---- host <-> device plumbing ------------------------------------------------------------------
def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("scorch_b200 needs a CUDA device: the kernels have no CPU fallback")
    return torch.device("cuda", torch.cuda.current_device())


def _up(t: torch.Tensor, dtype=None) -> torch.Tensor:
    """Tensor on the GPU (copied when it lives on the host), contiguous, optionally cast."""
    if not t.is_cuda:
        t = t.to(_device(), non_blocking=True)
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _down(t: torch.Tensor, to_host: bool) -> torch.Tensor:
    if not to_host:
        return t
    out = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
    out.copy_(t, non_blocking=True)
    torch.cuda.current_stream().synchronize()
    return out


def _on_host(*tensors) -> bool:
    return not any(isinstance(t, torch.Tensor) and t.is_cuda for t in tensors)


def _csr(mode_indices):
    return _up(mode_indices[1][0], torch.int32), _up(mode_indices[1][1], torch.int32)


# ---- SpMM ----------------------------------------------------------------------------------------
def _spmm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values,
          bias=None, relu=False):
    host = _on_host(A_values, B_values)
    pos, crd = _csr(A_mode_indices)
    n, k = int(B_shape[0]), int(B_shape[1])
    B = _up(B_values).view(n, k)
    val = _up(A_values)
    if val.dtype != B.dtype:
        raise RuntimeError(f"expected scalar type {val.dtype} but found {B.dtype}")
    b = None if bias is None else _up(bias)
    if val.dtype == torch.float32:
        C = K.spmm_csr(pos, crd, val, B, bias=b, relu=relu, n=n)
    else:
        if bias is not None:
            raise RuntimeError("fused bias/ReLU SpMM is float32 only")
        C = K.spmm_csr(pos, crd, val, B, n=n)
    return Tensor(_down(C.view(-1), host), [[], []], result_shape)


def spmm_csr_float_v2(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices,
                      B_values, tile_size: int = 256):
    """Reference: spmm_csr_float_v2, csrc/spmm.h:2007-2089 (``tile_size`` is a CPU cache-tiling
    knob with no effect on results; accepted and ignored)."""
    return _spmm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values)


def _spmm_variant(default_tile: Optional[int]):
    if default_tile is None:
        def fn(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values):
            return _spmm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices,
                         B_values)
    else:
        def fn(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values,
               tile_size: int = default_tile):
            return _spmm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices,
                         B_values)
    return fn


# typed family and legacy aliases (reference: csrc/ops.cpp:91-116)
prebuilt_spmm_csr_f32 = _spmm_variant(32)
prebuilt_spmm_csr_f64 = _spmm_variant(32)
prebuilt_spmm_csr_i32 = _spmm_variant(32)
prebuilt_spmm_csr_i64 = _spmm_variant(32)
spmm_csr_float = _spmm_variant(32)
spmm_csr_double = _spmm_variant(32)
# experimental CPU variants of the same product (reference: csrc/ops.cpp:118-165); one GPU kernel
# family stands behind all of them
spmm_csr_float_optimized = _spmm_variant(128)
spmm_csr_float_turbo = _spmm_variant(128)
spmm_csr_float_ultra = _spmm_variant(256)
spmm_csr_float_apex = _spmm_variant(256)
spmm_csr_float_untiled = _spmm_variant(None)
spmm_csr_float_direct = _spmm_variant(None)
spmm_csr_float_neon = _spmm_variant(None)
spmm_csr_float_row_panel = _spmm_variant(None)
spmm_csr_float_k_parallel = _spmm_variant(None)
spmm_csr_float_sorted_rows = _spmm_variant(None)
spmm_csr_float_neon2 = _spmm_variant(None)
spmm_csr_float_neon4 = _spmm_variant(None)
spmm_csr_float_tiled_neon = _spmm_variant(None)


def spmm_csr_float_tiled_i_k(result_shape, A_shape, A_mode_indices, A_values, B_shape,
                             B_mode_indices, B_values, i_tile_size: int = 16, k_tile_size: int = 32):
    return _spmm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values)


def spmm_csr_bias_relu_float(result_shape, A_shape, A_mode_indices, A_values, B_shape,
                             B_mode_indices, B_values, bias):
    """Reference: spmm_csr_bias_act<float, true>, csrc/spmm.h:28-89."""
    return _spmm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values,
                 bias=bias, relu=True)


def spmm_csr_bias_float(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices,
                        B_values, bias):
    """Reference: spmm_csr_bias_act<float, false>, csrc/spmm.h:28-89."""
    return _spmm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values,
                 bias=bias, relu=False)


def spmm_coo_float(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices,
                   B_values):
    """COO A (rows ascending) x dense B.  Reference: spmm_coo_float, csrc/spmm.h:247-373.  The row
    pointers are built on the device and the CSR kernel does the product."""
    host = _on_host(A_values, B_values)
    row = _up(A_mode_indices[0][0], torch.int32)
    col = _up(A_mode_indices[1][0], torch.int32)
    pos = K.coo_rows_to_csr_pos(row, int(A_shape[0]))
    n, k = int(B_shape[0]), int(B_shape[1])
    C = K.spmm_csr(pos, col, _up(A_values, torch.float32), _up(B_values, torch.float32).view(n, k), n=n)
    return Tensor(_down(C.view(-1), host), [[], []], result_shape)


# ---- SpMV ----------------------------------------------------------------------------------------
def _spmv(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values):
    """Reference: spmv_csr<T>, csrc/kernels.h:12-49."""
    host = _on_host(A_values, B_values)
    pos, crd = _csr(A_mode_indices)
    val, x = _up(A_values), _up(B_values)
    if val.dtype != x.dtype:
        raise RuntimeError(f"expected scalar type {val.dtype} but found {x.dtype}")
    y = K.spmv_csr(pos, crd, val, x)
    return Tensor(_down(y, host), [[]], result_shape)


prebuilt_spmv_csr_f32 = _spmv
prebuilt_spmv_csr_f64 = _spmv
prebuilt_spmv_csr_i32 = _spmv
prebuilt_spmv_csr_i64 = _spmv


# ---- SpGEMM --------------------------------------------------------------------------------------
def _spmspm(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices, B_values):
    """Reference: spmspm_csr<T>, csrc/kernels.h:51-202."""
    host = _on_host(A_values, B_values)
    Apos, Acrd = _csr(A_mode_indices)
    Bpos, Bcrd = _csr(B_mode_indices)
    Aval, Bval = _up(A_values), _up(B_values)
    if Aval.dtype != Bval.dtype:
        raise RuntimeError(f"expected scalar type {Aval.dtype} but found {Bval.dtype}")
    n = int(result_shape[1]) if len(result_shape) > 1 else int(B_shape[0])
    Cpos, Ccrd, Cval = K.spgemm_csr(Apos, Acrd, Aval, Bpos, Bcrd, Bval, n)
    return Tensor(_down(Cval, host), [[], [_down(Cpos, host), _down(Ccrd, host)]], result_shape)


prebuilt_spmspm_csr_f32 = _spmspm
prebuilt_spmspm_csr_f64 = _spmspm
prebuilt_spmspm_csr_i32 = _spmspm
prebuilt_spmspm_csr_i64 = _spmspm
spmspm_csr_float = _spmspm


def spmspm_coo_float(result_shape, A_shape, A_mode_indices, A_values, B_shape, B_mode_indices,
                     B_values):
    """COO x COO (both sorted by row, then column) -> COO with rows ascending and columns ascending
    within a row.  Reference: spmspm_coo_float_opt, csrc/kernels.h:397-501."""
    host = _on_host(A_values, B_values)
    Apos = K.coo_rows_to_csr_pos(_up(A_mode_indices[0][0], torch.int32), int(A_shape[0]))
    Bpos = K.coo_rows_to_csr_pos(_up(B_mode_indices[0][0], torch.int32), int(B_shape[0]))
    Acrd, Bcrd = _up(A_mode_indices[1][0], torch.int32), _up(B_mode_indices[1][0], torch.int32)
    Cpos, Ccrd, Cval = K.spgemm_csr(Apos, Acrd, _up(A_values, torch.float32), Bpos, Bcrd,
                                    _up(B_values, torch.float32), int(result_shape[1]))
    Crow = K.csr_pos_to_coo_rows(Cpos, Ccrd.numel())
    return Tensor(_down(Cval, host), [[_down(Crow, host)], [_down(Ccrd, host)]], result_shape)


# ---- SDDMM ---------------------------------------------------------------------------------------
def sddmm_coo_float_prebuilt(result_shape, S_shape, S_mode_indices, S_values, A_shape,
                             A_mode_indices, A_values, B_shape, B_mode_indices, B_values):
    """Reference: sddmm_coo_float_prebuilt, csrc/kernels.h:508-570.  Like the reference, the
    result shares the mask's coordinate tensors (csrc/kernels.h:567)."""
    host = _on_host(S_values, A_values, B_values)
    row = _up(S_mode_indices[0][0], torch.int32)
    col = _up(S_mode_indices[1][0], torch.int32)
    d = int(A_shape[1])
    Q = _up(A_values, torch.float32).view(int(A_shape[0]), d)
    Kt = _up(B_values, torch.float32).view(int(B_shape[0]), d)
    out = K.sddmm_coo(row, col, _up(S_values, torch.float32), Q, Kt)
    return Tensor(_down(out, host), S_mode_indices, result_shape)


def sddmm_csr_float(result_shape, S_shape, S_mode_indices, S_values, A_shape, A_mode_indices,
                    A_values, B_shape, B_mode_indices, B_values):
    """SDDMM with a CSR mask — what the reference reaches through its compiler for
    ``einsum("ij,ik,jk->ij", mask_csr, Q, K)`` (generator: src/scorch/ops.py:638-664); not a
    symbol of the reference's module.  Output format "o,o": fresh int32 (row, col) arrays and the
    values in mask order."""
    host = _on_host(S_values, A_values, B_values)
    pos, crd = _csr(S_mode_indices)
    d = int(A_shape[1])
    Q = _up(A_values, torch.float32).view(int(A_shape[0]), d)
    Kt = _up(B_values, torch.float32).view(int(B_shape[0]), d)
    out, row, col = K.sddmm_csr(pos, crd, _up(S_values, torch.float32), Q, Kt, want_coords=True)
    return Tensor(_down(out, host), [[_down(row, host)], [_down(col, host)]], result_shape)


def csr_row_softmax_float(pos, values, scale: float = 1.0):
    """Row softmax over CSR values (reference: bench/bench_sparse_transformer.py:277-297, caller
    side); not a symbol of the reference's module."""
    host = _on_host(values)
    return _down(K.csr_row_softmax(_up(pos, torch.int32), _up(values, torch.float32), scale), host)


REFERENCE_SYMBOLS = (
    "prebuilt_spmm_csr_f32", "prebuilt_spmm_csr_f64", "prebuilt_spmm_csr_i32", "prebuilt_spmm_csr_i64",
    "prebuilt_spmspm_csr_f32", "prebuilt_spmspm_csr_f64", "prebuilt_spmspm_csr_i32",
    "prebuilt_spmspm_csr_i64", "prebuilt_spmv_csr_f32", "prebuilt_spmv_csr_f64",
    "prebuilt_spmv_csr_i32", "prebuilt_spmv_csr_i64", "spmm_csr_float", "spmm_csr_double",
    "spmspm_csr_float", "spmm_csr_float_tiled_i_k", "spmm_csr_float_optimized",
    "spmm_csr_float_turbo", "spmm_csr_float_ultra", "spmm_csr_float_apex", "spmm_csr_float_untiled",
    "spmm_coo_float", "spmspm_coo_float", "spmm_csr_float_direct", "spmm_csr_float_neon",
    "spmm_csr_float_row_panel", "spmm_csr_float_k_parallel", "spmm_csr_float_sorted_rows",
    "spmm_csr_float_neon2", "spmm_csr_float_neon4", "spmm_csr_float_tiled_neon", "spmm_csr_float_v2",
    "spmm_csr_bias_relu_float", "spmm_csr_bias_float", "sddmm_coo_float_prebuilt",
    "Tensor", "TensorStorage", "TensorIndex",
)
