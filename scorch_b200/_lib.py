"""ctypes binding of ``libscorch_b200.so`` — the C ABI declared in ``include/scorch_b200.h``.

There is no CPU fallback: if the shared library is missing, ``lib()`` raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# SCORCH_B200_LIB points at another build of the same library (e.g. one compiled with different
# tuning macros); by default the in-tree build is loaded.
LIB_PATH = os.environ.get("SCORCH_B200_LIB") or os.path.join(_HERE, "libscorch_b200.so")

SB_OK = 0
SB_F32, SB_F64, SB_I32, SB_I64 = 0, 1, 2, 3
HEAVY_ROW_NNZ = 1024
STATIC_SPMV_MAX_NNZ = 1 << 26

_i64, _int, _ptr, _sz, _f32 = C.c_int64, C.c_int, C.c_void_p, C.c_size_t, C.c_float

# name -> (restype, argtypes); mirrors include/scorch_b200.h declaration by declaration
SIGNATURES = {
    "sb_abi_version": (_int, []),
    "sb_status_string": (C.c_char_p, [_int]),
    "sb_last_error": (C.c_char_p, []),
    "sb_csr_plan_bytes": (_sz, [_i64, _i64]),
    "sb_csr_plan_max_segments": (_i64, [_i64]),
    "sb_csr_plan_build": (_int, [_i64, _i64, _ptr, _ptr, _sz, _ptr]),
    "sb_csr_plan_counts": (_int, [_ptr, C.POINTER(_i64), C.POINTER(_i64), _ptr]),
    "sb_partition_rows_by_nnz": (_int, [_i64, _ptr, _int, _ptr, _ptr]),
    "sb_spmm_csr_scratch_bytes": (_sz, [_i64, _i64, _i64]),
    "sb_spmm_csr_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _int,
                               _ptr, _i64, _i64, _i64, _i64, _i64, _ptr, _i64, _ptr, _sz, _ptr]),
    "sb_spmm_csr_acc_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _int,
                                   _ptr, _i64, _i64, _i64, _i64, _i64, _ptr, _i64, _ptr, _sz, _ptr]),
    "sb_spmm_wide_select": (_int, [_int]),
    "sb_spmm_wide_status": (_int, []),
    "sb_probe_l2_gather": (_int, [_ptr, _i64, _i64, _i64, _ptr, _ptr]),
    "sb_spmm_csr_typed": (_int, [_int, _i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr,
                                 _i64, _ptr]),
    "sb_spmv_csr_scratch_bytes": (_sz, [_i64]),
    "sb_spmv_csr_f32": (_int, [_i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _ptr]),
    "sb_spmv_csr_typed": (_int, [_int, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "sb_spmv_csr_f32_static": (_int, [_i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "sb_sddmm_csr_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64,
                                _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "sb_sddmm_coo_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr, _i64,
                                _ptr, _i64, _i64, _i64, _i64, _ptr]),
    "sb_block_plan_bytes": (_sz, [_i64, _i64]),
    "sb_block_plan_build": (_int, [_i64, _i64, _i64, _ptr, _ptr, _ptr, _sz, C.POINTER(_i64),
                                   C.POINTER(_i64), _ptr]),
    "sb_sddmm_csr_blocked_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr,
                                        _i64, _ptr, _i64, _i64, _i64, _i64, _ptr, _i64, _i64, _ptr]),
    "sb_spmm_csr_blocked_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr,
                                       _int, _ptr, _i64, _i64, _i64, _i64, _i64, _ptr, _i64, _i64,
                                       _ptr]),
    "sb_attn_plan_bytes": (_sz, [_i64, _i64]),
    "sb_attn_plan_build": (_int, [_i64, _i64, _i64, _ptr, _ptr, _ptr, _sz, C.POINTER(_i64),
                                  C.POINTER(_i64), _ptr]),
    "sb_sparse_attention_scratch_bytes": (_sz, [_i64, _i64, _i64]),
    "sb_sparse_attention_csr_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr,
                                           _i64, _ptr, _i64, _f32, _ptr, _i64, _i64, _i64, _i64, _i64,
                                           _i64, _ptr, _i64, _i64, _ptr, _sz, _int, _ptr]),
    "sb_csr_validate_workspace_bytes": (_sz, []),
    "sb_csr_validate": (_int, [_i64, _i64, _i64, _ptr, _ptr, _int, _ptr, _ptr, _sz, _ptr]),
    "sb_attn_band_plan_bytes": (_sz, [_i64, _i64]),
    "sb_attn_band_plan_build": (_int, [_i64, _i64, _i64, _ptr, _ptr, _ptr, _sz, C.POINTER(_i64),
                                       C.POINTER(_i64), _ptr]),
    "sb_sparse_attention_band_f32": (_int, [_i64, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _i64, _ptr,
                                            _i64, _ptr, _i64, _f32, _ptr, _i64, _i64, _i64, _i64, _i64,
                                            _i64, _ptr, _i64, _ptr, _sz, _int, _ptr]),
    "sb_attn_band_probe": (_int, [_i64, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr,
                                  _ptr]),
    "sb_attn_band_status": (_int, []),
    "sb_csr_row_softmax_f32": (_int, [_i64, _i64, _ptr, _ptr, _ptr, _f32, _i64, _i64, _ptr]),
    "sb_spgemm_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "sb_spgemm_symbolic": (_int, [_i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                  C.POINTER(_i64), _ptr, _sz, _ptr]),
    "sb_spgemm_numeric": (_int, [_int, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                                 _ptr, _ptr, _ptr, _sz, _ptr]),
    "sb_csr_ewise_workspace_bytes": (_sz, [_i64]),
    "sb_csr_ewise_symbolic": (_int, [_int, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, C.POINTER(_i64), _ptr, _sz, _ptr]),
    "sb_csr_ewise_numeric": (_int, [_int, _int, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "sb_dense_to_csr_workspace_bytes": (_sz, [_i64]),
    "sb_dense_to_csr_count": (_int, [_i64, _i64, _ptr, _i64, _ptr, C.POINTER(_i64), _ptr, _sz, _ptr]),
    "sb_dense_to_csr_fill": (_int, [_i64, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _ptr]),
    "sb_csr_transpose_workspace_bytes": (_sz, [_i64, _i64]),
    "sb_csr_transpose": (_int, [_int, _i64, _i64, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _ptr]),
    "sb_topk_rows_to_csr_f32": (_int, [_i64, _i64, _i64, _ptr, _i64, _int, _ptr, _ptr, _ptr, _ptr]),
    "sb_csr_sym_normalize_f32": (_int, [_i64, _i64, _ptr, _ptr, _ptr, _ptr]),
    "sb_coo_rows_to_csr_pos": (_int, [_i64, _i64, _ptr, _ptr, _ptr]),
    "sb_csr_pos_to_coo_rows": (_int, [_i64, _i64, _ptr, _ptr, _ptr]),
}

_lib = None


class ScorchB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError via pybind)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"scorch_b200 status {status}: {message}")
        self.status = status


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m scorch_b200.build` "
                "(there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != SB_OK:
        raise ScorchB200Error(status, lib().sb_last_error().decode("utf-8", "replace"))
