"""The C-ABI library loads and exports every symbol include/scorch_b200.h declares; host-side
argument validation returns error codes (no GPU work is launched here)."""
from __future__ import annotations

import ctypes as C
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "scorch_b200.h")).read()
    return sorted(set(re.findall(r"SB_API\s+[\w\s\*]+?\b(sb_\w+)\s*\(", text)))


def test_header_symbols_all_exported_and_bound(sb_lib):
    from scorch_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(sb_lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_version_and_status_strings(sb_lib):
    assert sb_lib.sb_abi_version() == 1
    assert sb_lib.sb_status_string(0) == b"ok"
    assert b"overflow" in sb_lib.sb_status_string(3)


def test_size_queries_are_pure_host_functions(sb_lib):
    from scorch_b200._lib import HEAVY_ROW_NNZ
    assert sb_lib.sb_csr_plan_bytes(10, 0) >= 32
    nnz = 10 * HEAVY_ROW_NNZ
    assert sb_lib.sb_csr_plan_max_segments(nnz) >= 10
    # segment sums (k floats) + arrival counters (one per 16 columns) per segment and batch item
    assert sb_lib.sb_spmm_csr_scratch_bytes(7, 64, 2) == 7 * 2 * (64 * 4 + 4 * 4)
    assert sb_lib.sb_spmm_csr_scratch_bytes(0, 64, 1) == 0
    assert sb_lib.sb_spmv_csr_scratch_bytes(0) == 0
    assert sb_lib.sb_spmv_csr_scratch_bytes(5000) == 3 * 256  # 3 tiles -> three padded arrays
    small = sb_lib.sb_spgemm_workspace_bytes(100, 100, 0)
    big = sb_lib.sb_spgemm_workspace_bytes(100, 1 << 20, 0)
    assert 0 < small < big
    # the dense-row area is capped, so a huge column count cannot ask for unbounded memory
    assert sb_lib.sb_spgemm_workspace_bytes(1000, 1 << 30, 1) < (20 << 30)


def test_argument_validation_returns_codes_without_launching(sb_lib):
    from scorch_b200._lib import ScorchB200Error, check
    import pytest
    one = C.c_void_p(16)  # never dereferenced: validation fails first
    rc = sb_lib.sb_spmm_csr_f32(-1, 4, 4, 0, one, one, one, one, 4, None, 0, one, 4, 1, 0, 0, 0,
                                None, 0, None, 0, None)
    assert rc == 1 and b"negative" in sb_lib.sb_last_error()
    rc = sb_lib.sb_spmm_csr_f32(4, 4, 8, 0, one, one, one, one, 4, None, 0, one, 8, 1, 0, 0, 0,
                                None, 0, None, 0, None)
    assert rc == 1 and b"leading dimension" in sb_lib.sb_last_error()
    # nnz beyond int32: the reference would wrap (csrc/kernels.h:520); here it is an error code
    rc = sb_lib.sb_sddmm_coo_f32(4, 4, 4, 1 << 31, one, one, None, one, 4, one, 4, one, 1, 0, 0, 0, None)
    assert rc == 3
    # entry counts within a tile of 2^31: the kernels' int tile bounds would overflow
    rc = sb_lib.sb_spmv_csr_f32(4, 4, (1 << 31) - 100, one, one, one, one, one, one, 1 << 40, None)
    assert rc == 3 and b"int32" in sb_lib.sb_last_error()
    rc = sb_lib.sb_sddmm_csr_f32(4, 4, 4, (1 << 31) - 100, one, one, None, one, 4, one, 4, one, None, None,
                                 1, 0, 0, 0, None)
    assert rc == 3
    # the scalar SpMM path (here: float64) has a column limit from the launch grid
    rc = sb_lib.sb_spmm_csr_typed(1, 4, 4, 65536 * 32, 4, one, one, one, one, 65536 * 32, one, 65536 * 32, None)
    assert rc == 5 and b"scalar path" in sb_lib.sb_last_error()
    rc = sb_lib.sb_spmv_csr_typed(9, 4, 4, 0, one, one, one, one, one, None)
    assert rc == 5 or rc == 1
    rc = sb_lib.sb_csr_plan_build(4, 4, one, one, 8, None)
    assert rc == 4 and b"needs" in sb_lib.sb_last_error()
    with pytest.raises(ScorchB200Error) as e:
        check(sb_lib.sb_spgemm_symbolic(4, 4, 4, one, one, one, one, one, C.pointer(C.c_int64(0)),
                                        one, 16, None))
    assert e.value.status == 4


def test_argument_validation_of_the_attention_and_validation_entry_points(sb_lib):
    one = C.c_void_p(32)  # never dereferenced: validation fails first
    # band attention: head dimension 64 only, row pitch >= d, batch within the launch grid
    common = lambda d, ld, batch: sb_lib.sb_sparse_attention_band_f32(
        128, 128, d, 10, one, one, None, one, ld, one, ld, one, ld, 1.0, one, ld, batch, 0, 0, 0, 0,
        one, 0, one, 1 << 20, 3, None)
    assert common(32, 32, 1) == 1 and b"head dimension must be 64" in sb_lib.sb_last_error()
    assert common(64, 32, 1) == 1 and b"row pitch" in sb_lib.sb_last_error()
    assert common(64, 64, 70000) == 1 and b"batch" in sb_lib.sb_last_error()
    rc = sb_lib.sb_sparse_attention_band_f32(128, 128, 64, 10, one, one, None, one, 64, one, 64, one, 64, 1.0,
                                             one, 64, 1, 0, 0, 0, 0, one, 0, one, 1 << 20, 0, None)
    assert rc == 1 and b"stage" in sb_lib.sb_last_error()
    # an empty mask is nothing to do, whatever the pointers
    assert sb_lib.sb_sparse_attention_band_f32(0, 128, 64, 0, None, None, None, None, 64, None, 64, None, 64, 1.0,
                                               None, 64, 1, 0, 0, 0, 0, None, 0, None, 0, 3, None) == 0
    rc = sb_lib.sb_attn_band_plan_build(4, 4, 4, one, one, one, 8, None, None, None)
    assert rc == 4 and b"needs" in sb_lib.sb_last_error()
    assert sb_lib.sb_attn_band_plan_bytes(4096, 1 << 20) > (2 << 20) * 4
    rc = sb_lib.sb_attn_band_probe(128, 384, 64, 5, one, 64, one, 64, one, 64, one, None, None, None)
    assert rc == 1 and b"tile out of range" in sb_lib.sb_last_error()
    # CSR validation: sizes, pointers and the workspace are checked before anything is read
    report = (C.c_int32 * 4)()
    assert sb_lib.sb_csr_validate_workspace_bytes() == 32
    assert sb_lib.sb_csr_validate(-1, 4, 4, one, one, 1, report, one, 32, None) == 1
    assert sb_lib.sb_csr_validate(4, 4, 4, None, one, 1, report, one, 32, None) == 1
    assert sb_lib.sb_csr_validate(4, 4, 4, one, one, 1, report, one, 8, None) == 1
    assert b"workspace" in sb_lib.sb_last_error()
