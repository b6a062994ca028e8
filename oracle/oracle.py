"""numpy front end of the CPU oracle (``liboracle.so`` built from ``scorch_oracle.c``).

TEST INFRASTRUCTURE ONLY — imported by ``tests/``, the smoke check and the CPU-baseline legs of
the benchmark; never by the product package.  Each function names the reference kernel it
checks against (paths relative to the reference project).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None

_I32 = np.int32
_SUFFIX = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64",
           np.dtype(np.int32): "i32", np.dtype(np.int64): "i64"}


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "scorch_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE] + (["-B"] if force else []))
    return so


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.so_spgemm_symbolic.restype = C.c_int64
        _lib.so_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return int(lib().so_num_threads())


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def spmm_csr_v2(pos, crd, val, B, tile: int = 256):
    """spmm_csr_float_v2, csrc/spmm.h:2007-2089."""
    pos, crd, val, B = _c(pos, _I32), _c(crd, _I32), _c(val, np.float32), _c(B, np.float32)
    m, k = len(pos) - 1, B.shape[1]
    out = np.empty((m, k), np.float32)
    lib().so_spmm_csr_f32_v2(C.c_int(m), C.c_int(k), _p(pos), _p(crd), _p(val), _p(B), _p(out),
                             C.c_int(tile))
    return out


def spmm_csr_typed(pos, crd, val, B):
    """spmm_csr_typed<T>, csrc/spmm.h:91-150."""
    val = np.ascontiguousarray(val)
    sfx = _SUFFIX[val.dtype]
    pos, crd, B = _c(pos, _I32), _c(crd, _I32), _c(B, val.dtype)
    m, k = len(pos) - 1, B.shape[1]
    out = np.empty((m, k), val.dtype)
    getattr(lib(), "so_spmm_csr_" + sfx)(C.c_int(m), C.c_int(k), _p(pos), _p(crd), _p(val),
                                          _p(B), _p(out))
    return out


def spmm_csr_bias_act(pos, crd, val, B, bias, relu: bool):
    """spmm_csr_bias_act<float, relu>, csrc/spmm.h:28-89."""
    pos, crd, val, B = _c(pos, _I32), _c(crd, _I32), _c(val, np.float32), _c(B, np.float32)
    bias = _c(bias, np.float32)
    m, k = len(pos) - 1, B.shape[1]
    out = np.empty((m, k), np.float32)
    lib().so_spmm_csr_bias_act_f32(C.c_int(m), C.c_int(k), _p(pos), _p(crd), _p(val), _p(B),
                                   _p(bias), C.c_int(int(relu)), _p(out))
    return out


def spmv_csr(pos, crd, val, x):
    """spmv_csr<T>, csrc/kernels.h:12-49."""
    val = np.ascontiguousarray(val)
    sfx = _SUFFIX[val.dtype]
    pos, crd, x = _c(pos, _I32), _c(crd, _I32), _c(x, val.dtype)
    m = len(pos) - 1
    y = np.empty(m, val.dtype)
    getattr(lib(), "so_spmv_csr_" + sfx)(C.c_int(m), _p(pos), _p(crd), _p(val), _p(x), _p(y))
    return y


def sddmm_coo(row, col, sval, A, B):
    """sddmm_coo_float_prebuilt, csrc/kernels.h:508-570."""
    row, col, sval = _c(row, _I32), _c(col, _I32), _c(sval, np.float32)
    A, B = _c(A, np.float32), _c(B, np.float32)
    out = np.empty(len(sval), np.float32)
    lib().so_sddmm_coo_f32(C.c_int64(len(sval)), C.c_int(A.shape[1]), _p(row), _p(col), _p(sval),
                           _p(A), _p(B), _p(out))
    return out


def sddmm_csr(pos, crd, mval, Q, K):
    """Compiler-emitted SDDMM for a CSR mask (generator: src/scorch/ops.py:638-664).
    Returns (row, col, val) like the reference's all-COO output."""
    pos, crd, mval = _c(pos, _I32), _c(crd, _I32), _c(mval, np.float32)
    Q, K = _c(Q, np.float32), _c(K, np.float32)
    nnz = len(crd)
    r, c, v = np.empty(nnz, _I32), np.empty(nnz, _I32), np.empty(nnz, np.float32)
    lib().so_sddmm_csr_f32(C.c_int(len(pos) - 1), C.c_int(Q.shape[1]), _p(pos), _p(crd),
                           _p(mval), _p(Q), _p(K), _p(r), _p(c), _p(v))
    return r, c, v


def csr_row_softmax(pos, val):
    """_sparse_softmax_csr_vectorized, bench/bench_sparse_transformer.py:277-297."""
    pos, val = _c(pos, _I32), _c(val, np.float32)
    out = val.copy()
    lib().so_csr_row_softmax_f32(C.c_int(len(pos) - 1), _p(pos), _p(val), _p(out))
    return out


def spgemm_symbolic(Apos, Acrd, Bpos, Bcrd, n: int):
    """Symbolic phase of spmspm_csr<T>, csrc/kernels.h:69-111.  Returns (Cpos int32, total)."""
    Apos, Acrd, Bpos, Bcrd = (_c(a, _I32) for a in (Apos, Acrd, Bpos, Bcrd))
    m = len(Apos) - 1
    cpos = np.empty(m + 1, _I32)
    total = lib().so_spgemm_symbolic(C.c_int(m), C.c_int(n), _p(Apos), _p(Acrd), _p(Bpos),
                                     _p(Bcrd), _p(cpos))
    return cpos, int(total)


def spgemm(Apos, Acrd, Aval, Bpos, Bcrd, Bval, n: int):
    """spmspm_csr<T>, csrc/kernels.h:51-202.  Returns (Cpos, Ccrd, Cval)."""
    Aval = np.ascontiguousarray(Aval)
    sfx = _SUFFIX[Aval.dtype]
    Apos, Acrd, Bpos, Bcrd = (_c(a, _I32) for a in (Apos, Acrd, Bpos, Bcrd))
    Bval = _c(Bval, Aval.dtype)
    m = len(Apos) - 1
    cpos, total = spgemm_symbolic(Apos, Acrd, Bpos, Bcrd, n)
    if total >= 2 ** 31:
        raise OverflowError("SpGEMM output does not fit int32 row pointers")
    ccrd, cval = np.empty(total, _I32), np.empty(total, Aval.dtype)
    getattr(lib(), "so_spgemm_numeric_" + sfx)(C.c_int(m), C.c_int(n), _p(Apos), _p(Acrd),
                                                _p(Aval), _p(Bpos), _p(Bcrd), _p(Bval),
                                                _p(cpos), _p(ccrd), _p(cval))
    return cpos, ccrd, cval


# ---- float64 tolerance oracles ------------------------------------------------------------
def spmm_csr_acc64(pos, crd, val, B, bias=None, relu: bool = False):
    pos, crd, val, B = _c(pos, _I32), _c(crd, _I32), _c(val, np.float32), _c(B, np.float32)
    bias = None if bias is None else _c(bias, np.float32)
    m, k = len(pos) - 1, B.shape[1]
    out = np.empty((m, k), np.float64)
    lib().so_spmm_csr_acc64(C.c_int(m), C.c_int(k), _p(pos), _p(crd), _p(val), _p(B), _p(bias),
                            C.c_int(int(relu)), _p(out))
    return out


def spmv_csr_acc64(pos, crd, val, x):
    pos, crd, val, x = _c(pos, _I32), _c(crd, _I32), _c(val, np.float32), _c(x, np.float32)
    y = np.empty(len(pos) - 1, np.float64)
    lib().so_spmv_csr_acc64(C.c_int(len(pos) - 1), _p(pos), _p(crd), _p(val), _p(x), _p(y))
    return y


def sddmm_csr_acc64(pos, crd, mval, Q, K):
    pos, crd = _c(pos, _I32), _c(crd, _I32)
    mval = None if mval is None else _c(mval, np.float32)
    Q, K = _c(Q, np.float32), _c(K, np.float32)
    out = np.empty(len(crd), np.float64)
    lib().so_sddmm_csr_acc64(C.c_int(len(pos) - 1), C.c_int(Q.shape[1]), _p(pos), _p(crd),
                             _p(mval), _p(Q), _p(K), _p(out))
    return out


def csr_row_softmax_acc64(pos, val):
    pos, val = _c(pos, _I32), _c(val, np.float64)
    out = val.copy()
    lib().so_csr_row_softmax_acc64(C.c_int(len(pos) - 1), _p(pos), _p(val), _p(out))
    return out


def spgemm_values_acc64(Apos, Acrd, Aval, Bpos, Bcrd, Bval, n, Cpos, Ccrd):
    Apos, Acrd, Bpos, Bcrd, Cpos, Ccrd = (_c(a, _I32) for a in (Apos, Acrd, Bpos, Bcrd, Cpos, Ccrd))
    Aval, Bval = _c(Aval, np.float32), _c(Bval, np.float32)
    out = np.empty(len(Ccrd), np.float64)
    lib().so_spgemm_numeric_acc64(C.c_int(len(Apos) - 1), C.c_int(n), _p(Apos), _p(Acrd), _p(Aval),
                                  _p(Bpos), _p(Bcrd), _p(Bval), _p(Cpos), _p(Ccrd), _p(out))
    return out


# ---- format plumbing (numpy) ---------------------------------------------------------------
def dense_to_csr(A):
    """Row pointers, columns, values of the non-zero entries of a dense matrix in row-major
    order: what torch.Tensor.to_sparse_csr() gives the reference's callers
    (bench/bench_sparse_autoencoder.py:233,261).  -0.0 is dropped, NaN kept."""
    A = np.asarray(A)
    keep = A != 0
    pos = np.concatenate([[0], np.cumsum(keep.sum(axis=1))]).astype(np.int32)
    crd = np.nonzero(keep)[1].astype(np.int32)
    return pos, crd, A[keep]


def csr_sym_normalize_acc64(pos, crd):
    """val[p] = d_i^-1/2 d_j^-1/2 with d = stored entries per row (the pattern is A + I):
    bench/bench_gcn.py:233-267 (degree by scatter-add of ones, deg^-0.5, inf -> 0), in float64."""
    pos = np.asarray(pos, dtype=np.int64)
    deg = np.diff(pos).astype(np.float64)
    with np.errstate(divide="ignore"):
        dinv = np.where(deg > 0, deg ** -0.5, 0.0)
    rows = np.repeat(np.arange(len(deg)), np.diff(pos))
    return dinv[rows] * dinv[np.asarray(crd, dtype=np.int64)]


def allclose_report(got, want64, rtol=1e-4, atol=1e-5):
    """(ok, max_abs_err, n_violations) of |got - want| <= atol + rtol*|want| in float64."""
    got = np.asarray(got, dtype=np.float64).ravel()
    want64 = np.asarray(want64, dtype=np.float64).ravel()
    err = np.abs(got - want64)
    bad = err > (atol + rtol * np.abs(want64))
    ok = (not bad.any()) and bool(np.isfinite(got).all())
    return ok, (float(err.max()) if err.size else 0.0), int(bad.sum())


def csr_transpose(pos, crd, val, n):
    """CSR of the transpose (= CSC of the matrix), rows in ascending source-row order: what the
    torch-op fast path of STensor.change_mode_order produces for a 2-D compressed operand
    (src/scorch/stensor.py:785-896: argsort of new_row * cols + new_col, bincount, cumsum)."""
    pos, crd = np.asarray(pos, np.int64), np.asarray(crd, np.int64)
    m = len(pos) - 1
    row = np.repeat(np.arange(m, dtype=np.int64), np.diff(pos))
    order = np.argsort(crd * max(m, 1) + row, kind="stable")
    tpos = np.concatenate([[0], np.cumsum(np.bincount(crd, minlength=n))]).astype(np.int32)
    tval = None if val is None else np.asarray(val)[order]
    return tpos, row[order].astype(np.int32), tval


def topk_rows_to_csr(X, k, relu=False):
    """Exactly k entries per row: the k largest values of each row (ties between equal values go
    to the lower column), columns ascending, values clamped at zero when `relu` is set — the
    activation rule of benchmark configuration 3 (top-k of the pre-activations, ReLU'd)."""
    X = np.asarray(X, np.float32)
    m, n = X.shape
    crd = np.empty((m, k), np.int32)
    val = np.empty((m, k), np.float32)
    cols = np.arange(n)
    for i in range(m):
        pick = np.sort(np.lexsort((cols, -X[i].astype(np.float64)))[:k])
        crd[i] = pick
        val[i] = np.maximum(X[i, pick], 0) if relu else X[i, pick]
    pos = (np.arange(m + 1) * k).astype(np.int32)
    return pos, crd.reshape(-1), val.reshape(-1)


def csr_ewise(op, Apos, Acrd, Aval, Bpos, Bcrd, Bval):
    """Element-wise "mul" / "add" of two CSR matrices with the reference's output structure: the
    intersection / union of the stored columns per row, ascending, zeros that arise kept (what
    the compiler-emitted merge loops of the reference produce; pinned by the golden cases
    ewise_f32)."""
    Apos, Acrd, Bpos, Bcrd = (np.asarray(x) for x in (Apos, Acrd, Bpos, Bcrd))
    Aval, Bval = np.asarray(Aval), np.asarray(Bval)
    m = len(Apos) - 1
    pos, crd, val = [0], [], []
    for i in range(m):
        a = {int(c): Aval[p] for p, c in zip(range(Apos[i], Apos[i + 1]), Acrd[Apos[i]:Apos[i + 1]])}
        b = {int(c): Bval[p] for p, c in zip(range(Bpos[i], Bpos[i + 1]), Bcrd[Bpos[i]:Bpos[i + 1]])}
        cols = sorted(set(a) & set(b)) if op == "mul" else sorted(set(a) | set(b))
        for c in cols:
            crd.append(c)
            if op == "mul":
                val.append(a[c] * b[c])
            else:
                val.append(a[c] + b[c] if c in a and c in b else (a[c] if c in a else b[c]))
        pos.append(len(crd))
    return (np.asarray(pos, np.int32), np.asarray(crd, np.int32),
            np.asarray(val, Aval.dtype) if val else np.zeros(0, Aval.dtype))


# ---- 3-D compressed-fibre tensors (numpy) ---------------------------------------------------
def csf3_to_dense(shape, levels, val):
    """Dense (I, J, K) array of a tensor in the reference's ``d,s,s`` / ``s,s,s`` layout
    (src/scorch/storage.py, format.py:7-27): ``levels[0]`` is ``[]`` (dense i) or ``[pos0, crd0]``
    (the stored i slices), ``levels[1] = [pos1, crd1]`` the j of every stored (i, j) fibre,
    ``levels[2] = [pos2, crd2]`` the k of every entry of a fibre; ``val`` in that order."""
    I, J, K = shape
    out = np.zeros((I, J, K), dtype=np.float64)
    pos1, crd1 = (np.asarray(x) for x in levels[1])
    pos2, crd2 = (np.asarray(x) for x in levels[2])
    slices = np.asarray(levels[0][1]) if len(levels[0]) else np.arange(I)
    val = np.asarray(val)
    for r in range(len(pos1) - 1):
        for f in range(pos1[r], pos1[r + 1]):
            for p in range(pos2[f], pos2[f + 1]):
                out[slices[r], crd1[f], crd2[p]] = val[p]
    return out


def ttm_acc64(shape, levels, val, B):
    """C[i,j,m] = sum_k A[i,j,k] B[k,m] in float64 (the reference compiles this from
    einsum("ijk,km->ijm"), tests/test_scorch/test_kernels_comprehensive.py:418-445)."""
    return np.einsum("ijk,km->ijm", csf3_to_dense(shape, levels, val), np.asarray(B, np.float64))


def mttkrp_acc64(shape, levels, val, B, C):
    """D[i,m] = sum_jk A[i,j,k] B[j,m] C[k,m] in float64 (einsum("ijk,jm,km->im"),
    tests/test_scorch/test_kernels_comprehensive.py:450-482)."""
    return np.einsum("ijk,jm,km->im", csf3_to_dense(shape, levels, val), np.asarray(B, np.float64),
                     np.asarray(C, np.float64))
