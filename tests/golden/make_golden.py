"""Generate the golden vectors in this directory by running the REFERENCE itself.

Run in a container that has the reference checkout (its location: SCORCH_REFERENCE_ROOT, or a
directory named ``reference`` beside this repository) and the compiled reference extension
(``python oracle/build_ref.py``):

    python tests/golden/make_golden.py

The script imports the reference's Python package from its source tree, with the compiled
``scorch_ops`` from ``oracle/_ref`` on the path, calls its public API (``scorch.matmul``,
``scorch.einsum``, the fused prebuilt kernels) on small seeded inputs and stores inputs and
outputs in ``hotpath_golden.npz``.  The tests never need the reference: they read the file.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import build_ref, ref_loader  # noqa: E402

REF = build_ref.reference_root()

ref_ops = ref_loader.load()
assert ref_ops is not None, "build oracle/_ref first (python oracle/build_ref.py)"
sys.modules["scorch_ops"] = ref_ops
sys.path.insert(0, os.path.join(REF, "src"))
import scorch  # noqa: E402  (the reference package)

out = {}
rng = np.random.default_rng(20240)


def rand_csr(m, n, density, dtype=np.float32, ints=False, empty_rows=()):
    mask = rng.random((m, n)) < density
    for r in empty_rows:
        mask[r] = False
    if ints:
        dense = rng.integers(-9, 10, size=(m, n)).astype(dtype) * mask
        # make sure stored entries are non-zero so torch keeps them
        dense[mask & (dense == 0)] = 3
    else:
        dense = (rng.standard_normal((m, n)).astype(dtype)) * mask
    t = torch.from_numpy(dense).to_sparse_csr()
    return t


def put(prefix, **arrays):
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[f"{prefix}.{k}"] = np.ascontiguousarray(v)


def csr_arrays(t):
    return (t.crow_indices().to(torch.int32), t.col_indices().to(torch.int32), t.values())


# ---- SpMM (fp32 -> spmm_csr_float_v2; typed -> spmm_csr_typed) -----------------------------------
for name, dtype, ints, k in (("spmm_f32", np.float32, False, 20), ("spmm_f32_k300", np.float32, False, 300),
                             ("spmm_f64", np.float64, False, 9), ("spmm_i32", np.int32, True, 5),
                             ("spmm_i64", np.int64, True, 6)):
    A = rand_csr(37, 29, 0.2, dtype, ints, empty_rows=(0, 11, 36))
    if ints:
        B = torch.from_numpy(rng.integers(-9, 10, size=(29, k)).astype(dtype))
    else:
        B = torch.from_numpy(rng.standard_normal((29, k)).astype(dtype))
    C = scorch.matmul(A, B, format="dd")
    pos, crd, val = csr_arrays(A)
    put(name, pos=pos, crd=crd, val=val, B=B, C=C)

# ---- fused bias (+ReLU) --------------------------------------------------------------------------
A = rand_csr(41, 33, 0.15, empty_rows=(3, 40))
B = torch.from_numpy(rng.standard_normal((33, 24)).astype(np.float32))
bias = torch.from_numpy(rng.standard_normal(24).astype(np.float32))
pos, crd, val = csr_arrays(A)
for relu, fn in ((True, ref_ops.spmm_csr_bias_relu_float), (False, ref_ops.spmm_csr_bias_float)):
    r = fn([41, 24], [41, 33], [[], [pos, crd]], val, [33, 24], [[], []], B.flatten(), bias)
    put(f"spmm_bias_relu{int(relu)}", pos=pos, crd=crd, val=val, B=B, bias=bias,
        C=r.storage.value.view(41, 24))

# ---- SpMV ----------------------------------------------------------------------------------------
for name, dtype, ints in (("spmv_f32", np.float32, False), ("spmv_f64", np.float64, False),
                          ("spmv_i32", np.int32, True), ("spmv_i64", np.int64, True)):
    A = rand_csr(53, 47, 0.18, dtype, ints, empty_rows=(5,))
    x = torch.from_numpy((rng.integers(-9, 10, size=47) if ints else rng.standard_normal(47)).astype(dtype))
    y = scorch.matmul(A, x)
    pos, crd, val = csr_arrays(A)
    put(name, pos=pos, crd=crd, val=val, x=x, y=y)

# ---- SpGEMM (structure must be bit-exact; includes an exact cancellation) ---------------------------
for name, dtype, ints in (("spgemm_f32", np.float32, False), ("spgemm_f64", np.float64, False),
                          ("spgemm_i32", np.int32, True), ("spgemm_i64", np.int64, True)):
    A = rand_csr(45, 38, 0.12, dtype, ints, empty_rows=(7,))
    B = rand_csr(38, 51, 0.12, dtype, ints, empty_rows=(2,))
    Cs = scorch.matmul(A, B)
    cpos, ccrd = Cs.index.mode_indices[1]
    ap, ac, av = csr_arrays(A)
    bp, bc, bv = csr_arrays(B)
    put(name, Apos=ap, Acrd=ac, Aval=av, Bpos=bp, Bcrd=bc, Bval=bv, Cpos=cpos, Ccrd=ccrd,
        Cval=Cs.values, n=np.array([51]))

# cancellation: row 0 of A = [1, 1], B rows [2 at col 3] and [-2 at col 3] -> C[0,3] = 0 is KEPT
ap = torch.tensor([0, 2, 3], dtype=torch.int32); ac = torch.tensor([0, 1, 1], dtype=torch.int32)
av = torch.tensor([1.0, 1.0, 5.0]); bp = torch.tensor([0, 2, 4], dtype=torch.int32)
bc = torch.tensor([1, 3, 3, 4], dtype=torch.int32); bv = torch.tensor([7.0, 2.0, -2.0, 1.5])
r = ref_ops.prebuilt_spmspm_csr_f32([2, 5], [2, 2], [[], [ap, ac]], av, [2, 5], [[], [bp, bc]], bv)
put("spgemm_cancel", Apos=ap, Acrd=ac, Aval=av, Bpos=bp, Bcrd=bc, Bval=bv,
    Cpos=r.storage.index.mode_indices[1][0], Ccrd=r.storage.index.mode_indices[1][1],
    Cval=r.storage.value, n=np.array([5]))

# ---- SDDMM: COO mask (prebuilt) and CSR mask (compiler-emitted loop), both subscript forms ---------
M = (rng.random((35, 31)) < 0.2)
M[4] = False
mask_dense = torch.from_numpy((rng.standard_normal((35, 31)).astype(np.float32)) * M)
Q = torch.from_numpy(rng.standard_normal((35, 16)).astype(np.float32))
Kt = torch.from_numpy(rng.standard_normal((31, 16)).astype(np.float32))
coo = mask_dense.to_sparse_coo().coalesce()
r = scorch.einsum("ij,ik,jk->ij", coo, Q, Kt)
put("sddmm_coo", row=coo.indices()[0].to(torch.int32), col=coo.indices()[1].to(torch.int32),
    mval=coo.values(), Q=Q, K=Kt, out_val=r.values,
    out_row=r.index.mode_indices[0][0], out_col=r.index.mode_indices[1][0])
csr = mask_dense.to_sparse_csr()
r = scorch.einsum("ij,ik,jk->ij", csr, Q, Kt)
pos, crd, val = csr_arrays(csr)
put("sddmm_csr", pos=pos, crd=crd, mval=val, Q=Q, K=Kt, out_val=r.values,
    out_row=r.index.mode_indices[0][0], out_col=r.index.mode_indices[1][0],
    out_format=np.array([str(r.format)]))
r = scorch.einsum("ij,ik,kj->ij", csr, Q, Kt.t().contiguous())
put("sddmm_csr_kj", out_val=r.values, out_row=r.index.mode_indices[0][0],
    out_col=r.index.mode_indices[1][0])

# ---- CSR row softmax (the reference's caller-side function) -----------------------------------------
# The bench module needs matplotlib at import time; take just this one function's source from
# the reference file and execute it (nothing is copied into this repository).
import ast  # noqa: E402

_src = open(os.path.join(REF, "bench", "bench_sparse_transformer.py")).read()
_fn = next(n for n in ast.parse(_src).body
           if isinstance(n, ast.FunctionDef) and n.name == "_sparse_softmax_csr_vectorized")
_ns = {"torch": torch}
exec(compile(ast.Module(body=[_fn], type_ignores=[]), "bench_sparse_transformer.py", "exec"), _ns)
sm = _ns["_sparse_softmax_csr_vectorized"](csr.crow_indices(), csr.values(), 35)
put("softmax", pos=pos, val=val, out=sm)

# ---- element-wise CSR (x) CSR multiply and CSR + CSR add (compiler-emitted merge loops) -----------------
from scorch import STensor  # noqa: E402

# (float32 only: the reference's emitted code for these patterns rejects other value types)
for name, dtype in (("ewise_f32", np.float32),):
    A = rand_csr(33, 27, 0.3, dtype, empty_rows=(4, 32))
    B = rand_csr(33, 27, 0.3, dtype, empty_rows=(4, 9))
    a_st, b_st = STensor.from_torch(A), STensor.from_torch(B)
    prod = scorch.einsum("ij,ij->ij", a_st, b_st, format="ds")
    total = a_st + b_st
    ap, ac, av = csr_arrays(A)
    bp, bc, bv = csr_arrays(B)
    put(name, Apos=ap, Acrd=ac, Aval=av, Bpos=bp, Bcrd=bc, Bval=bv,
        mul_pos=prod.index.mode_indices[1][0], mul_crd=prod.index.mode_indices[1][1], mul_val=prod.values,
        mul_format=np.array([str(prod.format)]),
        add_pos=total.index.mode_indices[1][0], add_crd=total.index.mode_indices[1][1], add_val=total.values,
        add_format=np.array([str(total.format)]), n=np.array([27]))

# ---- 3-D compressed-fibre tensor times matrices: TTM and MTTKRP (compiler-emitted loops) ----------------
def csf_arrays(st):
    lv = st.index.mode_indices
    arrays = {"pos1": lv[1][0], "crd1": lv[1][1], "pos2": lv[2][0], "crd2": lv[2][1], "val": st.values}
    if len(lv[0]):
        arrays.update(pos0=lv[0][0], crd0=lv[0][1])
    return arrays


T3 = torch.from_numpy((rng.standard_normal((7, 6, 9)).astype(np.float32)) * (rng.random((7, 6, 9)) < 0.3))
T3[2] = 0            # an i slice without entries
T3[:, 4, :] = 0      # a j that no fibre uses
Bm = torch.from_numpy(rng.standard_normal((9, 5)).astype(np.float32))     # (K, M)
Bj = torch.from_numpy(rng.standard_normal((6, 5)).astype(np.float32))     # (J, M)
for fmt in ("dss", "sss"):
    a_st = STensor.from_torch(T3).to_sparse(fmt)
    ttm = scorch.einsum("ijk,km->ijm", a_st, STensor.from_torch(Bm), format="ddd")
    mk = scorch.einsum("ijk,jm,km->im", a_st, STensor.from_torch(Bj), STensor.from_torch(Bm), format="dd")
    put("tensor3_" + fmt, shape=np.array(T3.shape), dense=T3, B_km=Bm, B_jm=Bj,
        ttm=ttm.to_torch(), mttkrp=mk.to_torch(), format=np.array([str(a_st.format)]), **csf_arrays(a_st))

np.savez_compressed(os.path.join(HERE, "hotpath_golden.npz"), **out)
print("wrote", len(out), "arrays;", sum(v.nbytes for v in out.values()), "bytes")
