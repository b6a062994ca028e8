"""Pins the CPU oracle (oracle/scorch_oracle.c) to the reference: its own known-answer test,
golden vectors produced by running the reference, and the compiled reference extension."""
from __future__ import annotations

import numpy as np
import pytest
import torch

TOL = dict(rtol=1e-5, atol=1e-6)  # oracle (strict IEEE) vs reference (-ffast-math): last-bit noise


def test_known_answer_spgemm_from_reference_tests(oracle):
    # reference: tests/test_scorch/test_kernels.py:473-615 — diag(1..5) times an arrowhead matrix
    A = np.diag(np.arange(1, 6)).astype(np.float32)
    B = np.zeros((5, 5), np.float32)
    B[0] = [1, 2, 3, 4, 5]
    B[:, 0] = [1, 2, 3, 4, 5]
    B[np.arange(5), np.arange(5)] = [1, 2, 3, 4, 5]
    import scipy.sparse as sp
    a, b = sp.csr_matrix(A), sp.csr_matrix(B)
    a.sort_indices(); b.sort_indices()
    cpos, ccrd, cval = oracle.spgemm(a.indptr, a.indices, a.data, b.indptr, b.indices, b.data, 5)
    assert cpos.tolist() == [0, 5, 7, 9, 11, 13]
    assert ccrd.tolist() == [0, 1, 2, 3, 4, 0, 1, 0, 2, 0, 3, 0, 4]
    assert cval.tolist() == [1, 2, 3, 4, 5, 4, 4, 9, 9, 16, 16, 25, 25]


@pytest.mark.parametrize("case", ["spmm_f32", "spmm_f32_k300"])
def test_spmm_v2_vs_golden(oracle, golden, case):
    g = golden.case(case)
    got = oracle.spmm_csr_v2(g["pos"], g["crd"], g["val"], g["B"])
    np.testing.assert_allclose(got, g["C"], **TOL)
    # rows without entries are exactly zero (reference csrc/spmm.h:2051)
    empty = np.diff(g["pos"]) == 0
    assert empty.any() and (got[empty] == 0).all()


@pytest.mark.parametrize("case", ["spmm_f32", "spmm_f64", "spmm_i32", "spmm_i64"])
def test_spmm_typed_vs_golden(oracle, golden, case):
    g = golden.case(case)
    got = oracle.spmm_csr_typed(g["pos"], g["crd"], g["val"], g["B"])
    if got.dtype.kind == "i":
        assert (got == g["C"]).all()
    else:
        np.testing.assert_allclose(got, g["C"], **TOL)


@pytest.mark.parametrize("relu", [0, 1])
def test_spmm_bias_act_vs_golden(oracle, golden, relu):
    g = golden.case(f"spmm_bias_relu{relu}")
    got = oracle.spmm_csr_bias_act(g["pos"], g["crd"], g["val"], g["B"], g["bias"], bool(relu))
    np.testing.assert_allclose(got, g["C"], **TOL)
    empty = np.diff(g["pos"]) == 0
    want = np.maximum(g["bias"], 0) if relu else g["bias"]
    assert empty.any() and np.array_equal(got[empty], np.broadcast_to(want, got[empty].shape))


@pytest.mark.parametrize("case", ["spmv_f32", "spmv_f64", "spmv_i32", "spmv_i64"])
def test_spmv_vs_golden(oracle, golden, case):
    g = golden.case(case)
    got = oracle.spmv_csr(g["pos"], g["crd"], g["val"], g["x"])
    if got.dtype.kind == "i":
        assert (got == g["y"]).all()
    else:
        np.testing.assert_allclose(got, g["y"], **TOL)


@pytest.mark.parametrize("case", ["spgemm_f32", "spgemm_f64", "spgemm_i32", "spgemm_i64", "spgemm_cancel"])
def test_spgemm_vs_golden(oracle, golden, case):
    g = golden.case(case)
    cpos, ccrd, cval = oracle.spgemm(g["Apos"], g["Acrd"], g["Aval"], g["Bpos"], g["Bcrd"],
                                     g["Bval"], int(g["n"][0]))
    assert np.array_equal(cpos, g["Cpos"])  # bit-exact structure
    assert np.array_equal(ccrd, g["Ccrd"])
    if cval.dtype.kind == "i":
        assert np.array_equal(cval, g["Cval"])
    else:
        np.testing.assert_allclose(cval, g["Cval"], **TOL)


def test_spgemm_keeps_cancelled_entry(golden):
    g = golden.case("spgemm_cancel")
    row0 = slice(g["Cpos"][0], g["Cpos"][1])
    assert g["Ccrd"][row0].tolist() == [1, 3, 4] and g["Cval"][row0].tolist() == [7.0, 0.0, 1.5]


def test_sddmm_vs_golden(oracle, golden):
    g = golden.case("sddmm_coo")
    got = oracle.sddmm_coo(g["row"], g["col"], g["mval"], g["Q"], g["K"])
    np.testing.assert_allclose(got, g["out_val"], **TOL)
    assert np.array_equal(g["out_row"], g["row"]) and np.array_equal(g["out_col"], g["col"])
    c = golden.case("sddmm_csr")
    r, col, v = oracle.sddmm_csr(c["pos"], c["crd"], c["mval"], c["Q"], c["K"])
    assert str(c["out_format"][0]) == "o,o"
    assert np.array_equal(r, c["out_row"]) and np.array_equal(col, c["out_col"])
    assert r.dtype == np.int32 and c["out_row"].dtype == np.int32
    np.testing.assert_allclose(v, c["out_val"], **TOL)
    kj = golden.case("sddmm_csr_kj")  # "ij,ik,kj->ij": same numbers after the operand transpose
    np.testing.assert_allclose(v, kj["out_val"], **TOL)
    assert np.array_equal(r, kj["out_row"]) and np.array_equal(col, kj["out_col"])


def test_softmax_vs_golden(oracle, golden):
    g = golden.case("softmax")
    got = oracle.csr_row_softmax(g["pos"], g["val"])
    np.testing.assert_allclose(got, g["out"], rtol=1e-5, atol=1e-7)


def test_acc64_oracles_agree_with_restatement(oracle):
    rng = np.random.default_rng(3)
    import scipy.sparse as sp
    A = sp.random(80, 70, 0.1, format="csr", random_state=4, dtype=np.float32)
    A.sort_indices()
    B = rng.standard_normal((70, 12)).astype(np.float32)
    ok, err, bad = oracle.allclose_report(oracle.spmm_csr_v2(A.indptr, A.indices, A.data, B),
                                          oracle.spmm_csr_acc64(A.indptr, A.indices, A.data, B))
    assert ok, (err, bad)
    x = rng.standard_normal(70).astype(np.float32)
    ok, err, bad = oracle.allclose_report(oracle.spmv_csr(A.indptr, A.indices, A.data, x),
                                          oracle.spmv_csr_acc64(A.indptr, A.indices, A.data, x))
    assert ok, (err, bad)


# ---- against the compiled reference itself (skipped where oracle/_ref is absent) ------------------
def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def test_oracle_vs_compiled_reference(oracle, ref_ops):
    from scorch_b200 import workloads as W
    A = W.csr_uniform(512, 384, 0.03, seed=5)
    B = W.dense_normal(384, 40, seed=6)
    pos, crd, val = A.pos, A.crd, A.val
    args = ([512, 40], [512, 384], [[], [pos, crd]], val, [384, 40], [[], []], B.flatten())
    want = ref_ops.spmm_csr_float_v2(*args).storage.value.view(512, 40).numpy()
    np.testing.assert_allclose(oracle.spmm_csr_v2(pos.numpy(), crd.numpy(), val.numpy(), B.numpy()),
                               want, **TOL)
    x = W.dense_normal(384, 1, seed=7).flatten()
    want = ref_ops.prebuilt_spmv_csr_f32([512], [512, 384], [[], [pos, crd]], val, [384], [[]], x)
    np.testing.assert_allclose(oracle.spmv_csr(pos.numpy(), crd.numpy(), val.numpy(), x.numpy()),
                               want.storage.value.numpy(), **TOL)
    S = W.powerlaw_square(3000, mean_nnz=6.0, seed=8)
    r = ref_ops.prebuilt_spmspm_csr_f32([3000, 3000], [3000, 3000], [[], [S.pos, S.crd]], S.val,
                                        [3000, 3000], [[], [S.pos, S.crd]], S.val)
    cpos, ccrd, cval = oracle.spgemm(S.pos.numpy(), S.crd.numpy(), S.val.numpy(), S.pos.numpy(),
                                     S.crd.numpy(), S.val.numpy(), 3000)
    assert np.array_equal(cpos, r.storage.index.mode_indices[1][0].numpy())
    assert np.array_equal(ccrd, r.storage.index.mode_indices[1][1].numpy())
    np.testing.assert_allclose(cval, r.storage.value.numpy(), **TOL)


@pytest.mark.parametrize("op", ["mul", "add"])
def test_elementwise_vs_golden(oracle, golden, op):
    """The reference's compiled merge loops (einsum "ij,ij->ij" and A + B on CSR operands) pin
    the structure (intersection / union, zeros kept) and the values of the element-wise oracle."""
    g = golden.case("ewise_f32")
    pos, crd, val = oracle.csr_ewise(op, g["Apos"], g["Acrd"], g["Aval"], g["Bpos"], g["Bcrd"], g["Bval"])
    assert np.array_equal(pos, g[f"{op}_pos"]) and np.array_equal(crd, g[f"{op}_crd"])
    np.testing.assert_allclose(val, g[f"{op}_val"], rtol=1e-6, atol=0)
