"""The drop-in boundary exercised by the reference's OWN Python front end.

The reference package (``scorch``: matmul / einsum / @compile, registry and dispatch) is imported
from the copy that ``oracle/build_ref.py`` stages under ``oracle/_ref/pkg`` and is given a module
named ``scorch_ops`` to bind to, exactly as its ``prebuilt_kernels.py`` expects
(reference: src/scorch/prebuilt_kernels.py:8,96-101):

* ``gpu`` tests: this repository's ``scorch_b200.scorch_ops`` — every call must land in the GPU
  symbol (counted), and results must match the float64 oracle;
* CPU test: the reference's compiled extension — the stock path, which checks this test's own
  logic and the oracle against the reference's front end.

Mirrors the reference's dispatch tests (tests/test_scorch/test_matmul_dispatch.py:9-53,
test_prebuilt_kernel_registry.py:7-51, test_compile.py:70-127).  Skipped where the staged package
is absent.
"""
from __future__ import annotations

import sys

import numpy as np
import pytest
import torch

RTOL, ATOL = 1e-4, 1e-5

COUNTED = ("spmm_csr_float_v2", "prebuilt_spmm_csr_f64", "prebuilt_spmspm_csr_f32", "prebuilt_spmv_csr_f32",
           "sddmm_coo_float_prebuilt", "spmm_csr_bias_relu_float", "spmm_csr_bias_float")


class _Counting:
    """A module-like object that forwards to `inner` and counts calls of the dispatched symbols."""

    def __init__(self, inner):
        self._inner = inner
        self.calls = {}

    def __getattr__(self, name):
        fn = getattr(self._inner, name)
        if name not in COUNTED:
            return fn

        def counted(*a, **kw):
            self.calls[name] = self.calls.get(name, 0) + 1
            return fn(*a, **kw)
        return counted


def _reference_front_end(native_ops):
    """Import the staged reference package against `native_ops`; returns (scorch, counter, undo)."""
    from oracle import ref_loader
    pkg = ref_loader.reference_package_dir()
    if pkg is None:
        pytest.skip("the reference's Python package is not staged under oracle/_ref/pkg")
    saved = {k: v for k, v in sys.modules.items() if k == "scorch_ops" or k == "scorch" or k.startswith("scorch.")}
    for k in saved:
        del sys.modules[k]
    counter = _Counting(native_ops)
    sys.modules["scorch_ops"] = counter
    sys.path.insert(0, pkg)
    import scorch

    def undo():
        sys.path.remove(pkg)
        for k in [k for k in sys.modules if k == "scorch_ops" or k == "scorch" or k.startswith("scorch.")]:
            del sys.modules[k]
        sys.modules.update(saved)
    return scorch, counter, undo


def _inputs():
    g = torch.Generator().manual_seed(7)
    n, k = 96, 40
    a = torch.rand(n, n, generator=g) * (torch.rand(n, n, generator=g) < 0.08)
    a[5] = 0
    b = torch.rand(n, k, generator=g)
    b_sp = torch.rand(n, n, generator=g) * (torch.rand(n, n, generator=g) < 0.06)
    x = torch.rand(n, generator=g)
    q, kk = torch.randn(n, 24, generator=g), torch.randn(n, 24, generator=g)
    bias = torch.rand(k, generator=g)
    return a, b, b_sp, x, q, kk, bias


def _csr_np(t):
    c = t.to_sparse_csr()
    return (c.crow_indices().to(torch.int32).numpy(), c.col_indices().to(torch.int32).numpy(),
            c.values().numpy())


def _check_front_end(scorch, counter, oracle, monkeypatch):
    a, b, b_sp, x, q, kk, bias = _inputs()
    pos, crd, val = _csr_np(a)
    close = lambda got, want: oracle.allclose_report(np.asarray(got), want, RTOL, ATOL)[0]

    # CSR x dense -> torch.Tensor through spmm_csr_float_v2, torch.matmul forbidden on the way
    import scorch.ops as ref_ops_py

    def forbidden(*args, **kw):
        raise AssertionError("torch.matmul must not be used for a sparse matmul")
    with monkeypatch.context() as mp:
        mp.setattr(ref_ops_py.torch, "matmul", forbidden)
        c = scorch.matmul(a.to_sparse_csr(), b, format="dd")
    assert isinstance(c, torch.Tensor) and c.shape == (96, 40)
    assert close(c.numpy(), oracle.spmm_csr_acc64(pos, crd, val, b.numpy()))
    assert (c[5] == 0).all()
    assert counter.calls.get("spmm_csr_float_v2") == 1

    # float64 resolves to the typed symbol (registry test of the reference) and runs
    from scorch import STensor
    from scorch.prebuilt_kernels import resolve_prebuilt_matmul
    a64 = STensor.from_torch(a.double().to_sparse_csr())
    b64 = STensor.from_torch(b.double()).to_dense()
    assert resolve_prebuilt_matmul(a64, b64).symbol_name == "prebuilt_spmm_csr_f64"
    c64 = scorch.matmul(a64, b64, format="dd")
    np.testing.assert_allclose(c64.numpy(), a.double().numpy() @ b.double().numpy(), rtol=1e-12, atol=1e-12)
    assert counter.calls.get("prebuilt_spmm_csr_f64") == 1

    # CSR x vector -> dense 1-D tensor through prebuilt_spmv_csr_f32
    y = scorch.matmul(a.to_sparse_csr(), x)
    assert isinstance(y, torch.Tensor) and y.shape == (96,)
    assert close(y.numpy(), oracle.spmv_csr_acc64(pos, crd, val, x.numpy()))
    assert counter.calls.get("prebuilt_spmv_csr_f32") == 1

    # CSR x CSR -> sparse STensor, structure bit-exact, columns ascending
    bpos, bcrd, bval = _csr_np(b_sp)
    s = scorch.matmul(a.to_sparse_csr(), b_sp.to_sparse_csr())
    assert isinstance(s, STensor)
    wpos, wcrd, wval = oracle.spgemm(pos, crd, val, bpos, bcrd, bval, 96)
    gpos, gcrd = (t.numpy() for t in s.index.mode_indices[1])
    assert np.array_equal(gpos, wpos) and np.array_equal(gcrd, wcrd)
    assert close(s.values.numpy(), oracle.spgemm_values_acc64(pos, crd, val, bpos, bcrd, bval, 96, wpos, wcrd))
    assert counter.calls.get("prebuilt_spmspm_csr_f32") == 1

    # SDDMM with a COO mask -> the prebuilt SDDMM symbol, values in mask order
    mask = (a != 0).float().to_sparse_coo().coalesce()
    d = scorch.einsum("ij,ik,jk->ij", mask, q, kk)
    rows, cols = mask.indices()[0].to(torch.int32).numpy(), mask.indices()[1].to(torch.int32).numpy()
    want = (q.double().numpy()[rows] * kk.double().numpy()[cols]).sum(1)
    assert close(d.values.numpy(), want)
    assert counter.calls.get("sddmm_coo_float_prebuilt") == 1

    # the reference's own re-layout of a compressed operand (torch-op fast path of
    # change_mode_order) pins the oracle's transpose, which the device transpose is tested against
    t = STensor.from_torch(a.to_sparse_csr()).change_mode_order([1, 0])
    tpos, tcrd, tval = oracle.csr_transpose(pos, crd, val, 96)
    rp, rc = (x_.numpy() for x_ in t.index.mode_indices[1])
    assert np.array_equal(rp, tpos) and np.array_equal(rc, tcrd) and np.array_equal(t.values.numpy(), tval)

    # @scorch.compile: relu(A @ X + bias) fuses into the bias+ReLU SpMM symbol
    adj = STensor.from_torch(a.to_sparse_csr())

    @scorch.compile
    def fused(adj, feats, bias):
        h = scorch.matmul(adj, feats, format="dd")
        h = h + bias
        return torch.relu(h)

    r = fused(adj, b, bias)
    assert isinstance(r, torch.Tensor)
    assert close(r.numpy(), oracle.spmm_csr_acc64(pos, crd, val, b.numpy(), bias.numpy(), True))
    assert counter.calls.get("spmm_csr_bias_relu_float") == 1


@pytest.mark.gpu
def test_reference_front_end_over_the_gpu_symbols(oracle, monkeypatch):
    from scorch_b200 import scorch_ops as gpu_ops
    scorch, counter, undo = _reference_front_end(gpu_ops)
    try:
        _check_front_end(scorch, counter, oracle, monkeypatch)
    finally:
        undo()


def test_reference_front_end_over_its_own_extension(oracle, ref_ops, monkeypatch):
    scorch, counter, undo = _reference_front_end(ref_ops)
    try:
        _check_front_end(scorch, counter, oracle, monkeypatch)
    finally:
        undo()
