"""Host logic of the 3-D tensor contractions (TTM, MTTKRP over compressed-fibre tensors): the
layout produced from a dense tensor equals the reference's ``to_sparse`` arrays, the oracle equals
the reference's results, and the reduction to CSR x dense products is right — with the oracle
standing in for the CUDA SpMM, so none of this needs a GPU."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "hotpath_golden.npz"))


def levels_of(prefix):
    lv0 = [GOLD[prefix + "pos0"], GOLD[prefix + "crd0"]] if prefix + "pos0" in GOLD.files else []
    return [lv0, [GOLD[prefix + "pos1"], GOLD[prefix + "crd1"]], [GOLD[prefix + "pos2"], GOLD[prefix + "crd2"]]]


@pytest.mark.parametrize("fmt", ["dss", "sss"])
def test_layout_from_dense_matches_the_reference(fmt):
    from scorch_b200 import tensor3
    p = f"tensor3_{fmt}."
    st = tensor3.csf3_from_dense(torch.from_numpy(GOLD[p + "dense"]), fmt)
    assert str(st.format) == str(GOLD[p + "format"][0])
    want = levels_of(p)
    for got_level, want_level in zip(st.index.mode_indices, want):
        assert len(got_level) == len(want_level)
        for g, w in zip(got_level, want_level):
            assert g.dtype == torch.int32 and np.array_equal(g.numpy(), w)
    assert np.array_equal(st.values.numpy(), GOLD[p + "val"])
    assert torch.equal(tensor3.csf3_to_dense(st), torch.from_numpy(GOLD[p + "dense"]))


@pytest.mark.parametrize("fmt", ["dss", "sss"])
def test_oracle_matches_the_reference_results(oracle, fmt):
    p = f"tensor3_{fmt}."
    shape, lv, val = tuple(GOLD[p + "shape"]), levels_of(p), GOLD[p + "val"]
    assert np.array_equal(oracle.csf3_to_dense(shape, lv, val), GOLD[p + "dense"].astype(np.float64))
    np.testing.assert_allclose(oracle.ttm_acc64(shape, lv, val, GOLD[p + "B_km"]), GOLD[p + "ttm"],
                               rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(oracle.mttkrp_acc64(shape, lv, val, GOLD[p + "B_jm"], GOLD[p + "B_km"]),
                               GOLD[p + "mttkrp"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("fmt", ["dss", "sss"])
def test_reduction_to_csr_products(oracle, monkeypatch, fmt):
    """ttm / mttkrp with the CUDA SpMM replaced by the oracle's (and operands left on the host)."""
    from scorch_b200 import kernels as K, tensor3

    def cpu_spmm(pos, crd, val, B, **kw):
        return torch.from_numpy(oracle.spmm_csr_acc64(pos.numpy(), crd.numpy(), val.numpy(),
                                                      B.contiguous().numpy()).astype(np.float32))
    monkeypatch.setattr(K, "spmm_csr", cpu_spmm)
    monkeypatch.setattr(tensor3, "_on_device", lambda a, *d: (False, a, tuple(x.contiguous() for x in d)))
    rng = np.random.default_rng(5)
    dense = (rng.standard_normal((9, 7, 11)) * (rng.random((9, 7, 11)) < 0.25)).astype(np.float32)
    dense[3] = 0
    B, Bj = (rng.standard_normal(s).astype(np.float32) for s in ((11, 6), (7, 6)))
    st = tensor3.csf3_from_dense(torch.from_numpy(dense), fmt)
    got = tensor3.ttm(st, torch.from_numpy(B)).numpy()
    np.testing.assert_allclose(got, np.einsum("ijk,km->ijm", dense.astype(np.float64), B), rtol=1e-5, atol=1e-5)
    got = tensor3.mttkrp(st, torch.from_numpy(Bj), torch.from_numpy(B)).numpy()
    np.testing.assert_allclose(got, np.einsum("ijk,jm,km->im", dense.astype(np.float64), Bj, B), rtol=1e-5, atol=1e-5)
    # an all-zero tensor has no fibres
    empty = tensor3.csf3_from_dense(torch.zeros((4, 3, 5)), fmt)
    assert not tensor3.ttm(empty, torch.from_numpy(B[:5])).any()
    assert not tensor3.mttkrp(empty, torch.from_numpy(Bj[:3]), torch.from_numpy(B[:5])).any()
