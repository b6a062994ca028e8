"""Device-side format plumbing either side of the sparse kernels: dense -> CSR and the symmetric
GCN normalisation, against the numpy oracle (structure bit-exact, values within fp32 rounding)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,density", [(1, 1, 1.0), (7, 33, 0.3), (64, 64, 0.0), (129, 1000, 0.05),
                                          (300, 31, 0.9), (5, 4097, 0.5)])
def test_dense_to_csr_matches_oracle(oracle, m, n, density):
    from scorch_b200 import kernels as K
    rng = np.random.default_rng(m * 1000 + n)
    A = rng.standard_normal((m, n)).astype(np.float32)
    A[rng.random((m, n)) >= density] = 0.0
    if m > 2 and n > 3:
        A[1, :] = 0.0                    # an empty row
        A[2, 0] = -0.0                   # negative zero is not stored
        A[0, n - 1] = np.nan             # NaN is
    pos, crd, val = K.dense_to_csr(torch.from_numpy(A).cuda())
    wpos, wcrd, wval = oracle.dense_to_csr(A)
    assert np.array_equal(pos.cpu().numpy(), wpos)
    assert np.array_equal(crd.cpu().numpy(), wcrd)
    assert np.array_equal(val.cpu().numpy(), wval, equal_nan=True)
    # same structure as torch's own conversion
    ref = torch.from_numpy(np.nan_to_num(A, nan=1.0)).to_sparse_csr()
    assert np.array_equal(ref.crow_indices().numpy().astype(np.int32), wpos)


def test_dense_to_csr_of_a_column_slice():
    """A 2-D view with a row pitch larger than its width (a column panel of a wider matrix)."""
    from scorch_b200 import kernels as K
    rng = np.random.default_rng(1)
    big = rng.standard_normal((50, 96)).astype(np.float32)
    big[rng.random(big.shape) < 0.7] = 0.0
    view = torch.from_numpy(big).cuda()[:, 32:64]
    pos, crd, val = K.dense_to_csr(view)
    ref = torch.from_numpy(big[:, 32:64].copy()).to_sparse_csr()
    assert torch.equal(pos.cpu(), ref.crow_indices().int())
    assert torch.equal(crd.cpu(), ref.col_indices().int())
    assert torch.equal(val.cpu(), ref.values())


def test_csr_sym_normalize_matches_oracle_and_feeds_spmm(oracle):
    from scorch_b200 import kernels as K, workloads as W
    g = W.gcn_graph(3000, mean_deg=12.0, max_deg=500, seed=4)
    pos, crd = g.pos.numpy(), g.crd.numpy()
    val = K.csr_sym_normalize(g.pos.cuda(), g.crd.cuda())
    want = oracle.csr_sym_normalize_acc64(pos, crd)
    ok, err, bad = oracle.allclose_report(val.cpu().numpy(), want, 1e-6, 0.0)
    assert ok, (err, bad)
    ok, err, bad = oracle.allclose_report(g.val.numpy(), want, 1e-5, 0.0)   # the generator's torch ops
    assert ok, (err, bad)
    # rows without entries give zeros and do not divide by zero
    pos2 = np.array([0, 2, 2, 3], dtype=np.int32)
    crd2 = np.array([0, 2, 1], dtype=np.int32)
    v2 = K.csr_sym_normalize(torch.from_numpy(pos2).cuda(), torch.from_numpy(crd2).cuda()).cpu().numpy()
    assert np.allclose(v2, [0.5, 2 ** -0.5, 0.0]) and np.isfinite(v2).all()
