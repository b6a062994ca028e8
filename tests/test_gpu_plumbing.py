"""Device-side format plumbing either side of the sparse kernels: dense -> CSR, the symmetric GCN
normalisation, CSR transpose (mode-order re-layout) and per-row top-k -> CSR, against the numpy
oracle (structure bit-exact, values bit-exact or within fp32 rounding)."""
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


def _random_csr(m, n, lens, seed, dtype=np.float32):
    rng = np.random.default_rng(seed)
    lens = np.minimum(np.asarray(lens, np.int64), n)
    pos = np.zeros(m + 1, np.int64)
    np.cumsum(lens, out=pos[1:])
    crd = np.empty(pos[-1], np.int32)
    for i in range(m):
        if lens[i]:
            crd[pos[i]:pos[i + 1]] = np.sort(rng.choice(n, size=lens[i], replace=False))
    val = (rng.standard_normal(pos[-1]) * 8).astype(dtype)
    return pos.astype(np.int32), crd, val


@pytest.mark.parametrize("m,n,mean,dtype", [(1, 1, 1, np.float32), (50, 70, 5, np.float32), (4000, 300, 40, np.float64),
                                             (300, 4000, 3, np.int32), (2500, 9, 6, np.int64), (10, 10, 0, np.float32)])
def test_csr_transpose_matches_oracle(oracle, m, n, mean, dtype):
    """Output rows of every length class: empty, a few entries (warp sort), hundreds (CTA sort in
    shared memory), thousands (in-place sort); all four value types and pattern-only."""
    from scorch_b200 import kernels as K
    lens = np.random.default_rng(m + n).poisson(mean, size=m)
    if m > 5:
        lens[3] = 0
    pos, crd, val = _random_csr(m, n, lens, seed=m * 7 + n, dtype=dtype)
    tpos, tcrd, tval = K.csr_transpose(torch.from_numpy(pos).cuda(), torch.from_numpy(crd).cuda(),
                                       torch.from_numpy(val).cuda(), n)
    wpos, wcrd, wval = oracle.csr_transpose(pos, crd, val, n)
    assert np.array_equal(tpos.cpu().numpy(), wpos)
    assert np.array_equal(tcrd.cpu().numpy(), wcrd)
    assert np.array_equal(tval.cpu().numpy(), wval)
    p2, c2, v2 = K.csr_transpose(torch.from_numpy(pos).cuda(), torch.from_numpy(crd).cuda(), None, n)
    assert v2 is None and torch.equal(p2, tpos) and torch.equal(c2, tcrd)
    # transposing back gives the original arrays
    bpos, bcrd, bval = K.csr_transpose(tpos, tcrd, tval, m)
    assert np.array_equal(bpos.cpu().numpy(), pos) and np.array_equal(bcrd.cpu().numpy(), crd)
    assert np.array_equal(bval.cpu().numpy(), val)


def test_matmul_relayouts_an_operand_stored_in_the_other_mode_order(oracle):
    """A CSR operand whose physical layout is the transpose of the logical matrix (mode order
    [1, 0]) is re-laid-out on the device before dispatch, as the reference's matmul does
    (src/scorch/ops.py:333-346), instead of being rejected."""
    import scorch_b200 as scorch
    from scorch_b200.stensor import STensor, TensorIndex, TensorStorage
    pos, crd, val = _random_csr(120, 80, np.random.default_rng(5).poisson(6, size=120), seed=6)
    B = np.random.default_rng(7).standard_normal((120, 16)).astype(np.float32)
    # physical (120 x 80) CSR array = logical (80 x 120) matrix A^T stored column-major
    idx = TensorIndex([[], [torch.from_numpy(pos), torch.from_numpy(crd)]], "d,s", mode_order=[1, 0])
    a = STensor((120, 80), TensorStorage(idx, torch.from_numpy(val)))
    out = scorch.matmul(a, torch.from_numpy(B), format="dd")
    tpos, tcrd, tval = oracle.csr_transpose(pos, crd, val, 80)
    want = oracle.spmm_csr_acc64(tpos, tcrd, tval, B)
    assert out.shape == (80, 16)
    ok, err, bad = oracle.allclose_report(out.numpy(), want, 1e-4, 1e-5)
    assert ok, (err, bad)


@pytest.mark.parametrize("m,n,k,relu", [(1, 8, 8, False), (33, 100, 5, True), (64, 4096, 32, True), (7, 300, 0, False),
                                         (200, 257, 256, False)])
def test_topk_rows_to_csr_matches_oracle(oracle, m, n, k, relu):
    from scorch_b200 import kernels as K
    rng = np.random.default_rng(m + n + k)
    X = rng.standard_normal((m, n)).astype(np.float32)
    if n > 20:
        X[0, :10] = X[0, 11]          # ties around a value: the lower columns win
        X[-1, :] = 1.5                # a whole row of ties
    pos, crd, val = K.topk_rows_to_csr(torch.from_numpy(X).cuda(), k, relu=relu)
    wpos, wcrd, wval = oracle.topk_rows_to_csr(X, k, relu)
    assert np.array_equal(pos.cpu().numpy(), wpos)
    assert np.array_equal(crd.cpu().numpy(), wcrd)
    assert np.array_equal(val.cpu().numpy(), wval)


def test_topk_activations_match_the_config3_generator_and_feed_spmm(oracle):
    """Top-32 of |z| per row through the kernel = the activations the benchmark generator builds
    with torch.topk + sort, and the CSR goes straight into the SpMM."""
    from scorch_b200 import kernels as K, workloads as W
    g = torch.Generator(device="cuda").manual_seed(0)
    z = torch.randn((256, 32768), generator=g, device="cuda", dtype=torch.float32).abs_()
    pos, crd, val = K.topk_rows_to_csr(z, 32, relu=True)
    A = W.sae_activations(256, 32768, 32, seed=0, device="cuda")
    assert torch.equal(pos, A.pos) and torch.equal(crd, A.crd) and torch.equal(val, A.val)
    Wd = W.sae_decoder(32768, 128, seed=1, device="cuda")
    y = K.spmm_csr(pos, crd, val, Wd)
    want = oracle.spmm_csr_acc64(pos.cpu().numpy(), crd.cpu().numpy(), val.cpu().numpy(), Wd.cpu().numpy())
    ok, err, bad = oracle.allclose_report(y.cpu().numpy(), want, 1e-4, 1e-5)
    assert ok, (err, bad)
