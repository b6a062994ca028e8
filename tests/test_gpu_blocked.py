"""Dense-block (tensor-core, TF32x3) SDDMM / SpMM path against the float64 oracle and the
gather-kernel path, on masks whose aligned 16x16 blocks are partly dense."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def dev(a):
    return (torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a).cuda()


def band_mask(rows, cols, window, density, seed, values=True):
    rng = np.random.default_rng(seed)
    i, j = np.arange(rows)[:, None], np.arange(cols)[None, :]
    dense = (np.abs(i - j) <= window) | (rng.random((rows, cols)) < density)
    pos = np.concatenate([[0], np.cumsum(dense.sum(1))]).astype(np.int32)
    crd = np.nonzero(dense)[1].astype(np.int32)
    val = rng.standard_normal(len(crd)).astype(np.float32) if values else np.ones(len(crd), np.float32)
    return dense, pos, crd, val


def count_dense_blocks(dense):
    r, c = dense.shape
    full = dense[: r // 16 * 16, : c // 16 * 16].reshape(r // 16, 16, c // 16, 16)
    return int(full.all(axis=(1, 3)).sum())


@pytest.mark.parametrize("rows,cols,window", [(512, 512, 40), (500, 530, 24), (64, 64, 100), (40, 40, 3)])
def test_block_plan_matches_dense_scan(rows, cols, window):
    from scorch_b200 import kernels as K
    dense, pos, crd, _ = band_mask(rows, cols, window, 0.02, seed=rows)
    bp = K.BlockPlan(dev(pos), dev(crd), n=cols)
    assert bp.blocks == count_dense_blocks(dense)
    assert bp.blocks * 256 + bp.rem_nnz == len(crd)


@pytest.mark.parametrize("d", [16, 32, 64, 128])
def test_blocked_sddmm_vs_oracle(oracle, d):
    from scorch_b200 import kernels as K
    dense, pos, crd, mval = band_mask(500, 530, 30, 0.02, seed=d)
    rng = np.random.default_rng(d + 1)
    Q = rng.standard_normal((3, 500, d)).astype(np.float32)
    Km = rng.standard_normal((3, 530, d)).astype(np.float32)
    bp = K.BlockPlan(dev(pos), dev(crd), n=530)
    assert bp.blocks > 20 and bp.rem_nnz > 0
    got = K.sddmm_csr(dev(pos), dev(crd), dev(mval), dev(Q), dev(Km), block_plan=bp)
    plain = K.sddmm_csr(dev(pos), dev(crd), dev(mval), dev(Q), dev(Km))
    for u in range(3):
        want = oracle.sddmm_csr_acc64(pos, crd, mval, Q[u], Km[u])
        ok, err, bad = oracle.allclose_report(got[u].cpu().numpy(), want, RTOL, ATOL)
        assert ok, f"d={d} unit {u}: max err {err}, {bad} bad"
    torch.testing.assert_close(got, plain, rtol=RTOL, atol=ATOL)
    nomask = K.sddmm_csr(dev(pos), dev(crd), None, dev(Q[0]), dev(Km[0]), block_plan=bp)
    ok, err, bad = oracle.allclose_report(nomask.cpu().numpy(), oracle.sddmm_csr_acc64(pos, crd, None, Q[0], Km[0]), RTOL, ATOL)
    assert ok, (err, bad)


@pytest.mark.parametrize("k", [32, 64, 128])
def test_blocked_spmm_vs_oracle(oracle, k):
    from scorch_b200 import kernels as K
    dense, pos, crd, val = band_mask(500, 530, 30, 0.02, seed=k)
    val = (val / 8).astype(np.float32)
    rng = np.random.default_rng(k + 1)
    B = rng.standard_normal((2, 530, k)).astype(np.float32)
    vals = np.stack([val, val[::-1].copy()])
    bias = rng.standard_normal(k).astype(np.float32)
    bp = K.BlockPlan(dev(pos), dev(crd), n=530)
    got = K.spmm_csr(dev(pos), dev(crd), dev(vals), dev(B), block_plan=bp)
    for u in range(2):
        ok, err, bad = oracle.allclose_report(got[u].cpu().numpy(), oracle.spmm_csr_acc64(pos, crd, vals[u], B[u]), RTOL, ATOL)
        assert ok, f"k={k} unit {u}: max err {err}, {bad} bad"
    got = K.spmm_csr(dev(pos), dev(crd), dev(val), dev(B[0]), bias=dev(bias), relu=True, block_plan=bp)
    ok, err, bad = oracle.allclose_report(got.cpu().numpy(), oracle.spmm_csr_acc64(pos, crd, val, B[0], bias, True), RTOL, ATOL)
    assert ok, (err, bad)


def test_sparse_attention_auto_uses_blocks_and_matches_oracle(oracle):
    from scorch_b200 import pipelines as P, workloads as W
    mask = W.attention_mask(1024, window=64, density=0.01, seed=0)
    Q, Km, V = W.attention_qkv(1, 3, 1024, 64, seed=1)
    pos, crd, mv = dev(mask.pos), dev(mask.crd), dev(mask.val)
    bp = P.attention_block_plan(pos, crd)
    assert bp is not None and bp.dense_fraction > 0.7
    O = P.sparse_attention(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125)
    O_plain = P.sparse_attention(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125, block_plan=None)
    torch.testing.assert_close(O, O_plain, rtol=RTOL, atol=ATOL)
    p, c, m = mask.pos.numpy(), mask.crd.numpy(), mask.val.numpy()
    for u in range(3):
        s64 = oracle.sddmm_csr_acc64(p, c, m, Q[u].numpy(), Km[u].numpy()) * 0.125
        o64 = oracle.spmm_csr_acc64(p, c, oracle.csr_row_softmax_acc64(p, s64).astype(np.float32), V[u].numpy())
        ok, err, bad = oracle.allclose_report(O[u].cpu().numpy(), o64, RTOL, ATOL)
        assert ok, (u, err, bad)
    # a random mask has no dense blocks: the plain kernels are used
    rnd = W.csr_uniform(512, 512, 0.05, seed=3)
    assert P.attention_block_plan(dev(rnd.pos), dev(rnd.crd)) is None
