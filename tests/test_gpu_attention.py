"""The one-call sparse attention (blocks on the tensor cores with a running row softmax, scattered
entries through the gather kernels) against the float64 oracle of the three-operator sequence
SDDMM -> row softmax -> SpMM, and against the three-operator GPU path."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def dev(a):
    return (torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a).cuda()


def make_mask(rows, cols, window, density, seed, empty_rows=(), values=True):
    rng = np.random.default_rng(seed)
    i, j = np.arange(rows)[:, None], np.arange(cols)[None, :]
    dense = (np.abs(i - j) <= window) | (rng.random((rows, cols)) < density)
    for r in empty_rows:
        dense[r, :] = False
    pos = np.concatenate([[0], np.cumsum(dense.sum(1))]).astype(np.int32)
    crd = np.nonzero(dense)[1].astype(np.int32)
    val = (rng.uniform(0.5, 1.5, len(crd)) if values else np.ones(len(crd))).astype(np.float32)
    return dense, pos, crd, val


def count_blocks(dense, min_entries=64):
    """(blocks, entries inside them): aligned 16x16 blocks of complete row / column blocks with at
    least `min_entries` stored entries."""
    r, c = dense.shape
    cnt = dense[: r // 16 * 16, : c // 16 * 16].reshape(r // 16, 16, c // 16, 16).sum(axis=(1, 3))
    sel = cnt >= min_entries
    return int(sel.sum()), int(cnt[sel].sum())


def oracle_attention(oracle, pos, crd, mval, Q, Km, V, scale):
    s64 = oracle.sddmm_csr_acc64(pos, crd, mval, Q, Km) * scale
    p64 = oracle.csr_row_softmax_acc64(pos, s64)
    return oracle.spmm_csr_acc64(pos, crd, p64.astype(np.float32), V)


@pytest.mark.parametrize("rows,cols,window,density", [
    (512, 512, 40, 0.02), (500, 530, 24, 0.02), (500, 525, 300, 0.0), (64, 64, 100, 0.0),
    (40, 40, 3, 0.05), (256, 256, 0, 0.3), (100, 4000, 20, 0.01)])
def test_attn_plan_matches_dense_scan(rows, cols, window, density):
    from scorch_b200 import kernels as K
    dense, pos, crd, _ = make_mask(rows, cols, window, density, seed=rows + cols)
    ap = K.AttnPlan(dev(pos), dev(crd), n=cols)
    blocks, inside = count_blocks(dense)
    assert ap.blocks == blocks
    assert ap.rem_nnz == len(crd) - inside
    assert abs(ap.block_fraction - (inside / max(len(crd), 1))) < 1e-12


@pytest.mark.parametrize("d", [32, 64])
@pytest.mark.parametrize("rows,cols,window,density,empty", [
    (500, 500, 30, 0.02, (3, 17, 250)),     # band + scattered entries, a ragged last row block
    (256, 256, 40, 0.0, ()),                 # band only: full blocks, masked edge blocks, a few edge entries gathered
    (300, 300, 0, 0.05, (0,)),               # no blocks at all: everything goes through the gather kernels
    (128, 640, 24, 0.01, ()),                # K / V longer than Q
])
def test_sparse_attention_vs_oracle(oracle, d, rows, cols, window, density, empty):
    from scorch_b200 import kernels as K
    dense, pos, crd, mval = make_mask(rows, cols, window, density, seed=d + rows, empty_rows=empty)
    rng = np.random.default_rng(d + 1)
    Q = (rng.standard_normal((3, rows, d)) * 0.6).astype(np.float32)
    Km = (rng.standard_normal((3, cols, d)) * 0.6).astype(np.float32)
    V = rng.standard_normal((3, cols, d)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    ap = K.AttnPlan(dev(pos), dev(crd), n=cols)
    if window >= 24:
        assert ap.blocks > 0
    got = K.sparse_attention_csr(dev(pos), dev(crd), dev(mval), dev(Q), dev(Km), dev(V), scale=scale,
                                 attn_plan=ap)
    for u in range(3):
        want = oracle_attention(oracle, pos, crd, mval, Q[u], Km[u], V[u], scale)
        ok, err, bad = oracle.allclose_report(got[u].cpu().numpy(), want, RTOL, ATOL)
        assert ok, f"d={d} unit {u}: max err {err}, {bad} bad"
    for r in empty:
        assert torch.count_nonzero(got[:, r]) == 0
    # without mask values, one unit, 2-D operands
    got1 = K.sparse_attention_csr(dev(pos), dev(crd), None, dev(Q[0]), dev(Km[0]), dev(V[0]), scale=scale,
                                  attn_plan=ap)
    want = oracle_attention(oracle, pos, crd, None, Q[0], Km[0], V[0], scale)
    ok, err, bad = oracle.allclose_report(got1.cpu().numpy(), want, RTOL, ATOL)
    assert ok, (err, bad)


def test_sparse_attention_large_scores_are_stable(oracle):
    """Scores of several hundred: the running maximum keeps exp() in range, in the blocks and in
    the scattered entries alike."""
    from scorch_b200 import kernels as K
    dense, pos, crd, _ = make_mask(256, 256, 24, 0.02, seed=5)
    rng = np.random.default_rng(6)
    Q = (rng.standard_normal((256, 64)) * 4).astype(np.float32)
    Km = (rng.standard_normal((256, 64)) * 4).astype(np.float32)
    V = rng.standard_normal((256, 64)).astype(np.float32)
    got = K.sparse_attention_csr(dev(pos), dev(crd), None, dev(Q), dev(Km), dev(V), scale=1.0)
    assert torch.isfinite(got).all()
    want = oracle_attention(oracle, pos, crd, None, Q, Km, V, 1.0)
    # a score of magnitude 500 carries an fp32 rounding error of 3e-5, i.e. 3e-5 relative in exp()
    ok, err, bad = oracle.allclose_report(got.cpu().numpy(), want, 2e-3, 1e-4)
    assert ok, (err, bad)


def test_sparse_attention_stages_equal_whole_call():
    from scorch_b200 import kernels as K, workloads as W
    mask = W.attention_mask(1024, window=64, density=0.01, seed=0)
    Q, Km, V = W.attention_qkv(1, 3, 1024, 64, seed=1)
    pos, crd, mv = dev(mask.pos), dev(mask.crd), dev(mask.val)
    ap = K.AttnPlan(pos, crd)
    whole = K.sparse_attention_csr(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125, attn_plan=ap)
    out = torch.full_like(whole, float("nan"))
    for stage in (1, 2):
        K.sparse_attention_csr(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125, attn_plan=ap, out=out,
                               stages=stage)
    assert torch.equal(whole, out)
    again = K.sparse_attention_csr(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125, attn_plan=ap)
    assert torch.equal(whole, again)      # deterministic


def test_mask_values_rewritten_through_the_library_are_seen(oracle):
    """A mask-values tensor first seen as all ones, then overwritten in place by a library call
    (out= of another kernel writes through the raw pointer): the attention call must use the
    new values, not the remembered all-ones verdict."""
    from scorch_b200 import kernels as K
    dense, pos, crd, val = make_mask(256, 256, 24, 0.02, seed=11)
    rng = np.random.default_rng(12)
    Q, Km, V = (rng.standard_normal((256, 64)).astype(np.float32) * 0.3 for _ in range(3))
    dpos, dcrd = dev(pos), dev(crd)
    mv = torch.ones(len(crd), dtype=torch.float32, device="cuda")
    first = K.sparse_attention_csr(dpos, dcrd, mv, dev(Q), dev(Km), dev(V))
    ones = np.ones(len(crd), np.float32)
    ok, err, bad = oracle.allclose_report(first.cpu().numpy(),
                                          oracle_attention(oracle, pos, crd, ones, Q, Km, V, 1.0), RTOL, ATOL)
    assert ok, (err, bad)
    # new mask values = a scaled row softmax of some scores, written into the same tensor
    K.csr_row_softmax(dpos, dev(val), scale=0.5, out=mv)
    newval = mv.cpu().numpy()
    assert not np.allclose(newval, 1.0)
    second = K.sparse_attention_csr(dpos, dcrd, mv, dev(Q), dev(Km), dev(V))
    ok, err, bad = oracle.allclose_report(second.cpu().numpy(),
                                          oracle_attention(oracle, pos, crd, newval, Q, Km, V, 1.0), RTOL, ATOL)
    assert ok, (err, bad)


def test_pipeline_picks_the_attention_call_and_matches_three_operators(oracle):
    from scorch_b200 import pipelines as P, workloads as W
    mask = W.attention_mask(1024, window=64, density=0.01, seed=0)
    Q, Km, V = W.attention_qkv(1, 3, 1024, 64, seed=1)
    pos, crd, mv = dev(mask.pos), dev(mask.crd), dev(mask.val)
    from scorch_b200 import kernels as K
    ap = P.attention_plan(pos, crd, 64, 64)
    assert isinstance(ap, K.AttnPlan) and ap.block_fraction > 0.8     # +-64 fills a third of a 384-column window
    wide = W.attention_mask(1024, window=128, density=0.01, seed=0)
    bp = P.attention_plan(dev(wide.pos), dev(wide.crd), 64, 64)        # +-128 fills two thirds: the tcgen05 path
    assert isinstance(bp, K.AttnBandPlan) and bp.inside_fraction > 0.9 and bp.window_fill > 0.5
    assert isinstance(P.attention_plan(dev(wide.pos), dev(wide.crd), 32, 32), K.AttnPlan)
    assert P.attention_plan(pos, crd, 128, 128) is None and P.attention_plan(pos, crd, 64, 32) is None
    O = P.sparse_attention(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125)
    O3 = P.sparse_attention(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125, fused=False)
    torch.testing.assert_close(O, O3, rtol=2 * RTOL, atol=2 * ATOL)
    p, c, m = mask.pos.numpy(), mask.crd.numpy(), mask.val.numpy()
    for u in range(3):
        want = oracle_attention(oracle, p, c, m, Q[u].numpy(), Km[u].numpy(), V[u].numpy(), 0.125)
        ok, err, bad = oracle.allclose_report(O[u].cpu().numpy(), want, RTOL, ATOL)
        assert ok, (u, err, bad)
    # the scores are only available from the three-operator path
    scores = []
    P.sparse_attention(pos, crd, mv, dev(Q), dev(Km), dev(V), scale=0.125, scores_out=scores)
    assert len(scores) == 1 and scores[0].shape == (3, mask.nnz)
    # a random mask has no blocks: three operators
    rnd = W.csr_uniform(512, 512, 0.05, seed=3)
    assert P.attention_plan(dev(rnd.pos), dev(rnd.crd), 64, 64) is None
    # host-tensor front end
    host = P.HostSparseAttention(pos, crd, mv, 3, 1024, 64, chunks=2, scale=0.125)
    assert host.attn_plan is not None
    out_h = host(Q.pin_memory(), Km.pin_memory(), V.pin_memory())
    torch.testing.assert_close(out_h, O.cpu(), rtol=0, atol=0)


def test_sparse_attention_rejects_bad_arguments():
    from scorch_b200 import kernels as K
    dense, pos, crd, mval = make_mask(64, 64, 20, 0.0, seed=1)
    ap = K.AttnPlan(dev(pos), dev(crd))
    x = torch.zeros((64, 64), device="cuda")
    with pytest.raises(ValueError):
        K.sparse_attention_csr(dev(pos), dev(crd), None, x[:, :16].contiguous(), x[:, :16].contiguous(),
                               x[:, :16].contiguous(), attn_plan=ap)
    other = K.AttnPlan(dev(pos[:33]), dev(crd[: pos[32]]), n=64)
    with pytest.raises(ValueError):
        K.sparse_attention_csr(dev(pos), dev(crd), None, x, x, x, attn_plan=other)
    with pytest.raises(Exception) as e:
        K.sparse_attention_csr(dev(pos), dev(crd), None, x, x, x, attn_plan=ap, stages=0)
    assert "stage" in str(e.value)


def test_sparse_attention_without_scattered_entries(oracle):
    """A block-diagonal mask: every entry lies in a fully stored block, nothing is left for the
    gather kernels (rem_nnz == 0, the scratch holds the flags only)."""
    from scorch_b200 import kernels as K
    rows = 192
    dense = np.zeros((rows, rows), dtype=bool)
    for b in range(0, rows, 32):
        dense[b:b + 32, b:b + 32] = True
    pos = np.concatenate([[0], np.cumsum(dense.sum(1))]).astype(np.int32)
    crd = np.nonzero(dense)[1].astype(np.int32)
    rng = np.random.default_rng(0)
    mval = rng.uniform(0.5, 1.5, len(crd)).astype(np.float32)
    Q, Km, V = (rng.standard_normal((2, rows, 32)).astype(np.float32) for _ in range(3))
    ap = K.AttnPlan(dev(pos), dev(crd))
    assert ap.rem_nnz == 0 and ap.blocks == 6 * 4
    got = K.sparse_attention_csr(dev(pos), dev(crd), dev(mval), dev(Q), dev(Km), dev(V), scale=0.2, attn_plan=ap)
    for u in range(2):
        want = oracle_attention(oracle, pos, crd, mval, Q[u], Km[u], V[u], 0.2)
        ok, err, bad = oracle.allclose_report(got[u].cpu().numpy(), want, RTOL, ATOL)
        assert ok, (u, err, bad)


def test_sparse_attention_wide_rows_fall_back_to_the_gather_kernels(oracle):
    """Row blocks that touch more column blocks than the plan's counting table holds keep no
    blocks: their (long) rows go through the gather kernels, chunk after chunk."""
    from scorch_b200 import kernels as K
    rows, cols, d = 48, 20000, 64
    rng = np.random.default_rng(3)
    dense = rng.random((rows, cols)) < 0.06          # ~1200 entries per row, all 1250 column blocks touched
    dense[:, :64] = True                             # plus a dense stripe that would qualify as blocks
    pos = np.concatenate([[0], np.cumsum(dense.sum(1))]).astype(np.int32)
    crd = np.nonzero(dense)[1].astype(np.int32)
    Q = (rng.standard_normal((rows, d)) * 0.5).astype(np.float32)
    Km = (rng.standard_normal((cols, d)) * 0.5).astype(np.float32)
    V = rng.standard_normal((cols, d)).astype(np.float32)
    ap = K.AttnPlan(dev(pos), dev(crd), n=cols)
    assert ap.blocks == 0 and ap.rem_nnz == len(crd)
    got = K.sparse_attention_csr(dev(pos), dev(crd), None, dev(Q), dev(Km), dev(V), scale=0.125, attn_plan=ap)
    want = oracle_attention(oracle, pos, crd, None, Q, Km, V, 0.125)
    ok, err, bad = oracle.allclose_report(got.cpu().numpy(), want, RTOL, ATOL)
    assert ok, (err, bad)
