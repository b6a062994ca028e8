"""The five benchmark configurations at their FULL sizes.  The CPU oracle cannot redo a whole
2M-row product in seconds, so these tests combine (1) the oracle on a random sample of output
rows / heads, recomputed from the full operands, with (2) size-independent properties: linearity,
row sums, softmax rows summing to one, strictly ascending SpGEMM columns, agreement between the
dense-block and the gather path, bitwise repeatability."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def sample_rows_csr(pos, crd, val, rows):
    """CSR of the listed rows (host numpy) cut out of device CSR arrays."""
    pos_h = pos.cpu().numpy().astype(np.int64)
    lens = pos_h[rows + 1] - pos_h[rows]
    spos = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    idx = np.concatenate([np.arange(pos_h[r], pos_h[r + 1]) for r in rows]) if len(rows) else np.zeros(0, np.int64)
    idx_t = torch.from_numpy(idx).to(crd.device)
    return spos, crd[idx_t].cpu().numpy(), val[idx_t].cpu().numpy()


def check(oracle, got, want, what):
    ok, err, bad = oracle.allclose_report(got, want, RTOL, ATOL)
    assert ok, f"{what}: max abs err {err:.3e}, {bad} outside tolerance"


def test_c2_full_sparse_attention(oracle):
    from scorch_b200 import kernels as K, pipelines as P, workloads as W
    mask = W.attention_mask(4096, 128, 0.01, seed=0)
    Q, Km, V = (t.cuda() for t in W.attention_qkv(4, 8, 4096, 64, seed=1))
    pos, crd, mv = mask.pos.cuda(), mask.crd.cuda(), mask.val.cuda()
    bp = P.attention_block_plan(pos, crd)
    assert bp is not None and bp.blocks * 256 + bp.rem_nnz == mask.nnz
    scores = []
    O = P.sparse_attention(pos, crd, mv, Q, Km, V, scale=0.125, scores_out=scores, block_plan=bp)
    O_gather = P.sparse_attention(pos, crd, mv, Q, Km, V, scale=0.125, block_plan=None)
    torch.testing.assert_close(O, O_gather, rtol=RTOL, atol=ATOL)     # block path == gather path
    assert torch.equal(O, P.sparse_attention(pos, crd, mv, Q, Km, V, scale=0.125, block_plan=bp))
    p = scores[0]
    rows = torch.repeat_interleave(torch.arange(4096, device="cuda"), (pos[1:] - pos[:-1]).long())
    sums = torch.zeros((32, 4096), device="cuda", dtype=torch.float64).index_add_(1, rows, p.double())
    assert (sums - 1).abs().max().item() < 1e-5                         # softmax rows sum to one
    # SDDMM is linear in Q
    s1 = K.sddmm_csr(pos, crd, mv, Q, Km, block_plan=bp)
    s2 = K.sddmm_csr(pos, crd, mv, 2 * Q, Km, block_plan=bp)
    torch.testing.assert_close(s2, 2 * s1, rtol=1e-5, atol=1e-6)
    pn, cn, mn = mask.pos.numpy(), mask.crd.numpy(), mask.val.numpy()
    for u in (0, 13, 31):                                               # three heads against the oracle
        s64 = oracle.sddmm_csr_acc64(pn, cn, mn, Q[u].cpu().numpy(), Km[u].cpu().numpy())
        check(oracle, s1[u].cpu().numpy(), s64, f"scores head {u}")
        p64 = oracle.csr_row_softmax_acc64(pn, s64 * 0.125)
        check(oracle, p[u].cpu().numpy(), p64, f"probabilities head {u}")
        check(oracle, O[u].cpu().numpy(), oracle.spmm_csr_acc64(pn, cn, p64.astype(np.float32), V[u].cpu().numpy()),
              f"attention output head {u}")


def test_c2_full_one_call_attention_both_tensor_core_paths(oracle):
    """Configuration 2 at full size through the single attention call: the plan the pipeline picks
    (128-row tiles on tcgen05) and the 16x16-block plan agree with each other, rows of the output
    are convex combinations of V rows (linearity in V), and three heads match the oracle."""
    from scorch_b200 import kernels as K, pipelines as P, workloads as W
    mask = W.attention_mask(4096, 128, 0.01, seed=0)
    Q, Km, V = (t.cuda() for t in W.attention_qkv(4, 8, 4096, 64, seed=1))
    pos, crd, mv = mask.pos.cuda(), mask.crd.cuda(), mask.val.cuda()
    plan = P.attention_plan(pos, crd, 64, 64)
    assert isinstance(plan, K.AttnBandPlan) and plan.inside + plan.rem_nnz == mask.nnz
    O = K.sparse_attention_csr(pos, crd, mv, Q, Km, V, scale=0.125, attn_plan=plan)
    assert K.attn_band_status() == 0
    O_blocks = K.sparse_attention_csr(pos, crd, mv, Q, Km, V, scale=0.125, attn_plan=K.attn_plan_for(pos, crd))
    torch.testing.assert_close(O, O_blocks, rtol=RTOL, atol=ATOL)
    assert torch.equal(O, K.sparse_attention_csr(pos, crd, mv, Q, Km, V, scale=0.125, attn_plan=plan))
    O2 = K.sparse_attention_csr(pos, crd, mv, Q, Km, 2 * V + 1, scale=0.125, attn_plan=plan)
    torch.testing.assert_close(O2, 2 * O + 1, rtol=RTOL, atol=2 * ATOL)      # softmax rows sum to one
    pn, cn, mn = mask.pos.numpy(), mask.crd.numpy(), mask.val.numpy()
    for u in (0, 13, 31):
        s64 = oracle.sddmm_csr_acc64(pn, cn, mn, Q[u].cpu().numpy(), Km[u].cpu().numpy()) * 0.125
        p64 = oracle.csr_row_softmax_acc64(pn, s64)
        check(oracle, O[u].cpu().numpy(), oracle.spmm_csr_acc64(pn, cn, p64.astype(np.float32), V[u].cpu().numpy()),
              f"one-call attention output head {u}")


def test_c3_full_sae_decode(oracle):
    from scorch_b200 import kernels as K, workloads as W
    A = W.sae_activations(8192, 32768, 32, seed=0, device="cuda")
    Wd = W.sae_decoder(32768, 4096, seed=1, device="cuda")
    assert A.nnz == 8192 * 32
    Y = K.spmm_csr(A.pos, A.crd, A.val, Wd)
    assert torch.equal(Y, K.spmm_csr(A.pos, A.crd, A.val, Wd))
    rows = np.sort(np.random.default_rng(0).choice(8192, 64, replace=False))
    spos, scrd, sval = sample_rows_csr(A.pos, A.crd, A.val, rows)
    check(oracle, Y[torch.from_numpy(rows).cuda()].cpu().numpy(),
          oracle.spmm_csr_acc64(spos, scrd, sval, Wd.cpu().numpy()), "sampled rows")
    # linear in the dense operand
    torch.testing.assert_close(K.spmm_csr(A.pos, A.crd, A.val, -3 * Wd), -3 * Y, rtol=1e-5, atol=1e-6)


def test_c4_full_gcn_graph_spmm(oracle):
    from scorch_b200 import kernels as K, workloads as W
    n = 2_000_000
    g = W.gcn_graph(n, seed=0, device="cuda")
    lens = (g.pos[1:] - g.pos[:-1])
    assert int(lens.max()) > 40_000 and 1.9e8 < g.nnz < 2.1e8
    plan = K.CsrPlan(g.pos, g.nnz)
    assert plan.heavy_rows > 1000 and plan.segments > plan.heavy_rows
    # A @ ones = row sums of A (fp64 segment sums computed independently with torch)
    ones = torch.ones((n, 64), device="cuda")
    Y1 = K.spmm_csr(g.pos, g.crd, g.val, ones, plan=plan)
    csum = torch.cumsum(g.val.double(), 0)
    csum = torch.cat([torch.zeros(1, device="cuda", dtype=torch.float64), csum])
    rowsum = csum[g.pos[1:].long()] - csum[g.pos[:-1].long()]
    assert (Y1[:, 0].double() - rowsum).abs().max().item() < 1e-4
    assert (Y1 == Y1[:, :1]).all()
    # sampled rows (the heaviest rows included) against the oracle, with the fused ReLU epilogue
    X = W.randn_on((n, 64), seed=1, device="cuda")
    Y = K.spmm_csr(g.pos, g.crd, g.val, X, relu=True, plan=plan)
    heavy = torch.topk(lens, 4).indices.cpu().numpy()
    rows = np.unique(np.concatenate([heavy, np.random.default_rng(1).choice(n, 200, replace=False)]))
    spos, scrd, sval = sample_rows_csr(g.pos, g.crd, g.val, rows)
    check(oracle, Y[torch.from_numpy(rows).cuda()].cpu().numpy(),
          oracle.spmm_csr_acc64(spos, scrd, sval, X.cpu().numpy(), None, True), "sampled rows")
    assert torch.equal(Y, K.spmm_csr(g.pos, g.crd, g.val, X, relu=True, plan=plan))


def test_c5_full_spgemm_and_spmv(oracle):
    from scorch_b200 import kernels as K, workloads as W
    n = 2_000_000
    A = W.powerlaw_square(n, seed=0, device="cuda")
    x = W.randn_on((n,), seed=1, device="cuda")
    # SpMV against independent fp64 segment sums
    y = K.spmv_csr(A.pos, A.crd, A.val, x)
    prod = A.val.double() * x[A.crd.long()].double()
    csum = torch.cat([torch.zeros(1, device="cuda", dtype=torch.float64), torch.cumsum(prod, 0)])
    y64 = csum[A.pos[1:].long()] - csum[A.pos[:-1].long()]
    absum = torch.cat([torch.zeros(1, device="cuda", dtype=torch.float64), torch.cumsum(prod.abs(), 0)])
    scale = absum[A.pos[1:].long()] - absum[A.pos[:-1].long()]
    # fp64 prefix differences carry ~1e-16 * total of rounding: compare against the row's magnitude
    assert ((y.double() - y64).abs() <= 1e-5 + 1e-4 * y64.abs() + 1e-6 * scale).all()
    assert torch.equal(y, K.spmv_csr(A.pos, A.crd, A.val, x))
    # SpGEMM structure properties at full size
    t = {}
    Cpos, Ccrd, Cval = K.spgemm_csr(A.pos, A.crd, A.val, A.pos, A.crd, A.val, n, timings=t)
    assert Cpos.dtype == torch.int32 and Ccrd.dtype == torch.int32
    assert int(Cpos[0]) == 0 and int(Cpos[-1]) == Ccrd.numel() and 2.5e8 < Ccrd.numel() < 2.9e8
    assert (Cpos[1:] >= Cpos[:-1]).all() and int(Ccrd.min()) >= 0 and int(Ccrd.max()) < n
    rows_of = torch.repeat_interleave(torch.arange(n, device="cuda"), (Cpos[1:] - Cpos[:-1]).long())
    key = rows_of * n + Ccrd.long()
    assert (key[1:] > key[:-1]).all()                  # columns strictly ascending within every row
    del key, rows_of
    # sampled rows (the longest rows of A and of C included): structure bit-exact, values in tolerance
    lensA = A.pos[1:] - A.pos[:-1]
    lensC = Cpos[1:] - Cpos[:-1]
    rows = np.unique(np.concatenate([torch.topk(lensA, 2).indices.cpu().numpy(),
                                     torch.topk(lensC, 2).indices.cpu().numpy(),
                                     np.random.default_rng(2).choice(n, 3000, replace=False)]))
    spos, scrd, sval = sample_rows_csr(A.pos, A.crd, A.val, rows)
    Bp, Bc, Bv = A.pos.cpu().numpy(), A.crd.cpu().numpy(), A.val.cpu().numpy()
    wpos, wcrd, _ = oracle.spgemm(spos, scrd, sval, Bp, Bc, Bv, n)
    gpos, gcrd, gval = sample_rows_csr(Cpos, Ccrd, Cval, rows)
    assert np.array_equal(gpos, wpos) and np.array_equal(gcrd, wcrd)
    check(oracle, gval, oracle.spgemm_values_acc64(spos, scrd, sval, Bp, Bc, Bv, n, wpos, wcrd), "sampled C rows")
    assert t["symbolic_ms"] > 0 and t["numeric_ms"] > 0
