"""Randomised small cases (hypothesis) of the four kernels against the oracle: shapes, row-length
patterns and column widths are drawn, including empty matrices, empty rows and rows that hold
every column.  Each case also runs twice and must give identical bits (a scheduling-dependent
result would show up as a difference between the runs)."""
from __future__ import annotations

import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5
SETTINGS = dict(max_examples=40, deadline=None, derandomize=True,
                suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@st.composite
def csr_matrices(draw, max_rows=60, max_cols=70):
    m = draw(st.integers(0, max_rows))
    n = draw(st.integers(1, max_cols))
    seed = draw(st.integers(0, 2**31 - 1))
    kind = draw(st.sampled_from(["sparse", "mixed", "full_rows"]))
    rng = np.random.default_rng(seed)
    if kind == "sparse":
        lens = rng.integers(0, min(n, 4) + 1, size=m)
    elif kind == "mixed":
        lens = rng.integers(0, n + 1, size=m)
    else:
        lens = np.where(rng.random(m) < 0.3, n, rng.integers(0, 3, size=m))
    lens = np.minimum(lens, n)
    pos = np.zeros(m + 1, np.int64)
    np.cumsum(lens, out=pos[1:])
    crd = np.empty(pos[-1], np.int32)
    for i in range(m):
        if lens[i]:
            crd[pos[i]:pos[i + 1]] = np.sort(rng.choice(n, size=lens[i], replace=False))
    val = rng.standard_normal(pos[-1]).astype(np.float32)
    return m, n, pos.astype(np.int32), crd, val, rng


@settings(**SETTINGS)
@given(csr_matrices(), st.sampled_from([1, 3, 4, 8, 20, 32, 64, 65, 256, 260]), st.booleans(), st.booleans())
def test_spmm_random(oracle, A, k, with_bias, relu):
    from scorch_b200 import kernels as K
    m, n, pos, crd, val, rng = A
    B = rng.standard_normal((n, k)).astype(np.float32)
    bias = rng.standard_normal(k).astype(np.float32) if with_bias else None
    args = (dev(pos), dev(crd), dev(val), dev(B))
    got = K.spmm_csr(*args, bias=None if bias is None else dev(bias), relu=relu)
    want = oracle.spmm_csr_acc64(pos, crd, val, B, bias, relu)
    ok, err, bad = oracle.allclose_report(got.cpu().numpy(), want, RTOL, ATOL * max(1, n // 8))
    assert ok, (m, n, k, err, bad)
    assert torch.equal(got, K.spmm_csr(*args, bias=None if bias is None else dev(bias), relu=relu))


@settings(**SETTINGS)
@given(csr_matrices())
def test_spmv_random(oracle, A):
    from scorch_b200 import kernels as K
    m, n, pos, crd, val, rng = A
    x = rng.standard_normal(n).astype(np.float32)
    got = K.spmv_csr(dev(pos), dev(crd), dev(val), dev(x))
    ok, err, bad = oracle.allclose_report(got.cpu().numpy(), oracle.spmv_csr_acc64(pos, crd, val, x), RTOL,
                                          ATOL * max(1, n // 8))
    assert ok, (m, n, err, bad)
    assert torch.equal(got, K.spmv_csr(dev(pos), dev(crd), dev(val), dev(x)))


@settings(**SETTINGS)
@given(csr_matrices(), st.sampled_from([1, 4, 7, 16, 64, 100]))
def test_sddmm_and_softmax_random(oracle, A, d):
    from scorch_b200 import kernels as K
    m, n, pos, crd, val, rng = A
    Q = rng.standard_normal((m, d)).astype(np.float32)
    Kt = rng.standard_normal((n, d)).astype(np.float32)
    got, row, col = K.sddmm_csr(dev(pos), dev(crd), dev(val), dev(Q), dev(Kt), want_coords=True)
    want = oracle.sddmm_csr_acc64(pos, crd, val, Q, Kt)
    ok, err, bad = oracle.allclose_report(got.cpu().numpy(), want, RTOL, ATOL * max(1, d // 8))
    assert ok, (m, n, d, err, bad)
    assert np.array_equal(col.cpu().numpy(), crd)
    assert np.array_equal(row.cpu().numpy(), np.repeat(np.arange(m, dtype=np.int32), np.diff(pos)))
    sm = K.csr_row_softmax(dev(pos), got)
    ok, err, bad = oracle.allclose_report(sm.cpu().numpy(),
                                          oracle.csr_row_softmax_acc64(pos, got.cpu().numpy().astype(np.float64)),
                                          RTOL, ATOL)
    assert ok, (m, n, d, err, bad)


@settings(**SETTINGS)
@given(csr_matrices(max_rows=40, max_cols=40), st.integers(0, 2**31 - 1))
def test_spgemm_and_elementwise_random(oracle, A, seed_b):
    from scorch_b200 import kernels as K
    m, n, pos, crd, val, rng = A
    rb = np.random.default_rng(seed_b)
    cols = int(rb.integers(1, 50))
    lens = np.minimum(rb.integers(0, 6, size=n), cols)
    bpos = np.zeros(n + 1, np.int64)
    np.cumsum(lens, out=bpos[1:])
    bcrd = np.concatenate([np.sort(rb.choice(cols, size=l, replace=False)) for l in lens] + [np.zeros(0, np.int64)]
                          ).astype(np.int32)
    bval = rb.standard_normal(bpos[-1]).astype(np.float32)
    bpos = bpos.astype(np.int32)
    cpos, ccrd, cval = K.spgemm_csr(dev(pos), dev(crd), dev(val), dev(bpos), dev(bcrd), dev(bval), cols)
    wpos, wcrd, _ = oracle.spgemm(pos, crd, val, bpos, bcrd, bval, cols)
    assert np.array_equal(cpos.cpu().numpy(), wpos) and np.array_equal(ccrd.cpu().numpy(), wcrd)
    want = oracle.spgemm_values_acc64(pos, crd, val, bpos, bcrd, bval, cols, wpos, wcrd)
    ok, err, bad = oracle.allclose_report(cval.cpu().numpy(), want, RTOL, ATOL * 4)
    assert ok, (m, n, cols, err, bad)
    # element-wise ops of A with a second matrix of A's shape
    lens2 = np.minimum(rb.integers(0, 5, size=m), n)
    p2 = np.zeros(m + 1, np.int64)
    np.cumsum(lens2, out=p2[1:])
    c2 = np.concatenate([np.sort(rb.choice(n, size=l, replace=False)) for l in lens2] + [np.zeros(0, np.int64)]
                        ).astype(np.int32)
    v2 = rb.standard_normal(p2[-1]).astype(np.float32)
    p2 = p2.astype(np.int32)
    for op in ("mul", "add"):
        gp, gc, gv = K.csr_ewise(op, dev(pos), dev(crd), dev(val), dev(p2), dev(c2), dev(v2))
        wp, wc, wv = oracle.csr_ewise(op, pos, crd, val, p2, c2, v2)
        assert np.array_equal(gp.cpu().numpy(), wp) and np.array_equal(gc.cpu().numpy(), wc)
        assert np.array_equal(gv.cpu().numpy(), wv)


@settings(**dict(SETTINGS, max_examples=25))
@given(csr_matrices(max_rows=300, max_cols=500), st.sampled_from([32, 64]), st.booleans(), st.booleans())
def test_one_call_attention_random(oracle, A, d, band, pattern_only):
    """Both tensor-core paths of the one-call attention on arbitrary masks (any mask is valid for
    either plan: what does not fit the blocks / windows goes through the scattered-entry kernel)."""
    from scorch_b200 import kernels as K
    m, n, pos, crd, val, rng = A
    if band and d != 64:
        d = 64
    mval = np.ones_like(val) if pattern_only else (np.abs(val) + 0.5).astype(np.float32)
    Q = (rng.standard_normal((2, m, d)) * 0.5).astype(np.float32)
    Km = (rng.standard_normal((2, n, d)) * 0.5).astype(np.float32)
    V = rng.standard_normal((2, n, d)).astype(np.float32)
    p, c = dev(pos), dev(crd)
    plan = K.AttnBandPlan(p, c, n=n) if band else K.AttnPlan(p, c, n=n)
    got = K.sparse_attention_csr(p, c, dev(mval), dev(Q), dev(Km), dev(V), scale=0.2, attn_plan=plan)
    if band:
        assert K.attn_band_status() == 0
    for u in range(2):
        s64 = oracle.sddmm_csr_acc64(pos, crd, mval, Q[u], Km[u]) * 0.2
        p64 = oracle.csr_row_softmax_acc64(pos, s64)
        want = oracle.spmm_csr_acc64(pos, crd, p64.astype(np.float32), V[u])
        ok, err, bad = oracle.allclose_report(got[u].cpu().numpy(), want, RTOL, ATOL)
        assert ok, (m, n, d, band, err, bad)
    assert torch.equal(got, K.sparse_attention_csr(p, c, dev(mval), dev(Q), dev(Km), dev(V), scale=0.2,
                                                   attn_plan=plan))
