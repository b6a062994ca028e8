"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle and the golden
vectors produced by the reference.  Tolerance for floating-point values: rtol 1e-4 / atol 1e-5
against a float64-accumulating oracle; integer results and all index structures are bit-exact.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def assert_close(oracle, got, want64, what=""):
    ok, err, bad = oracle.allclose_report(got.detach().cpu().numpy() if torch.is_tensor(got) else got,
                                          want64, RTOL, ATOL)
    assert ok, f"{what}: max abs err {err:.3e}, {bad} elements outside rtol {RTOL} / atol {ATOL}"


def random_csr(m, n, row_lens, seed, dtype=np.float32):
    """CSR with the given row lengths, columns uniform without replacement."""
    rng = np.random.default_rng(seed)
    row_lens = np.minimum(np.asarray(row_lens, np.int64), n)
    pos = np.zeros(m + 1, np.int64)
    np.cumsum(row_lens, out=pos[1:])
    crd = np.empty(pos[-1], np.int32)
    for i in range(m):
        if row_lens[i]:
            crd[pos[i]:pos[i + 1]] = np.sort(rng.choice(n, size=row_lens[i], replace=False))
    if np.dtype(dtype).kind == "i":
        val = rng.integers(-9, 10, size=pos[-1]).astype(dtype)
    else:
        val = rng.standard_normal(pos[-1]).astype(dtype)
    return pos.astype(np.int32), crd, val


# ================================ SpMM ==========================================================
@pytest.mark.parametrize("case", ["spmm_f32", "spmm_f32_k300", "spmm_f64", "spmm_i32", "spmm_i64"])
def test_spmm_golden_through_reference_symbols(golden, case):
    """Host tensors in, host tensor out, through the drop-in symbol the registry resolves."""
    from scorch_b200 import scorch_ops
    g = golden.case(case)
    m, n, k = len(g["pos"]) - 1, g["B"].shape[0], g["B"].shape[1]
    sym = {"spmm_f32": "spmm_csr_float_v2", "spmm_f32_k300": "spmm_csr_float_v2",
           "spmm_f64": "prebuilt_spmm_csr_f64", "spmm_i32": "prebuilt_spmm_csr_i32",
           "spmm_i64": "prebuilt_spmm_csr_i64"}[case]
    r = getattr(scorch_ops, sym)([m, k], [m, n], [[], [torch.from_numpy(g["pos"]), torch.from_numpy(g["crd"])]],
                                 torch.from_numpy(g["val"]), [n, k], [[], []],
                                 torch.from_numpy(g["B"]).flatten())
    got = r.storage.value
    assert not got.is_cuda and got.shape == (m * k,) and r.storage.index.mode_indices == [[], []]
    got = got.view(m, k).numpy()
    if got.dtype.kind == "i":
        assert np.array_equal(got, g["C"])
    else:
        np.testing.assert_allclose(got, g["C"], rtol=RTOL, atol=ATOL)
    empty = np.diff(g["pos"]) == 0
    assert (got[empty] == 0).all()


@pytest.mark.parametrize("relu", [0, 1])
def test_spmm_bias_golden(golden, relu):
    from scorch_b200 import scorch_ops
    g = golden.case(f"spmm_bias_relu{relu}")
    m, n, k = len(g["pos"]) - 1, g["B"].shape[0], g["B"].shape[1]
    fn = scorch_ops.spmm_csr_bias_relu_float if relu else scorch_ops.spmm_csr_bias_float
    r = fn([m, k], [m, n], [[], [torch.from_numpy(g["pos"]), torch.from_numpy(g["crd"])]],
           torch.from_numpy(g["val"]), [n, k], [[], []], torch.from_numpy(g["B"]).flatten(),
           torch.from_numpy(g["bias"]))
    got = r.storage.value.view(m, k).numpy()
    np.testing.assert_allclose(got, g["C"], rtol=RTOL, atol=ATOL)
    empty = np.diff(g["pos"]) == 0  # every row starts from the bias (csrc/spmm.h:56-58)
    want = np.maximum(g["bias"], 0) if relu else g["bias"]
    assert np.array_equal(got[empty], np.broadcast_to(want, got[empty].shape))


@pytest.mark.parametrize("k", [4, 7, 16, 20, 33, 64, 100, 128, 256, 300, 512, 1000])
def test_spmm_vs_oracle_all_column_widths(oracle, k):
    from scorch_b200 import kernels as K
    rng = np.random.default_rng(k)
    m, n = 257, 193
    lens = rng.integers(0, 70, size=m)
    lens[[0, 5, 256]] = 0
    pos, crd, val = random_csr(m, n, lens, seed=k)
    B = rng.standard_normal((n, k)).astype(np.float32)
    got = K.spmm_csr(dev(pos), dev(crd), dev(val), dev(B))
    assert_close(oracle, got, oracle.spmm_csr_acc64(pos, crd, val, B), f"k={k}")
    bias = rng.standard_normal(k).astype(np.float32)
    got = K.spmm_csr(dev(pos), dev(crd), dev(val), dev(B), bias=dev(bias), relu=True)
    assert_close(oracle, got, oracle.spmm_csr_acc64(pos, crd, val, B, bias, True), f"k={k} bias+relu")


@pytest.mark.parametrize("k", [8, 16, 20, 32, 64, 72, 128, 256, 300])
def test_spmm_many_short_rows(oracle, k):
    """Mean row length below the short-row threshold: a row per lane group (narrow tiles) or
    several rows per warp; rows too long for a lane group, empty rows and heavy rows mixed in,
    plain and accumulating, with and without the heavy-row plan."""
    from scorch_b200 import kernels as K
    from scorch_b200._lib import HEAVY_ROW_NNZ as T
    rng = np.random.default_rng(100 + k)
    m, n = 1003, 4000
    lens = rng.poisson(9, size=m)
    lens[rng.integers(0, m, 25)] = 0
    lens[[3, 40, 41, 500, 1002]] = [65, 300, 64, 1024, 97]
    lens[[7, 600]] = [T + 9, 2 * T + 100]
    pos, crd, val = random_csr(m, n, lens, seed=200 + k)
    assert len(crd) < 24 * m            # below the short-row threshold for every width
    val = (val / np.sqrt(np.repeat(np.maximum(lens, 1), lens))).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    bias = rng.standard_normal(k).astype(np.float32)
    C0 = rng.standard_normal((m, k)).astype(np.float32)
    dpos, dcrd, dval, dB = dev(pos), dev(crd), dev(val), dev(B)
    want = oracle.spmm_csr_acc64(pos, crd, val, B)
    plan = K.CsrPlan(dpos, len(crd))
    assert plan.segments == 2 + 3
    got = K.spmm_csr(dpos, dcrd, dval, dB, plan=plan)
    assert_close(oracle, got, want, f"short rows k={k}")
    assert torch.equal(got, K.spmm_csr(dpos, dcrd, dval, dB, plan=plan))
    got = K.spmm_csr(dpos, dcrd, dval, dB, bias=dev(bias), relu=True, plan=plan, out=dev(C0.copy()),
                     accumulate=k % 4 == 0)
    w2 = want + bias.astype(np.float64) + (C0.astype(np.float64) if k % 4 == 0 else 0)
    assert_close(oracle, got, np.maximum(w2, 0), f"short rows k={k} epilogue")


@pytest.mark.parametrize("k", [64, 256, 520])
def test_spmm_heavy_rows_and_plan(oracle, k):
    """Rows around and far above the heavy threshold go through the segment kernels."""
    from scorch_b200 import kernels as K
    from scorch_b200._lib import HEAVY_ROW_NNZ as T
    m, n = 40, 6000
    lens = np.full(m, 9)
    lens[[1, 7, 8, 20, 39]] = [T, T + 1, 2 * T, 5 * T + 17, 3 * T - 1]
    lens[3] = 0
    pos, crd, val = random_csr(m, n, lens, seed=11)
    # degree-normalised values (like D^-1/2 A D^-1/2) keep the long sums O(1), so that the
    # tolerance measures the kernel and not the conditioning of a 5000-term N(0,1) sum
    val = (val / np.sqrt(np.repeat(np.maximum(lens, 1), lens))).astype(np.float32)
    B = np.random.default_rng(12).standard_normal((n, k)).astype(np.float32)
    dpos = dev(pos)
    plan = K.CsrPlan(dpos, len(crd))
    assert plan.heavy_rows == 4 and plan.segments == 2 + 2 + 6 + 3
    bias = np.random.default_rng(13).standard_normal(k).astype(np.float32)
    got = K.spmm_csr(dpos, dev(crd), dev(val), dev(B), bias=dev(bias), relu=False, plan=plan)
    assert_close(oracle, got, oracle.spmm_csr_acc64(pos, crd, val, B, bias, False), "heavy rows")
    # bitwise reproducible: partial sums are combined in a fixed order
    again = K.spmm_csr(dpos, dev(crd), dev(val), dev(B), bias=dev(bias), relu=False, plan=plan)
    assert torch.equal(got, again)


@pytest.mark.parametrize("k", [64, 256])
def test_spmm_accumulating_form(oracle, k):
    """sb_spmm_csr_acc_f32: act(bias + C + A B) with short, empty and multi-segment heavy rows."""
    from scorch_b200 import kernels as K
    from scorch_b200._lib import HEAVY_ROW_NNZ as T
    m, n = 50, 5000
    lens = np.full(m, 11)
    lens[[2, 9, 30]] = [T + 5, 3 * T + 1, 0]
    pos, crd, val = random_csr(m, n, lens, seed=21)
    val = (val / np.sqrt(np.repeat(np.maximum(lens, 1), lens))).astype(np.float32)
    rng = np.random.default_rng(22)
    B = rng.standard_normal((n, k)).astype(np.float32)
    C0 = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(k).astype(np.float32)
    for relu in (False, True):
        out = dev(C0.copy())
        got = K.spmm_csr(dev(pos), dev(crd), dev(val), dev(B), bias=dev(bias), relu=relu, out=out,
                         accumulate=True)
        assert got.data_ptr() == out.data_ptr()
        want = oracle.spmm_csr_acc64(pos, crd, val, B) + C0.astype(np.float64) + bias.astype(np.float64)
        if relu:
            want = np.maximum(want, 0)
        assert_close(oracle, got, want, f"accumulate relu={relu}")
    with pytest.raises(ValueError):
        K.spmm_csr(dev(pos), dev(crd), dev(val), dev(B), accumulate=True)


def test_spmm_batched_shared_structure(oracle):
    from scorch_b200 import kernels as K
    rng = np.random.default_rng(5)
    m, n, k, batch = 130, 90, 64, 3
    pos, crd, _ = random_csr(m, n, rng.integers(0, 40, size=m), seed=6)
    vals = rng.standard_normal((batch, len(crd))).astype(np.float32)
    Bs = rng.standard_normal((batch, n, k)).astype(np.float32)
    got = K.spmm_csr(dev(pos), dev(crd), dev(vals), dev(Bs))
    assert got.shape == (batch, m, k)
    for b in range(batch):
        assert_close(oracle, got[b], oracle.spmm_csr_acc64(pos, crd, vals[b], Bs[b]), f"batch {b}")


def test_spmm_degenerate_shapes(oracle):
    from scorch_b200 import kernels as K
    pos = np.zeros(6, np.int32)
    out = K.spmm_csr(dev(pos), dev(np.zeros(0, np.int32)), dev(np.zeros(0, np.float32)),
                     dev(np.ones((4, 8), np.float32)))
    assert out.shape == (5, 8) and (out == 0).all()
    out = K.spmm_csr(dev(np.zeros(1, np.int32)), dev(np.zeros(0, np.int32)),
                     dev(np.zeros(0, np.float32)), dev(np.ones((4, 8), np.float32)))
    assert out.shape == (0, 8)


def test_c1_config_full_size(oracle):
    """BASELINE config 1: 4096x4096, 1 % uniform, k = 64, through scorch.matmul on host tensors."""
    import scorch_b200 as scorch
    from scorch_b200 import workloads as W
    A = W.csr_uniform(4096, 4096, 0.01, seed=0)
    B = W.dense_normal(4096, 64, seed=1)
    C = scorch.matmul(A.torch_csr(), B, format="dd")
    assert isinstance(C, torch.Tensor) and not C.is_cuda and C.shape == (4096, 64)
    assert_close(oracle, C, oracle.spmm_csr_acc64(A.pos.numpy(), A.crd.numpy(), A.val.numpy(), B.numpy()), "C1")
    # and against the fp32 restatement of the reference kernel
    ref32 = oracle.spmm_csr_v2(A.pos.numpy(), A.crd.numpy(), A.val.numpy(), B.numpy())
    np.testing.assert_allclose(C.numpy(), ref32, rtol=RTOL, atol=ATOL)


# ================================ SpMV ==========================================================
@pytest.mark.parametrize("case,sym", [("spmv_f32", "prebuilt_spmv_csr_f32"), ("spmv_f64", "prebuilt_spmv_csr_f64"),
                                      ("spmv_i32", "prebuilt_spmv_csr_i32"), ("spmv_i64", "prebuilt_spmv_csr_i64")])
def test_spmv_golden(golden, case, sym):
    from scorch_b200 import scorch_ops
    g = golden.case(case)
    m, n = len(g["pos"]) - 1, len(g["x"])
    r = getattr(scorch_ops, sym)([m], [m, n], [[], [torch.from_numpy(g["pos"]), torch.from_numpy(g["crd"])]],
                                 torch.from_numpy(g["val"]), [n], [[]], torch.from_numpy(g["x"]))
    got = r.storage.value.numpy()
    assert r.storage.index.mode_indices == [[]]
    if got.dtype.kind == "i":
        assert np.array_equal(got, g["y"])
    else:
        np.testing.assert_allclose(got, g["y"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("mean", [1, 4, 9, 30, 100])
def test_spmv_vs_oracle_group_widths_and_heavy_rows(oracle, mean):
    from scorch_b200 import kernels as K
    from scorch_b200._lib import HEAVY_ROW_NNZ as T
    rng = np.random.default_rng(mean)
    m, n = 3001, 9000
    lens = rng.poisson(mean, size=m)
    lens[[2, 1500, 3000]] = [T + 3, 4 * T, 0]
    pos, crd, val = random_csr(m, n, lens, seed=mean + 1)
    x = rng.standard_normal(n).astype(np.float32)
    got = K.spmv_csr(dev(pos), dev(crd), dev(val), dev(x))
    assert_close(oracle, got, oracle.spmv_csr_acc64(pos, crd, val, x), f"mean {mean}")
    assert torch.equal(got, K.spmv_csr(dev(pos), dev(crd), dev(val), dev(x)))


# ================================ SDDMM / softmax ================================================
def test_sddmm_golden_coo_and_csr(golden):
    import scorch_b200 as scorch
    from scorch_b200.stensor import STensor
    g = golden.case("sddmm_coo")
    m, n = g["Q"].shape[0], g["K"].shape[0]
    ind = torch.from_numpy(np.stack([g["row"], g["col"]]).astype(np.int64))
    S = STensor.from_coo(indices=ind, values=torch.from_numpy(g["mval"]), shape=(m, n))
    r = scorch.einsum("ij,ik,jk->ij", S, torch.from_numpy(g["Q"]), torch.from_numpy(g["K"]))
    assert str(r.format) == "o,o"
    np.testing.assert_allclose(r.values.numpy(), g["out_val"], rtol=RTOL, atol=ATOL)
    # the COO route shares the mask's coordinate tensors (csrc/kernels.h:567)
    assert r.index.mode_indices[0][0] is S.index.mode_indices[0][0]
    c = golden.case("sddmm_csr")
    Sc = STensor.from_csr_arrays((m, n), torch.from_numpy(c["pos"]), torch.from_numpy(c["crd"]),
                                 torch.from_numpy(c["mval"]))
    for expr, Kop in (("ij,ik,jk->ij", torch.from_numpy(c["K"])),
                      ("ij,ik,kj->ij", torch.from_numpy(c["K"]).t().contiguous())):
        r = scorch.einsum(expr, Sc, torch.from_numpy(c["Q"]), Kop)
        assert str(r.format) == "o,o"
        row, col = r.index.mode_indices[0][0], r.index.mode_indices[1][0]
        assert row.dtype == torch.int32 and col.dtype == torch.int32
        assert np.array_equal(row.numpy(), c["out_row"]) and np.array_equal(col.numpy(), c["out_col"])
        np.testing.assert_allclose(r.values.numpy(), c["out_val"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("d", [4, 7, 16, 20, 64, 100, 128, 256, 300, 512, 520])
def test_sddmm_vs_oracle_all_depths(oracle, d):
    from scorch_b200 import kernels as K
    rng = np.random.default_rng(d)
    m, n = 301, 211
    lens = rng.integers(0, 12, size=m)  # short rows: most 32-entry chunks cross several rows
    lens[[0, 17, 300]] = 0
    lens[40] = 150
    pos, crd, mval = random_csr(m, n, lens, seed=d)
    Q = rng.standard_normal((m, d)).astype(np.float32)
    Km = rng.standard_normal((n, d)).astype(np.float32)
    want = oracle.sddmm_csr_acc64(pos, crd, mval, Q, Km)
    out, row, col = K.sddmm_csr(dev(pos), dev(crd), dev(mval), dev(Q), dev(Km), want_coords=True)
    assert_close(oracle, out, want, f"d={d}")
    rows = np.repeat(np.arange(m, dtype=np.int32), np.diff(pos))
    assert np.array_equal(row.cpu().numpy(), rows) and np.array_equal(col.cpu().numpy(), crd)
    out2 = K.sddmm_coo(dev(rows), dev(crd), dev(mval), dev(Q), dev(Km))
    assert_close(oracle, out2, want, f"coo d={d}")
    out3 = K.sddmm_csr(dev(pos), dev(crd), None, dev(Q), dev(Km))  # implicit all-ones mask
    assert_close(oracle, out3, oracle.sddmm_csr_acc64(pos, crd, None, Q, Km), f"no mask d={d}")


def test_softmax_golden_and_edge_rows(oracle, golden):
    from scorch_b200 import kernels as K
    g = golden.case("softmax")
    got = K.csr_row_softmax(dev(g["pos"]), dev(g["val"]))
    np.testing.assert_allclose(got.cpu().numpy(), g["out"], rtol=RTOL, atol=ATOL)
    rng = np.random.default_rng(0)
    lens = np.array([0, 1, 31, 32, 33, 384, 385, 400, 5000, 0, 2])
    pos = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    val = (rng.standard_normal(pos[-1]) * 4).astype(np.float32)
    want = oracle.csr_row_softmax_acc64(pos, val.astype(np.float64) * 0.5)
    got = K.csr_row_softmax(dev(pos), dev(val), scale=0.5)
    assert_close(oracle, got, want, "softmax")
    inplace = dev(val)
    K.csr_row_softmax(dev(pos), inplace, scale=0.5, out=inplace)
    assert torch.equal(inplace, got)
    sums = np.add.reduceat(got.cpu().numpy().astype(np.float64), pos[:-1][lens > 0])
    np.testing.assert_allclose(sums, 1.0, atol=1e-5)


def test_c2_sparse_attention_reduced_and_batched(oracle):
    """BASELINE config 2 at seq 1024 (band 32 + 1 % random), 2x3 heads: whole pipeline vs fp64."""
    from scorch_b200 import kernels as K, pipelines as P, workloads as W
    mask = W.attention_mask(1024, window=32, density=0.01, seed=0)
    Q, Km, V = W.attention_qkv(2, 3, 1024, 64, seed=1)
    scores = []
    O = P.sparse_attention(dev(mask.pos), dev(mask.crd), dev(mask.val), dev(Q), dev(Km), dev(V),
                           scale=1.0, scores_out=scores)
    pos, crd, mv = mask.pos.numpy(), mask.crd.numpy(), mask.val.numpy()
    for u in range(6):
        s64 = oracle.sddmm_csr_acc64(pos, crd, mv, Q[u].numpy(), Km[u].numpy())
        p64 = oracle.csr_row_softmax_acc64(pos, s64)
        assert_close(oracle, scores[0][u], p64, f"probabilities unit {u}")
        o64 = oracle.spmm_csr_acc64(pos, crd, p64.astype(np.float32), V[u].numpy())
        assert_close(oracle, O[u], o64, f"attention output unit {u}")


def test_host_sparse_attention_pipeline_matches_device_path():
    """Pinned host operands, chunked copy/compute overlap: same numbers as the resident path."""
    from scorch_b200 import pipelines as P, workloads as W
    mask = W.attention_mask(512, window=16, density=0.02, seed=3)
    Q, Km, V = (t.pin_memory() for t in W.attention_qkv(1, 7, 512, 64, seed=4))
    pos, crd, mv = dev(mask.pos), dev(mask.crd), dev(mask.val)
    want = P.sparse_attention(pos, crd, mv, Q.cuda(), Km.cuda(), V.cuda(), scale=0.125).cpu()
    host = P.HostSparseAttention(pos, crd, mv, units=7, seq=512, d=64, chunks=3, scale=0.125)
    for _ in range(2):  # buffers and streams are reused from call to call
        got = host(Q, Km, V)
        assert not got.is_cuda and torch.equal(got, want)


def test_c3_sae_decode_reduced(oracle):
    from scorch_b200 import kernels as K, workloads as W
    A = W.sae_activations(512, 4096, 32, seed=0)
    Wd = W.sae_decoder(4096, 1024, seed=1)
    Y = K.spmm_csr(dev(A.pos), dev(A.crd), dev(A.val), dev(Wd))
    assert_close(oracle, Y, oracle.spmm_csr_acc64(A.pos.numpy(), A.crd.numpy(), A.val.numpy(), Wd.numpy()), "C3")


def test_c4_gcn_reduced(oracle):
    from scorch_b200 import pipelines as P, workloads as W
    g = W.gcn_graph(20000, mean_deg=30.0, max_deg=5000, seed=0)
    assert int((g.pos[1:] - g.pos[:-1]).max()) > 1024  # has heavy hub rows
    X = W.randn_on((20000, 256), seed=1)
    W1, W2 = W.glorot(256, 256, seed=0), W.glorot(256, 64, seed=1)
    out = P.gcn_forward(dev(g.pos), dev(g.crd), dev(g.val), dev(X), dev(W1), dev(W2))
    pos, crd, val = g.pos.numpy(), g.crd.numpy(), g.val.numpy()
    xw = X.double().numpy() @ W1.double().numpy()
    h = np.maximum(oracle.spmm_csr_acc64(pos, crd, val, xw.astype(np.float32)), 0)
    want = oracle.spmm_csr_acc64(pos, crd, val, (h @ W2.double().numpy()).astype(np.float32))
    ok, err, bad = oracle.allclose_report(out.cpu().numpy(), want, 2e-3, 1e-4)  # two chained layers
    assert ok, (err, bad)


# ================================ SpGEMM =========================================================
@pytest.mark.parametrize("case,sym", [("spgemm_f32", "prebuilt_spmspm_csr_f32"), ("spgemm_f64", "prebuilt_spmspm_csr_f64"),
                                      ("spgemm_i32", "prebuilt_spmspm_csr_i32"), ("spgemm_i64", "prebuilt_spmspm_csr_i64"),
                                      ("spgemm_cancel", "spmspm_csr_float")])
def test_spgemm_golden(golden, case, sym):
    from scorch_b200 import scorch_ops
    g = golden.case(case)
    m, kb, n = len(g["Apos"]) - 1, len(g["Bpos"]) - 1, int(g["n"][0])
    t = torch.from_numpy
    r = getattr(scorch_ops, sym)([m, n], [m, kb], [[], [t(g["Apos"]), t(g["Acrd"])]], t(g["Aval"]),
                                 [kb, n], [[], [t(g["Bpos"]), t(g["Bcrd"])]], t(g["Bval"]))
    cpos, ccrd = r.storage.index.mode_indices[1]
    assert cpos.dtype == torch.int32 and ccrd.dtype == torch.int32
    assert np.array_equal(cpos.numpy(), g["Cpos"]) and np.array_equal(ccrd.numpy(), g["Ccrd"])
    got = r.storage.value.numpy()
    if got.dtype.kind == "i":
        assert np.array_equal(got, g["Cval"])
    else:
        np.testing.assert_allclose(got, g["Cval"], rtol=RTOL, atol=ATOL)


def test_spgemm_all_bins_vs_oracle(oracle):
    """Power-law rows exercise every bin: warp hash (64/256), CTA hash (2048/16384), dense rows."""
    from scorch_b200 import kernels as K, workloads as W
    A = W.powerlaw_square(60000, mean_nnz=12.0, seed=3)
    pos, crd, val = A.pos.numpy(), A.crd.numpy(), A.val.numpy()
    lens = np.diff(pos)
    upper = np.add.reduceat(lens[crd], pos[:-1])  # every row has >= 1 entry
    for lo, hi in ((1, 32), (33, 128), (129, 512), (513, 2048), (2049, 8192), (8193, 1 << 30)):
        assert ((upper >= lo) & (upper <= hi)).any(), f"no row with upper bound in [{lo},{hi}]"
    cpos, ccrd, cval = K.spgemm_csr(dev(pos), dev(crd), dev(val), dev(pos), dev(crd), dev(val), 60000)
    wpos, wcrd, _ = oracle.spgemm(pos, crd, val, pos, crd, val, 60000)
    assert np.array_equal(cpos.cpu().numpy(), wpos)  # bit-exact structure
    assert np.array_equal(ccrd.cpu().numpy(), wcrd)
    want = oracle.spgemm_values_acc64(pos, crd, val, pos, crd, val, 60000, wpos, wcrd)
    assert_close(oracle, cval, want, "spgemm values")
    # reproducible to the last bit, like the reference: sums are accumulated order-independently
    for _ in range(2):
        _, _, again = K.spgemm_csr(dev(pos), dev(crd), dev(val), dev(pos), dev(crd), dev(val), 60000)
        assert torch.equal(cval, again)
    # a denser product (many products per output entry) in float64 as well
    B = W.powerlaw_square(3000, mean_nnz=60.0, seed=5)
    bp, bc = B.pos.numpy(), B.crd.numpy()
    for dtype, tol in ((np.float32, (RTOL, ATOL)), (np.float64, (1e-12, 1e-13))):
        bv = B.val.numpy().astype(dtype)
        p1, c1, v1 = K.spgemm_csr(dev(bp), dev(bc), dev(bv), dev(bp), dev(bc), dev(bv), 3000)
        p2, c2, v2 = K.spgemm_csr(dev(bp), dev(bc), dev(bv), dev(bp), dev(bc), dev(bv), 3000)
        assert torch.equal(v1, v2) and torch.equal(c1, c2)
        w_pos, w_crd, _ = oracle.spgemm(bp, bc, bv, bp, bc, bv, 3000)
        assert np.array_equal(p1.cpu().numpy(), w_pos) and np.array_equal(c1.cpu().numpy(), w_crd)
        if dtype == np.float32:
            w64 = oracle.spgemm_values_acc64(bp, bc, bv, bp, bc, bv, 3000, w_pos, w_crd)
            ok, err, bad = oracle.allclose_report(v1.cpu().numpy(), w64, *tol)
            assert ok, (err, bad)
            assert len(w_crd) < 0.7 * int(np.diff(bp)[bc].sum())   # really several products per entry
        else:
            _, _, w = oracle.spgemm(bp, bc, bv, bp, bc, bv, 3000)
            np.testing.assert_allclose(v1.cpu().numpy(), w, rtol=tol[0], atol=tol[1])


def test_spgemm_non_finite_operands_propagate():
    """Rows that touch an infinite or NaN operand are added as plain floats, so the non-finite
    values reach the entries they belong to; the other rows are unaffected."""
    from scorch_b200 import kernels as K
    Apos, Acrd, Aval = random_csr(40, 30, np.random.default_rng(1).integers(1, 6, 40), seed=2)
    Bpos, Bcrd, Bval = random_csr(30, 50, np.random.default_rng(3).integers(1, 6, 30), seed=4)
    clean = K.spgemm_csr(dev(Apos), dev(Acrd), dev(Aval), dev(Bpos), dev(Bcrd), dev(Bval), 50)[2].cpu().numpy()
    Aval2 = Aval.copy()
    Aval2[Apos[7]] = np.inf            # first entry of row 7
    cpos, ccrd, cval = K.spgemm_csr(dev(Apos), dev(Acrd), dev(Aval2), dev(Bpos), dev(Bcrd), dev(Bval), 50)
    cpos, cval = cpos.cpu().numpy(), cval.cpu().numpy()
    row7 = slice(cpos[7], cpos[8])
    assert not np.isfinite(cval[row7]).all()
    keep = np.ones(len(cval), bool)
    keep[row7] = False
    assert np.array_equal(cval[keep], clean[keep])


def test_spgemm_rectangular_and_empty(oracle):
    from scorch_b200 import kernels as K
    Apos, Acrd, Aval = random_csr(70, 50, np.random.default_rng(1).integers(0, 9, 70), seed=2)
    Bpos, Bcrd, Bval = random_csr(50, 90, np.random.default_rng(3).integers(0, 9, 50), seed=4)
    cpos, ccrd, cval = K.spgemm_csr(dev(Apos), dev(Acrd), dev(Aval), dev(Bpos), dev(Bcrd), dev(Bval), 90)
    wpos, wcrd, wval = oracle.spgemm(Apos, Acrd, Aval, Bpos, Bcrd, Bval, 90)
    assert np.array_equal(cpos.cpu().numpy(), wpos) and np.array_equal(ccrd.cpu().numpy(), wcrd)
    np.testing.assert_allclose(cval.cpu().numpy(), wval, rtol=RTOL, atol=ATOL)
    z = np.zeros(71, np.int32)
    cpos, ccrd, cval = K.spgemm_csr(dev(z), dev(np.zeros(0, np.int32)), dev(np.zeros(0, np.float32)),
                                    dev(Bpos[:1].repeat(51)), dev(np.zeros(0, np.int32)),
                                    dev(np.zeros(0, np.float32)), 90)
    assert cpos.cpu().tolist() == [0] * 71 and ccrd.numel() == 0 and cval.numel() == 0


# ================================ plumbing =======================================================
def test_partition_and_coo_csr_plumbing():
    from scorch_b200 import kernels as K
    pos, crd, _ = random_csr(1000, 500, np.random.default_rng(0).integers(0, 30, 1000), seed=1)
    b = K.partition_rows_by_nnz(dev(pos), 4)
    assert b[0] == 0 and b[-1] == 1000 and b == sorted(b)
    nnz = int(pos[-1])
    for g in range(1, 4):
        assert b[g] == int(np.searchsorted(pos, nnz * g // 4, side="left"))
    rows = K.csr_pos_to_coo_rows(dev(pos), nnz)
    assert np.array_equal(rows.cpu().numpy(), np.repeat(np.arange(1000, dtype=np.int32), np.diff(pos)))
    assert np.array_equal(K.coo_rows_to_csr_pos(rows, 1000).cpu().numpy(), pos)
