"""Sparse attention over banded masks on the tcgen05 tensor cores (128-row tiles, 384-column windows,
scores / probabilities / output in tensor memory) against the float64 oracle of the three-operator
sequence SDDMM -> row softmax -> SpMM, and against the block (mma.sync) path."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from test_gpu_attention import dev, make_mask, oracle_attention

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def window_start(tile, n, rows=128, cols=384):
    return max(0, min(tile * rows - (cols - rows) // 2, n - cols))


@pytest.mark.parametrize("rows,cols,tile", [(128, 384, 0), (512, 512, 2), (300, 200, 2), (1024, 1024, 7)])
def test_probe_scores_are_q_k_transposed(rows, cols, tile):
    """The tensor-core path alone: Q K^T of one tile against its window (operand staging, shared
    memory descriptors, tcgen05.mma with the TF32x3 split, tcgen05.ld)."""
    from scorch_b200 import kernels as K
    rng = np.random.default_rng(rows + tile)
    Q = rng.standard_normal((rows, 64)).astype(np.float32)
    Km = rng.standard_normal((cols, 64)).astype(np.float32)
    got = K.attn_band_probe(dev(Q), dev(Km), tile=tile)[0].cpu().numpy()
    assert K.attn_band_status() == 0
    c0 = window_start(tile, cols)
    want = np.zeros((128, 384))
    q = Q[tile * 128: tile * 128 + 128].astype(np.float64)
    k = Km[c0: c0 + 384].astype(np.float64)
    want[: q.shape[0], : k.shape[0]] = q @ k.T
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=2e-5)


def test_probe_tensor_memory_image():
    """P = exp2(log2(e) S - row max) written back to tensor memory as hi / lo parts and O = P V read
    from there as the A operand (every window column stored, scale 1)."""
    from scorch_b200 import kernels as K
    gen = torch.Generator(device="cuda").manual_seed(11)
    Q = torch.randn((128, 64), generator=gen, device="cuda") * 0.5
    Km = torch.randn((384, 64), generator=gen, device="cuda") * 0.5
    V = torch.randn((384, 64), generator=gen, device="cuda")
    raw, image, _ = K.attn_band_probe(Q, Km, V, tile=0)
    assert K.attn_band_status() == 0
    S = (Q.double() @ Km.double().T) * 1.4426950408889634
    P = torch.exp2(S - S.max(1, keepdim=True).values)
    hi = image[:, :384].double()
    assert ((P - hi).abs() <= P * 2.0 ** -10 + 1e-6).all()   # hi = P truncated to TF32 (10 mantissa bits)
    torch.testing.assert_close(image[:, 384:448].double(), P @ V.double(), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("rows,cols,window,density", [
    (512, 512, 40, 0.02), (500, 530, 24, 0.02), (300, 300, 200, 0.0), (64, 64, 100, 0.0),
    (1000, 1000, 128, 0.01), (100, 4000, 20, 0.01)])
def test_band_plan_matches_dense_scan(rows, cols, window, density):
    from scorch_b200 import kernels as K
    dense, pos, crd, _ = make_mask(rows, cols, window, density, seed=rows + cols)
    bp = K.AttnBandPlan(dev(pos), dev(crd), n=cols)
    inside = 0
    for t in range((rows + 127) // 128):
        c0 = window_start(t, cols)
        inside += int(dense[t * 128: t * 128 + 128, c0: c0 + 384].sum())
    assert bp.inside == inside
    assert bp.rem_nnz == len(crd) - inside


@pytest.mark.parametrize("rows,cols,window,density,empty,values", [
    (512, 512, 40, 0.02, (3, 17, 250), True),    # band + scattered entries, mask values
    (500, 500, 128, 0.01, (), False),             # the benchmark's shape of mask, ragged last tile, pattern mask
    (256, 256, 40, 0.0, (), True),                # band only: no remainder
    (300, 300, 0, 0.05, (0,), True),              # diagonal + scattered: windows nearly empty
    (128, 640, 24, 0.01, (), True),               # K / V longer than Q
    (200, 100, 30, 0.02, (), True),               # fewer columns than a window
])
def test_band_attention_vs_oracle(oracle, rows, cols, window, density, empty, values):
    from scorch_b200 import kernels as K
    d = 64
    dense, pos, crd, mval = make_mask(rows, cols, window, density, seed=rows + 7, empty_rows=empty,
                                      values=values)
    rng = np.random.default_rng(rows)
    Q = (rng.standard_normal((3, rows, d)) * 0.6).astype(np.float32)
    Km = (rng.standard_normal((3, cols, d)) * 0.6).astype(np.float32)
    V = rng.standard_normal((3, cols, d)).astype(np.float32)
    scale = 1.0 / np.sqrt(d)
    bp = K.AttnBandPlan(dev(pos), dev(crd), n=cols)
    got = K.sparse_attention_csr(dev(pos), dev(crd), dev(mval), dev(Q), dev(Km), dev(V), scale=scale,
                                 attn_plan=bp)
    assert K.attn_band_status() == 0
    for u in range(3):
        want = oracle_attention(oracle, pos, crd, mval, Q[u], Km[u], V[u], scale)
        np.testing.assert_allclose(got[u].cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    for r in empty:
        assert not got[:, r].any()


def test_band_path_agrees_with_block_path_and_is_reproducible():
    from scorch_b200 import kernels as K
    d, rows = 64, 1024
    dense, pos, crd, mval = make_mask(rows, rows, 128, 0.01, seed=5)
    gen = torch.Generator(device="cuda").manual_seed(3)
    Q, Km, V = (torch.randn((4, rows, d), generator=gen, device="cuda") * 0.5 for _ in range(3))
    p, c, w = dev(pos), dev(crd), dev(mval)
    a = K.sparse_attention_csr(p, c, w, Q, Km, V, scale=0.125, attn_plan=K.AttnBandPlan(p, c))
    b = K.sparse_attention_csr(p, c, w, Q, Km, V, scale=0.125, attn_plan=K.AttnPlan(p, c))
    torch.testing.assert_close(a, b, rtol=RTOL, atol=ATOL)
    a2 = K.sparse_attention_csr(p, c, w, Q, Km, V, scale=0.125, attn_plan=K.AttnBandPlan(p, c))
    assert torch.equal(a, a2)
    assert K.attn_band_status() == 0
