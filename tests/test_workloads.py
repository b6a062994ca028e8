"""Synthetic-input generators: structure invariants at reduced sizes."""
from __future__ import annotations

import numpy as np
import torch

from scorch_b200 import workloads as W


def _check_csr(c, exact_row=None):
    pos, crd = c.pos.numpy().astype(np.int64), c.crd.numpy()
    assert c.pos.dtype == torch.int32 and c.crd.dtype == torch.int32 and c.val.dtype == torch.float32
    assert pos[0] == 0 and pos[-1] == len(crd) == c.val.numel() and (np.diff(pos) >= 0).all()
    assert crd.min() >= 0 and crd.max() < c.shape[1]
    rows = np.repeat(np.arange(c.shape[0]), np.diff(pos))
    key = rows * c.shape[1] + crd
    assert (np.diff(key) > 0).all()  # ascending and unique within every row
    if exact_row is not None:
        assert (np.diff(pos) == exact_row).all()


def test_c1_uniform():
    c = W.csr_uniform(512, 512, 0.01, seed=0)
    _check_csr(c)
    assert abs(c.nnz - 512 * 512 * 0.01) < 400
    assert torch.equal(W.csr_uniform(512, 512, 0.01, seed=0).crd, c.crd)


def test_c2_mask_and_qkv():
    c = W.attention_mask(256, window=8, density=0.01, seed=0)
    _check_csr(c)
    dense = c.torch_csr().to_dense()
    i = torch.arange(256)
    assert (dense[(i[:, None] - i[None, :]).abs() <= 8] == 1).all()
    q, k, v = W.attention_qkv(1, 2, 256, 16, seed=1)
    assert q.shape == (2, 256, 16) and abs(q.std().item() - 8 ** -0.5) < 0.02


def test_c3_exact_k_per_row():
    c = W.sae_activations(64, 512, 8, seed=0)
    _check_csr(c, exact_row=8)
    assert (c.val > 0).all()
    w = W.sae_decoder(512, 32, seed=1)
    assert abs(w.std().item() - 512 ** -0.5) < 0.01


def test_c4_graph_is_symmetric_normalised_with_self_loops():
    g = W.gcn_graph(2000, mean_deg=8.0, max_deg=300, seed=0)
    _check_csr(g)
    d = g.torch_csr().to_dense()
    assert torch.allclose(d, d.t()) and (torch.diagonal(d) > 0).all()
    deg = (d != 0).sum(1).float()
    want = (d != 0).float() / torch.sqrt(deg[:, None] * deg[None, :])
    assert torch.allclose(d, want, atol=1e-6)


def test_c5_powerlaw_rows():
    c = W.powerlaw_square(20000, mean_nnz=12.0, seed=0)
    _check_csr(c)
    lens = np.diff(c.pos.numpy())
    assert 9 < lens.mean() < 13 and lens.max() > 20 * lens.mean() and lens.min() >= 1
    assert (c.val.abs() <= 1).all()
