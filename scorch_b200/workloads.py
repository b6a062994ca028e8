"""Seeded synthetic inputs with the shapes and distributions of the five benchmark configurations
(the reference benchmarks on SuiteSparse / Planetoid / OGB / MNIST-style data that cannot be
fetched; these stand in for them).  All generators are deterministic for a given seed and
device type, return int32 indices sorted ascending and unique within a row, float32 values, and
contiguous tensors.  Sizes can be scaled down for tests.

  C1  uniform 1 % CSR x dense            (csr_uniform)
  C2  sparse-attention mask + Q, K, V    (attention_mask, attention_qkv)
  C3  sparse-autoencoder decode          (sae_activations, sae_decoder)
  C4  power-law graph, GCN-normalised    (gcn_graph, glorot)
  C5  power-law square matrix            (powerlaw_square)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch


@dataclass
class Csr:
    """CSR arrays as the kernels take them."""
    shape: Tuple[int, int]
    pos: torch.Tensor  # int32 [m+1]
    crd: torch.Tensor  # int32 [nnz]
    val: torch.Tensor  # [nnz]

    @property
    def nnz(self) -> int:
        return int(self.crd.numel())

    def to(self, device) -> "Csr":
        return Csr(self.shape, self.pos.to(device), self.crd.to(device), self.val.to(device))

    def torch_csr(self) -> torch.Tensor:
        return torch.sparse_csr_tensor(self.pos, self.crd, self.val, size=self.shape)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


# ---- C1 ------------------------------------------------------------------------------------------
def csr_uniform(m: int = 4096, n: int = 4096, density: float = 0.01, seed: int = 0) -> Csr:
    """Row counts ~ Binomial(n, density); columns uniform without replacement per row; N(0,1)."""
    rng = np.random.default_rng(seed)
    counts = rng.binomial(n, density, size=m).astype(np.int64)
    pos = np.zeros(m + 1, np.int64)
    np.cumsum(counts, out=pos[1:])
    crd = np.empty(pos[-1], np.int32)
    for i in range(m):
        if counts[i]:
            crd[pos[i]:pos[i + 1]] = np.sort(rng.choice(n, size=counts[i], replace=False))
    val = rng.standard_normal(pos[-1]).astype(np.float32)
    return Csr((m, n), torch.from_numpy(pos.astype(np.int32)), torch.from_numpy(crd),
               torch.from_numpy(val))


def dense_normal(rows: int, cols: int, seed: int, std: float = 1.0) -> torch.Tensor:
    rng = np.random.default_rng(seed)
    return torch.from_numpy((rng.standard_normal((rows, cols)) * std).astype(np.float32))


# ---- C2 ------------------------------------------------------------------------------------------
def attention_mask(seq: int = 4096, window: int = 128, density: float = 0.01, seed: int = 0) -> Csr:
    """Band |i-j| <= window united with Bernoulli(density) pairs; values 1.0; one mask for all heads."""
    rng = np.random.default_rng(seed)
    i = np.arange(seq)[:, None]
    j = np.arange(seq)[None, :]
    dense = (np.abs(i - j) <= window) | (rng.random((seq, seq)) < density)
    counts = dense.sum(1)
    pos = np.zeros(seq + 1, np.int64)
    np.cumsum(counts, out=pos[1:])
    crd = np.nonzero(dense)[1].astype(np.int32)  # row-major order: ascending within a row
    val = np.ones(pos[-1], np.float32)
    return Csr((seq, seq), torch.from_numpy(pos.astype(np.int32)), torch.from_numpy(crd),
               torch.from_numpy(val))


def attention_qkv(batch: int = 4, heads: int = 8, seq: int = 4096, d: int = 64, seed: int = 1):
    """Q, K, V ~ N(0, 1/8), shape (batch*heads, seq, d)."""
    rng = np.random.default_rng(seed)
    std = 8.0 ** -0.5
    out = []
    for _ in range(3):
        out.append(torch.from_numpy((rng.standard_normal((batch * heads, seq, d)) * std)
                                    .astype(np.float32)))
    return tuple(out)


# ---- C3 ------------------------------------------------------------------------------------------
def sae_activations(batch: int = 8192, latent: int = 32768, k: int = 32, seed: int = 0,
                    device="cpu") -> Csr:
    """Exactly k stored entries per row: top-k of |N(0,1)| per row, values |z| (> 0)."""
    g = _gen(seed, device)
    rows_per = max(1, min(batch, (1 << 26) // latent))
    crd = torch.empty((batch, k), dtype=torch.int32, device=device)
    val = torch.empty((batch, k), dtype=torch.float32, device=device)
    for r0 in range(0, batch, rows_per):
        r1 = min(batch, r0 + rows_per)
        z = torch.randn((r1 - r0, latent), generator=g, device=device, dtype=torch.float32).abs_()
        v, c = torch.topk(z, k, dim=1)
        c, order = torch.sort(c, dim=1)
        crd[r0:r1] = c.to(torch.int32)
        val[r0:r1] = torch.gather(v, 1, order)
    pos = torch.arange(0, (batch + 1) * k, k, dtype=torch.int32, device=device)
    return Csr((batch, latent), pos, crd.reshape(-1).contiguous(), val.reshape(-1).contiguous())


def sae_decoder(latent: int = 32768, width: int = 4096, seed: int = 1, device="cpu") -> torch.Tensor:
    g = _gen(seed, device)
    return torch.randn((latent, width), generator=g, device=device, dtype=torch.float32) * (latent ** -0.5)


# ---- power-law helpers -----------------------------------------------------------------------------
def _powerlaw_degrees(n: int, exponent: float, mean: float, cap: Optional[int], g, device):
    """d = clamp(floor(x_min * (1-u)^(-1/(exponent-1))), 1, cap) with x_min bisected to the mean."""
    u = torch.rand(n, generator=g, device=device, dtype=torch.float64)
    base = (1.0 - u).clamp_min(1e-300).pow(-1.0 / (exponent - 1.0))

    def degrees(xmin: float) -> torch.Tensor:
        d = torch.floor(base * xmin).clamp_min(1.0)
        if cap is not None:
            d = d.clamp_max(float(cap))
        return d

    lo, hi = 1e-3, float(mean) * 4 + 4
    for _ in range(60):
        mid = 0.5 * (lo + hi)
        if degrees(mid).mean().item() < mean:
            lo = mid
        else:
            hi = mid
    return degrees(hi).clamp_max(float(n)).to(torch.int64)


def _csr_from_keys(keys: torch.Tensor, n_rows: int, n_cols: int):
    """Unique sorted (row*n_cols+col) keys -> pos, crd."""
    keys = torch.unique(keys)  # sorted
    row = torch.div(keys, n_cols, rounding_mode="floor")
    crd = (keys - row * n_cols).to(torch.int32)
    counts = torch.bincount(row, minlength=n_rows)
    pos = torch.zeros(n_rows + 1, dtype=torch.int64, device=keys.device)
    pos[1:] = torch.cumsum(counts, 0)
    return pos.to(torch.int32), crd, row


# ---- C4 ------------------------------------------------------------------------------------------
def gcn_graph(n: int = 2_000_000, exponent: float = 2.1, mean_deg: float = 50.0,
              max_deg: int = 50_000, seed: int = 0, device="cpu") -> Csr:
    """Power-law out-degrees, uniform destinations, symmetrised, self-loops, values
    1/sqrt(deg_i * deg_j) with deg = row count of A+I (the D^-1/2 (A+I) D^-1/2 normalisation)."""
    g = _gen(seed, device)
    deg = _powerlaw_degrees(n, exponent, mean_deg, min(max_deg, n), g, device)
    src = torch.repeat_interleave(torch.arange(n, device=device, dtype=torch.int64), deg)
    dst = torch.randint(0, n, (src.numel(),), generator=g, device=device, dtype=torch.int64)
    loops = torch.arange(n, device=device, dtype=torch.int64)
    keys = torch.cat([src * n + dst, dst * n + src, loops * n + loops])
    del src, dst
    pos, crd, row = _csr_from_keys(keys, n, n)
    del keys
    rowdeg = (pos[1:] - pos[:-1]).to(torch.float32)
    dinv = rowdeg.rsqrt()
    val = dinv[row] * dinv[crd.long()]
    return Csr((n, n), pos, crd, val.contiguous())


def glorot(fan_in: int, fan_out: int, seed: int = 0, device="cpu") -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    limit = math.sqrt(6.0 / (fan_in + fan_out))
    w = (torch.rand((fan_in, fan_out), generator=g, dtype=torch.float32) * 2 - 1) * limit
    return w.to(device)


def randn_on(shape, seed: int, device="cpu") -> torch.Tensor:
    return torch.randn(shape, generator=_gen(seed, device), device=device, dtype=torch.float32)


# ---- C5 ------------------------------------------------------------------------------------------
def powerlaw_square(n: int = 2_000_000, exponent: float = 2.3, mean_nnz: float = 12.0, seed: int = 0,
                    device="cpu") -> Csr:
    """Row lengths power-law (no cap), columns uniform, de-duplicated, values U(-1, 1)."""
    g = _gen(seed, device)
    deg = _powerlaw_degrees(n, exponent, mean_nnz, None, g, device)
    row = torch.repeat_interleave(torch.arange(n, device=device, dtype=torch.int64), deg)
    col = torch.randint(0, n, (row.numel(),), generator=g, device=device, dtype=torch.int64)
    pos, crd, _ = _csr_from_keys(row * n + col, n, n)
    val = torch.rand(crd.numel(), generator=g, device=device, dtype=torch.float32) * 2 - 1
    return Csr((n, n), pos, crd, val)
