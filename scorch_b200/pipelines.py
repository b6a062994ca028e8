"""The two application-level callers of the kernels that the benchmark configurations name, kept
on the device end to end.

* ``sparse_attention`` — per (batch, head): S = SDDMM(mask, Q, K), row softmax over the stored
  entries, O = SpMM(S, V).  Reference caller: bench/bench_sparse_transformer.py:304-382, which
  loops over heads in Python and does the softmax with torch scatter ops; here all heads go
  through one batched launch per stage, or — for masks with enough well-filled 16x16 blocks and
  head dimension 32 / 64 — through the single attention call that never writes the scores.
* ``gcn_forward`` — H = ReLU(A_hat (X W1)), out = A_hat (H W2), transform first like the
  reference's bench (bench/bench_gcn.py:314-329).  The dense X·W products are cuBLAS calls
  through torch (outside the sparse path); the two A_hat products are the SpMM kernel, the first
  with the fused ReLU epilogue.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import kernels as K


def attention_block_plan(pos: torch.Tensor, crd: torch.Tensor) -> Optional[K.BlockPlan]:
    """The mask's block plan if enough of it sits in dense 16x16 blocks to use the tensor-core
    kernels (band / window masks do; purely random masks do not), else None."""
    bp = K.block_plan_for(pos, crd)
    return bp if bp.dense_fraction >= K.BLOCKED_MIN_DENSE_FRACTION else None


BAND_MIN_INSIDE_FRACTION = 0.5   # share of the mask inside the tiles' windows ...
BAND_MIN_WINDOW_FILL = 0.5       # ... and share of the window cells that are stored, for the band path


def attention_plan(pos: torch.Tensor, crd: torch.Tensor, d: int, dv: int):
    """The mask's plan if the one-call path applies (square mask, head dimension 32 / 64 for Q, K
    and V), else None: a ``kernels.AttnBandPlan`` (128-row tiles on tcgen05) for head dimension 64
    when most of the mask lies in well-filled windows around the diagonal, else a
    ``kernels.AttnPlan`` when enough of the mask sits in well-filled 16x16 blocks.
    SCORCH_B200_NO_BAND=1 leaves the band path out."""
    if d != dv or d not in K.FUSED_ATTENTION_D:
        return None
    if d == 64 and not os.environ.get("SCORCH_B200_NO_BAND"):
        bp = K.attn_band_plan_for(pos, crd)
        if bp.inside_fraction >= BAND_MIN_INSIDE_FRACTION and bp.window_fill >= BAND_MIN_WINDOW_FILL:
            return bp
    ap = K.attn_plan_for(pos, crd)
    return ap if ap.block_fraction >= K.BLOCKED_MIN_DENSE_FRACTION else None


def sparse_attention(pos: torch.Tensor, crd: torch.Tensor, mask_val: Optional[torch.Tensor],
                     Q: torch.Tensor, Kmat: torch.Tensor, V: torch.Tensor, scale: float = 1.0,
                     plan: Optional[K.CsrPlan] = None, scores_out: Optional[list] = None,
                     block_plan="auto", fused="auto") -> torch.Tensor:
    """Q, K, V: (units, seq, d) with units = batch*heads.  Returns O (units, seq, d).
    ``block_plan``: "auto" (use the dense-block kernels when the mask has enough dense blocks),
    None (gather kernels only) or a ``kernels.BlockPlan``.
    ``fused``: "auto" (one attention call when the mask and head dimension qualify, the scores
    are not asked for and ``block_plan`` is "auto"), False (always the three operators) or a
    ``kernels.AttnPlan``."""
    if isinstance(fused, str):
        fused = (attention_plan(pos, crd, Q.shape[-1], V.shape[-1])
                 if scores_out is None and isinstance(block_plan, str) and Kmat.shape[-2] == Q.shape[-2]
                 else None)
    if fused:
        if scores_out is not None:
            raise ValueError("the one-call attention path does not produce the scores")
        return K.sparse_attention_csr(pos, crd, mask_val, Q, Kmat, V, scale=scale, attn_plan=fused)
    if isinstance(block_plan, str):
        block_plan = attention_block_plan(pos, crd)
    s = K.sddmm_csr(pos, crd, mask_val, Q, Kmat, block_plan=block_plan)   # (units, nnz)
    K.csr_row_softmax(pos, s, scale=scale, out=s)                         # in place
    if scores_out is not None:
        scores_out.append(s)
    return K.spmm_csr(pos, crd, s, V, plan=plan, block_plan=block_plan)


def gcn_forward(pos, crd, val, X, W1, W2, plan: Optional[K.CsrPlan] = None) -> torch.Tensor:
    xw = torch.matmul(X, W1)
    h = K.spmm_csr(pos, crd, val, xw, relu=True, plan=plan)
    hw = torch.matmul(h, W2)
    return K.spmm_csr(pos, crd, val, hw, plan=plan)


def chunk_bounds(units: int, chunks: int, shrink: bool = True) -> list:
    """First unit of each chunk (+ ``units`` at the end).  ``shrink``: chunk sizes in the ratio
    (2c-1) : ... : 5 : 3 : 1 — the last chunk, whose kernels and copy back cannot overlap with
    anything, is the smallest; otherwise equal chunks.  Chunks may be empty when units < chunks."""
    weights = [2 * (chunks - c) - 1 if shrink else 1 for c in range(chunks)]
    acc, bounds = 0, [0]
    for w in weights:
        acc += w
        bounds.append(max(bounds[-1], min(units, round(units * acc / sum(weights)))))
    bounds[-1] = units
    return bounds


class HostSparseAttention:
    """``sparse_attention`` for operands that live in (pinned) host memory, as the reference's
    callers hold them: the (batch*heads) units are cut into chunks and pipelined over copy and
    compute streams — host->device copies of chunk c+1, kernels of chunk c and device->host copy
    of chunk c-1 overlap, so a step costs about the PCIe time of its inputs instead of copy +
    compute.  The chunks shrink towards the end (weights 7:5:3:1 for four chunks): what cannot
    overlap is the last chunk's kernels and its copy back, so that chunk is the smallest.
    Measured on B200 (32 heads, 100 MB in, 34 MB out): 2.22 ms with shrinking chunks against 2.29
    with equal ones; Q, K and V on a copy stream each (``copy_streams=3``) was slower, 2.43 ms."""

    def __init__(self, pos, crd, mask_val, units: int, seq: int, d: int, chunks: int = 4,
                 scale: float = 1.0, shrink: bool = True, copy_streams: int = 1):
        dev = pos.device
        self.pos, self.crd, self.mask_val, self.scale = pos, crd, mask_val, scale
        self.units, self.seq, self.d = units, seq, d
        self.plan = K.plan_for(pos, crd.numel())
        self.attn_plan = attention_plan(pos, crd, d, d)
        self.block_plan = None if self.attn_plan else attention_block_plan(pos, crd)
        self.bounds = chunk_bounds(units, chunks, shrink)
        self.dev = [torch.empty((units, seq, d), dtype=torch.float32, device=dev) for _ in range(3)]
        self.scores = (None if self.attn_plan else
                       torch.empty((units, crd.numel()), dtype=torch.float32, device=dev))
        self.out = torch.empty((units, seq, d), dtype=torch.float32, device=dev)
        ins = [torch.cuda.Stream(device=dev) for _ in range(copy_streams)]
        self.s_in = [ins[i % copy_streams] for i in range(3)]
        self.s_out = torch.cuda.Stream(device=dev)

    def __call__(self, Qh: torch.Tensor, Kh: torch.Tensor, Vh: torch.Tensor,
                 out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out_host is None:
            out_host = torch.empty((self.units, self.seq, self.d), dtype=torch.float32, pin_memory=True)
        main = torch.cuda.current_stream()
        for st in self.s_in:             # earlier work on these buffers is done
            st.wait_stream(main)
        self.s_out.wait_stream(main)
        for c in range(len(self.bounds) - 1):
            u0, u1 = self.bounds[c], self.bounds[c + 1]
            if u0 == u1:
                continue
            for st, dst, src in zip(self.s_in, self.dev, (Qh, Kh, Vh)):
                with torch.cuda.stream(st):
                    dst[u0:u1].copy_(src[u0:u1], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(st)
                main.wait_event(arrived)
            if self.attn_plan:
                K.sparse_attention_csr(self.pos, self.crd, self.mask_val, self.dev[0][u0:u1],
                                       self.dev[1][u0:u1], self.dev[2][u0:u1], scale=self.scale,
                                       attn_plan=self.attn_plan, out=self.out[u0:u1])
            else:
                s = K.sddmm_csr(self.pos, self.crd, self.mask_val, self.dev[0][u0:u1], self.dev[1][u0:u1],
                                out=self.scores[u0:u1], block_plan=self.block_plan)
                K.csr_row_softmax(self.pos, s, scale=self.scale, out=s)
                K.spmm_csr(self.pos, self.crd, s, self.dev[2][u0:u1], plan=self.plan, out=self.out[u0:u1],
                           block_plan=self.block_plan)
            computed = torch.cuda.Event()
            computed.record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed)
                out_host[u0:u1].copy_(self.out[u0:u1], non_blocking=True)
        main.wait_stream(self.s_out)
        main.synchronize()
        return out_host
