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


class HostGcnForward:
    """The two-layer GCN forward  A_hat ReLU(A_hat X W1) W2  (reference caller: bench/bench_gcn.py:314-329)
    for features that live in pinned host memory and a result that goes back there, with the
    copies overlapped with the kernels instead of put around them:

    * the rows of X arrive in ``in_chunks`` pieces on a copy stream; the first layer runs as
      accumulating SpMM passes over the same row chunks (``sharded._pipelined_layer``), so the
      transform and the pass of chunk c start when chunk c has arrived — the layer costs about
      the PCIe time of X plus its last pass instead of copy + layer;
    * with one rank the second layer is cut into ``out_blocks`` row blocks (balanced by stored
      entries); the rows of block b go back to the host while block b+1 is multiplied.  With
      several ranks the second layer runs as in ``sharded.gcn_forward_sharded`` and the rank's
      rows are copied back at the end.

    Measured on B200 (2 M nodes, 2.05 GB in, 0.51 GB out): 82 ms with copy -> forward -> copy, 51.9 ms
    with 8 chunks / 8 blocks, 50.7 ms with 16 / 16, 61.5 ms with 32 / 16 (the X copy alone is 37 ms).

    ``pos, crd, val``: the global normalised adjacency matrix in CSR on the device; every rank
    keeps its row block (and its own split by row chunk)."""

    def __init__(self, pos, crd, val, W1: torch.Tensor, W2: torch.Tensor, rank: int = 0, world: int = 1,
                 group=None, in_chunks: int = 16, out_blocks: int = 16):
        from . import sharded as S
        env = os.environ.get("SCORCH_B200_HOST_GCN_CHUNKS")      # "<in_chunks>,<out_blocks>"
        if env:
            in_chunks, out_blocks = (int(x) for x in env.split(","))
        self.S, self.group = S, group
        self.W1, self.W2 = W1, W2
        dev = pos.device
        # one rank: equal pieces (the copy is the pace-maker); several ranks: the split tuned for the gathers
        self.shard = (S.ShardedCsr.from_global(pos, crd, val, rank, world, chunks=in_chunks, chunks2=1)
                      if world == 1 else S.ShardedCsr.from_global(pos, crd, val, rank, world))
        self.rows = self.shard.rows
        self.k_in, self.k_out = W1.shape[0], W2.shape[1]
        self.x = torch.empty((self.rows, self.k_in), dtype=torch.float32, device=dev)
        self.out = torch.empty((self.rows, self.k_out), dtype=torch.float32, device=dev)
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.out_blocks = []
        if world == 1:
            local = self.shard.local
            bounds = S.row_bounds(local.pos, max(1, min(out_blocks, max(1, self.rows))))
            for b in range(len(bounds) - 1):
                blk, _ = S.row_block(local.pos, local.crd, local.val, b, len(bounds) - 1, bounds=bounds)
                self.out_blocks.append((bounds[b], bounds[b + 1], blk))
            self.t2 = torch.empty((self.rows, self.k_out), dtype=torch.float32, device=dev)

    def __call__(self, x_host: torch.Tensor, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        S, shard = self.S, self.shard
        if tuple(x_host.shape) != (self.rows, self.k_in):
            raise ValueError(f"x_host must hold this rank's rows: {(self.rows, self.k_in)}")
        if out_host is None:
            out_host = torch.empty((self.rows, self.k_out), dtype=torch.float32, pin_memory=True)
        main = torch.cuda.current_stream()
        self.s_in.wait_stream(main)       # earlier readers of the staging buffers are done
        self.s_out.wait_stream(main)
        offsets = shard.splits[0].offsets
        ready = []
        with torch.cuda.stream(self.s_in):
            for c in range(len(offsets) - 1):
                lo, hi = min(offsets[c], self.rows), min(offsets[c + 1], self.rows)
                if hi > lo:
                    self.x[lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_in)
                ready.append(ev)
        if shard.world > 1:
            out = S.gcn_forward_sharded(shard, self.x, self.W1, self.W2, group=self.group, x_ready=ready)
            out_host.copy_(out, non_blocking=True)
            main.synchronize()
            return out_host
        # (no look-ahead: with one rank there is no gather to keep busy, and chunk c's pass should not wait
        # for chunk c + 2 to arrive)
        H = S.gcn_forward_sharded(shard, self.x, self.W1, self.W2, x_ready=ready, first_layer_only=True,
                                  lookahead=0)
        torch.matmul(H, self.W2, out=self.t2)
        for r0, r1, blk in self.out_blocks:
            if r1 == r0:
                continue
            S.sharded_spmm_replicated(blk, self.t2, out=self.out[r0:r1])
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                out_host[r0:r1].copy_(self.out[r0:r1], non_blocking=True)
        main.wait_stream(self.s_out)
        main.synchronize()
        return out_host
