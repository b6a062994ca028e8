"""Row-sharded SpMM and GCN layers over the GPUs of one box (one process per GPU).

The reference is single-process (its only parallelism is OpenMP inside one kernel,
csrc/spmm.h:2035-2077); this module is the multi-GPU form of the same products:

* rows of the sparse matrix are cut into contiguous blocks balanced by stored entries
  (``sb_partition_rows_by_nnz``); rank g owns block g and computes those output rows;
* a product whose dense operand is the same on every rank (weights, a replicated feature matrix)
  needs no communication: ``row_block`` + the SpMM kernel on the local rows
  (``sharded_spmm_replicated``);
* the dense operand of a GCN layer is produced row-sharded by the previous layer, so every
  layer all-gathers it (NCCL over NVLink).  The gather is cut into ROW CHUNKS: every rank's
  block of operand rows is cut into pieces at the same offsets (equal pieces, or in given
  proportions: a small first piece shortens the start-up during which nothing can be
  multiplied yet), gather c collects piece c of every rank, and the rank's matrix block is
  split once, at set-up, into sub-matrices, the c-th holding the entries whose column falls
  into piece c of its owner.  The layer is then

      C  = A_0 G_0;   C += A_1 G_1;   ...;   C = act(C + A_last G_last)

  with gather c+1 in flight on a communication stream while sub-matrix c is multiplied.  Every
  pass reads full-width operand rows (1 KB at 256 columns) and reads its part of the matrix
  once; the random gathers of one pass are confined to one chunk of the operand, which the L2
  cache holds a good part of;
* SpMV shards like SpMM with a replicated operand (``sharded_spmv``; ``gather_vector`` when every
  rank needs the whole result); SpGEMM shards by row blocks of A balanced by the number of
  products (``product_bounds``), B replicated, each rank running both phases on its block; one
  all-gather of the per-rank entry counts turns the local row pointers into global ones
  (``sharded_spgemm``);
* the (batch, head) units of a sparse-attention call are independent: ``unit_range`` gives each
  rank a contiguous share, no communication;
* blocks have different row counts, so each rank's block is padded to the largest block and the
  column indices are remapped ONCE, at set-up, to the gathered layout of their chunk (column j,
  owned by rank q at offset o inside chunk c = [start_c, start_c + rows_c), becomes
  q * rows_c + o - start_c).  Nothing is repacked at run time and gathered data always lands in
  local HBM before a kernel reads it;
* the two layers of a GCN may be cut differently (``chunks=(first, second)``): the wide first
  layer into a few large pieces, the narrow second one into more.

``spmm_fn`` lets the CPU tests (gloo) run this host logic with a CPU SpMM; the default is the
CUDA kernel.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def row_bounds(pos: torch.Tensor, parts: int) -> List[int]:
    """First row of each nnz-balanced block (+ m at the end).  Device row pointers go through
    the CUDA kernel; host row pointers (set-up code, tests) through torch.searchsorted."""
    if pos.is_cuda:
        from . import kernels as K
        return K.partition_rows_by_nnz(pos, parts)
    m = pos.numel() - 1
    nnz = int(pos[-1])
    targets = torch.tensor([(nnz * g) // parts for g in range(parts)], dtype=pos.dtype)
    b = torch.searchsorted(pos.contiguous(), targets, right=False).tolist()
    return [min(int(x), m) for x in b] + [m]


@dataclass
class CsrBlock:
    """A CSR matrix with the state the SpMM wrapper caches for it."""
    pos: torch.Tensor          # int32 [rows + 1]
    crd: torch.Tensor          # int32 [nnz]
    val: torch.Tensor
    plan: object = None

    @property
    def rows(self) -> int:
        return self.pos.numel() - 1

    @property
    def nnz(self) -> int:
        return int(self.crd.numel())


def row_block(pos: torch.Tensor, crd: torch.Tensor, val: torch.Tensor, rank: int, world: int,
              bounds: Optional[List[int]] = None):
    """Rank's nnz-balanced row block of a CSR matrix, columns untouched: (CsrBlock, bounds)."""
    bounds = row_bounds(pos, world) if bounds is None else bounds
    r0, r1 = bounds[rank], bounds[rank + 1]
    p0, p1 = int(pos[r0]), int(pos[r1])
    lpos = (pos[r0:r1 + 1] - p0).to(torch.int32).contiguous()
    return CsrBlock(lpos, crd[p0:p1].contiguous(), val[p0:p1].contiguous()), bounds


def default_chunks(world: int):
    """(first layer, second layer) row chunks of a GCN: one piece with one rank (nothing to
    overlap).  Otherwise the first piece is an eighth of the rows, so that the first gather is
    short, and the 256-wide first layer goes in pieces of 1/8, 3/8, 1/2 up to four ranks (every
    extra pass cost 0.3-0.4 ms at four ranks, and the gathers are short against the passes) and of
    1/8, 1/8, 1/4, 1/4, 1/4 beyond (gather and pass take about as long there, so finer pieces
    overlap better); the 64-wide second layer goes in eight equal pieces.
    SCORCH_B200_GCN_CHUNKS overrides: "6" (both layers), "4;8" (first; second), or proportions
    such as "1,1,2,2,2;8"."""
    env = os.environ.get("SCORCH_B200_GCN_CHUNKS")
    if env:
        parts = [[int(x) for x in p.split(",")] for p in env.split(";")]
        parts = [p[0] if len(p) == 1 else p for p in parts]
        return parts[0], parts[-1]
    if world == 1:
        return 1, 1
    return ([1, 3, 4] if world <= 4 else [1, 1, 2, 2, 2]), 8


def chunk_offsets(rows: int, spec) -> List[int]:
    """Row offsets [0, ..., rows] of the chunks: `spec` equal pieces (int) or pieces in the given
    proportions (sequence).  Every piece holds at least one row where rows allow."""
    weights = [1] * int(spec) if isinstance(spec, int) else [int(w) for w in spec]
    if not weights or any(w <= 0 for w in weights):
        raise ValueError("chunks must be a positive count or a sequence of positive proportions")
    total, acc, out = sum(weights), 0, [0]
    for w in weights:
        acc += w
        out.append(max(out[-1], -(-rows * acc // total)))
    out[-1] = rows
    return out


@dataclass
class Split:
    """A rank's row block split by operand row chunk: chunk c covers rows [offsets[c],
    offsets[c+1]) of every rank's (padded) block; blocks[c] holds the entries whose column lies
    there, renumbered to the layout an all-gather of those pieces produces."""
    offsets: List[int]
    blocks: List[CsrBlock]

    @property
    def chunks(self) -> int:
        return len(self.blocks)

    def rows_of(self, c: int) -> int:
        return self.offsets[c + 1] - self.offsets[c]


@dataclass
class ShardedCsr:
    """One rank's row block of a square CSR matrix, split by operand row chunk (one split per
    layer kind: ``splits[0]`` for the first layer, ``splits[-1]`` for the last)."""
    rank: int
    world: int
    bounds: List[int]          # world+1 row bounds of the global matrix
    max_rows: int              # rows of the largest block = rows per rank in the padded layout
    splits: List[Split]
    n_global: int
    local: CsrBlock            # the unsplit row block with global column indices
    _buffers: dict = field(default_factory=dict)

    @property
    def blocks(self) -> List[CsrBlock]:
        return self.splits[0].blocks

    @property
    def chunks(self) -> int:
        return self.splits[0].chunks

    @property
    def rows(self) -> int:
        return self.bounds[self.rank + 1] - self.bounds[self.rank]

    @property
    def nnz(self) -> int:
        return self.local.nnz

    @staticmethod
    def from_global(pos: torch.Tensor, crd: torch.Tensor, val: torch.Tensor, rank: int, world: int,
                    n_cols: Optional[int] = None, chunks=None, chunks2=None) -> "ShardedCsr":
        """``chunks``: row chunks of the first layer, a count or a sequence of proportions;
        ``chunks2``: the same for the second layer (default: like the first).  With neither,
        ``default_chunks(world)``."""
        m = pos.numel() - 1
        n_cols = m if n_cols is None else n_cols
        if n_cols != m:
            raise ValueError("sharded layers need a square matrix (features are sharded like rows); "
                             "use row_block / sharded_spmm_replicated for a replicated operand")
        local, bounds = row_block(pos, crd, val, rank, world)
        if chunks is None:
            chunks, default2 = default_chunks(world)
            chunks2 = default2 if chunks2 is None else chunks2
        specs = [chunks, chunks if chunks2 is None else chunks2]
        largest = max(bounds[g + 1] - bounds[g] for g in range(world))
        splits, seen = [], {}
        for spec in specs:
            key = spec if isinstance(spec, int) else tuple(spec)
            if key not in seen:
                offsets = chunk_offsets(max(1, largest), spec)
                seen[key] = Split(offsets, _split_by_chunk(local, bounds, offsets))
            splits.append(seen[key])
        return ShardedCsr(rank, world, bounds, max(1, largest), splits, m, local)

    def buffer(self, name: str, shape, device) -> torch.Tensor:
        key = (name, tuple(shape))
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.zeros(shape, dtype=torch.float32, device=device)
            self._buffers[key] = buf
        return buf


def _split_by_chunk(local: CsrBlock, bounds: List[int], offsets: List[int]) -> List[CsrBlock]:
    """Sub-matrix c keeps the entries whose column lies in rows [offsets[c], offsets[c+1]) of its
    owner's block, renumbered to the layout an all-gather of those pieces produces.  Columns stay
    ascending within a row (owner, then offset, is the global order)."""
    dev = local.crd.device
    rows, chunks = local.rows, len(offsets) - 1
    starts = torch.tensor(bounds[:-1], dtype=torch.int64, device=dev)
    cuts = torch.tensor(offsets, dtype=torch.int64, device=dev)
    j = local.crd.to(torch.int64)
    owner = torch.bucketize(j, starts, right=True) - 1
    off = j - starts[owner]
    del j
    c = torch.bucketize(off, cuts[1:-1].contiguous(), right=True)
    width = cuts[1:] - cuts[:-1]
    newcol = (owner * width[c] + (off - cuts[c])).to(torch.int32)
    del owner, off
    if chunks == 1:
        return [CsrBlock(local.pos, newcol, local.val)]
    lens = (local.pos[1:] - local.pos[:-1]).to(torch.int64)
    row = torch.repeat_interleave(torch.arange(rows, dtype=torch.int64, device=dev), lens)
    key = c * rows + row
    del c, row
    order = torch.sort(key, stable=True).indices
    counts = torch.bincount(key, minlength=chunks * rows)
    del key
    crd_s, val_s = newcol[order].contiguous(), local.val[order].contiguous()
    del order, newcol
    pos_all = torch.zeros(chunks * rows + 1, dtype=torch.int64, device=dev)
    pos_all[1:] = torch.cumsum(counts, 0)
    ends = pos_all[::rows][:chunks + 1].tolist() if rows else [0] * (chunks + 1)
    out = []
    for ci in range(chunks):
        e0, e1 = int(ends[ci]), int(ends[ci + 1])
        p = (pos_all[ci * rows: ci * rows + rows + 1] - e0).to(torch.int32).contiguous()
        out.append(CsrBlock(p, crd_s[e0:e1], val_s[e0:e1]))
    return out


def _default_spmm(block: CsrBlock, B: torch.Tensor, out: torch.Tensor, relu: bool,
                  accumulate: bool = False) -> None:
    from . import kernels as K
    if block.plan is None:
        block.plan = K.CsrPlan(block.pos, block.nnz)
    K.spmm_csr(block.pos, block.crd, block.val, B, relu=relu, plan=block.plan, out=out,
               accumulate=accumulate)


def sharded_spmm_replicated(block: CsrBlock, B: torch.Tensor, bias=None, relu: bool = False,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """This rank's rows of act(bias + A B) for a dense operand every rank holds (a weight matrix,
    a replicated feature matrix): no communication, any matrix shape."""
    from . import kernels as K
    if block.plan is None:
        block.plan = K.CsrPlan(block.pos, block.nnz)
    return K.spmm_csr(block.pos, block.crd, block.val, B, bias=bias, relu=relu, plan=block.plan, out=out)


class Timeline:
    """Optional per-step record of where a sharded forward spends its time: CUDA events around
    the dense transforms, the waits for gathered chunks and the SpMM launches on the main stream,
    and around each all-gather on the communication stream.  ``summary()`` synchronises."""

    def __init__(self):
        self.spans = []   # (label, start event, end event)
        self.steps = 0

    def span(self, label: str, stream=None):
        return _Span(self, label, stream)

    def summary(self) -> dict:
        """Mean milliseconds per step and label."""
        out = {}
        for label, a, b in self.spans:
            b.synchronize()
            out[label] = out.get(label, 0.0) + a.elapsed_time(b)
        steps = max(1, self.steps)
        return {k: v / steps for k, v in out.items()}


class _Span:
    def __init__(self, tl: Optional[Timeline], label: str, stream):
        self.tl, self.label, self.stream = tl, label, stream

    def __enter__(self):
        if self.tl is not None:
            self.a = torch.cuda.Event(enable_timing=True)
            self.a.record(self.stream)
        return self

    def __exit__(self, *exc):
        if self.tl is not None:
            b = torch.cuda.Event(enable_timing=True)
            b.record(self.stream)
            self.tl.spans.append((self.label, self.a, b))
        return False


def _span(tl: Optional[Timeline], label: str, stream=None):
    return _Span(tl, label, stream)


class _Gatherer:
    """Issues one chunk's all-gather on the communication stream and hands back the event the
    consumer has to wait for."""

    def __init__(self, shard: ShardedCsr, dev, group, timeline: Optional[Timeline] = None):
        self.shard, self.dev, self.group, self.tl = shard, dev, group, timeline
        self.on_gpu = dev.type == "cuda"
        self.comm = None
        if self.on_gpu and shard.world > 1:
            self.comm = shard._buffers.get("comm_stream")
            if self.comm is None:
                # high priority: the gather's few CTAs are placed ahead of the SpMM's pending ones
                self.comm = shard._buffers["comm_stream"] = torch.cuda.Stream(device=dev, priority=-1)
        self.main = torch.cuda.current_stream(dev) if self.on_gpu else None

    def gather(self, name: str, send: torch.Tensor, produced=None):
        """Returns (gathered buffer, event or None).  ``produced``: the event after which ``send``
        holds its data (default: everything issued on the main stream so far)."""
        shard = self.shard
        if shard.world == 1:
            if produced is not None:
                self.main.wait_event(produced)
            return send, None
        buf = shard.buffer(name, (shard.world * send.shape[0], send.shape[1]), self.dev)
        if self.comm is None:
            dist.all_gather_into_tensor(buf, send, group=self.group)
            return buf, None
        if produced is None:
            produced = torch.cuda.Event()
            produced.record(self.main)
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(produced)
            with _span(self.tl if self.on_gpu else None, "all_gather", self.comm):
                dist.all_gather_into_tensor(buf, send, group=self.group)
            done = torch.cuda.Event()
            done.record(self.comm)
        return buf, done

    def wait(self, event) -> None:
        if event is not None:
            with _span(self.tl, "wait_for_gather", self.main):
                self.main.wait_event(event)


def _pipelined_layer(shard: ShardedCsr, split: Split, g: _Gatherer, name: str, x_local: torch.Tensor,
                     weight: Optional[torch.Tensor], out: torch.Tensor, relu: bool,
                     spmm_fn: Callable, lookahead: int, tl: Optional[Timeline], label: str,
                     x_ready: Optional[Sequence] = None) -> None:
    """out = act(A (x_local W)) over this rank's rows, chunk by chunk (W = None: act(A x)).
    ``x_ready``: one CUDA event per chunk after which that chunk's rows of ``x_local`` are valid
    (rows that are still arriving, e.g. by a host-to-device copy on another stream)."""
    S, dev = split.chunks, x_local.device
    k = out.shape[1]
    send = shard.buffer(name + "send", (shard.max_rows, k), dev)
    pending = []
    tlg = tl if dev.type == "cuda" else None
    # with several ranks the dense transforms run on a stream of their own, beside the SpMM passes
    # (0.6 ms of 11.9 at four ranks); SCORCH_B200_GCN_TRANSFORM_STREAM=0 puts them back on the main
    # stream, =1 also moves them there for a chunked layer on one rank
    side = None
    want_side = os.environ.get("SCORCH_B200_GCN_TRANSFORM_STREAM", "1" if shard.world > 1 else "0")
    if dev.type == "cuda" and S > 1 and want_side != "0":
        side = shard._buffers.get("transform_stream")
        if side is None:
            side = shard._buffers["transform_stream"] = torch.cuda.Stream(device=dev)
        ready = torch.cuda.Event()
        ready.record(g.main)          # the layer's input and the send buffer are free from here on
        side.wait_event(ready)

    def produce(c):
        lo, hi = min(split.offsets[c], shard.rows), min(split.offsets[c + 1], shard.rows)
        produced = None
        with torch.cuda.stream(side) if side is not None else _span(None, ""):
            if x_ready is not None and x_ready[c] is not None:
                (side if side is not None else g.main).wait_event(x_ready[c])
            if hi > lo:
                with _span(tlg, "dense_transform", side):
                    if weight is not None:
                        torch.matmul(x_local[lo:hi], weight, out=send[lo:hi])
                    else:
                        send[lo:hi].copy_(x_local[lo:hi])
            if side is not None:
                produced = torch.cuda.Event()
                produced.record(side)
        pending.append(g.gather(f"{name}recv{c}", send[split.offsets[c]:split.offsets[c + 1]], produced))

    def consume(c):
        buf, ev = pending[c]
        g.wait(ev)
        with _span(tlg, label):
            spmm_fn(split.blocks[c], buf, out, relu and c == S - 1, c > 0)

    for c in range(S):
        produce(c)
        if c >= lookahead:
            consume(c - lookahead)
    for c in range(max(0, S - lookahead), S):
        consume(c)


def sharded_layer(shard: ShardedCsr, x_local: torch.Tensor, weight: Optional[torch.Tensor],
                  relu: bool = False, group=None, spmm_fn: Optional[Callable] = None,
                  lookahead: int = 2, timeline: Optional[Timeline] = None) -> torch.Tensor:
    """Rows [bounds[rank], bounds[rank+1]) of  act(A (X W))  (W = None: act(A X)).

    ``x_local`` holds this rank's rows of X.  Per row chunk: local transform into the send
    buffer, all-gather of that piece from every rank on the communication stream, SpMM of the
    chunk's sub-matrix (accumulating into the output) as soon as the piece has arrived."""
    spmm_fn = spmm_fn or _default_spmm
    dev = x_local.device
    k = weight.shape[1] if weight is not None else x_local.shape[1]
    out = torch.empty((shard.rows, k), dtype=torch.float32, device=dev)
    g = _Gatherer(shard, dev, group, timeline)
    split = shard.splits[0] if k > 128 else shard.splits[-1]
    _pipelined_layer(shard, split, g, f"layer{k}", x_local, weight, out, relu, spmm_fn, lookahead, timeline,
                     "spmm")
    return out


def gcn_forward_sharded(shard: ShardedCsr, x_local: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor,
                        group=None, spmm_fn: Optional[Callable] = None, lookahead: int = 2,
                        timeline: Optional[Timeline] = None, x_ready: Optional[Sequence] = None,
                        first_layer_only: bool = False) -> torch.Tensor:
    """This rank's rows of  A_hat ReLU(A_hat X W1) W2  (reference caller: bench/bench_gcn.py:314-329;
    transform first, then the sparse product, as there).

    Per layer the local transform of row chunk c (cuBLAS through torch) is all-gathered while the
    sub-matrices of earlier chunks are multiplied; transforms run ``lookahead`` chunks ahead of
    the SpMMs on the main stream so that the communication stream always has a gather queued.
    Exposed communication is one chunk's transform + gather at the start of each layer.  With one
    rank and one chunk every layer is a single full-width SpMM.
    ``x_ready``: per first-layer chunk, the event after which that chunk's rows of ``x_local`` are
    valid; ``first_layer_only``: return the hidden layer ReLU(A_hat X W1) (this rank's rows)."""
    spmm_fn = spmm_fn or _default_spmm
    lookahead = int(os.environ.get("SCORCH_B200_GCN_LOOKAHEAD", lookahead))
    dev = x_local.device
    k1, k2 = W1.shape[1], W2.shape[1]
    g = _Gatherer(shard, dev, group, timeline)
    H = shard.buffer("hidden", (shard.rows, k1), dev)
    out = torch.empty((shard.rows, k2), dtype=torch.float32, device=dev)
    _pipelined_layer(shard, shard.splits[0], g, "l1", x_local, W1, H, True, spmm_fn, lookahead, timeline,
                     "spmm_layer1", x_ready=x_ready)
    if first_layer_only:
        return H
    _pipelined_layer(shard, shard.splits[-1], g, "l2", H, W2, out, False, spmm_fn, lookahead, timeline,
                     "spmm_layer2")
    if timeline is not None:
        timeline.steps += 1
    return out


def gather_rows(shard: ShardedCsr, local: torch.Tensor, group=None) -> torch.Tensor:
    """All ranks' row blocks concatenated in global row order (for checks and final outputs)."""
    if shard.world == 1:
        return local
    k = local.shape[1]
    largest = max(shard.bounds[g + 1] - shard.bounds[g] for g in range(shard.world))
    send = torch.zeros((largest, k), dtype=local.dtype, device=local.device)
    send[:shard.rows] = local
    buf = torch.empty((shard.world * largest, k), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, send, group=group)
    parts = [buf[g * largest: g * largest + (shard.bounds[g + 1] - shard.bounds[g])]
             for g in range(shard.world)]
    return torch.cat(parts, 0)


# ---- SpMV / SpGEMM / independent units ------------------------------------------------------------
def unit_range(units: int, rank: int, world: int):
    """Contiguous share [first, last) of `units` independent work items (the (batch, head) pairs
    of a sparse-attention call) for this rank; shares differ by at most one."""
    return (units * rank) // world, (units * (rank + 1)) // world


def sharded_spmv(block: CsrBlock, x: torch.Tensor, spmv_fn: Optional[Callable] = None) -> torch.Tensor:
    """This rank's rows of A x for a vector every rank holds (no communication)."""
    if spmv_fn is not None:
        return spmv_fn(block, x)
    from . import kernels as K
    return K.spmv_csr(block.pos, block.crd, block.val, x)


def gather_vector(local: torch.Tensor, bounds: List[int], group=None) -> torch.Tensor:
    """The row blocks of a sharded vector concatenated on every rank (one all-gather of blocks
    padded to the largest one)."""
    world = len(bounds) - 1
    if world == 1:
        return local
    largest = max(bounds[g + 1] - bounds[g] for g in range(world))
    send = torch.zeros(largest, dtype=local.dtype, device=local.device)
    send[:local.numel()] = local
    buf = torch.empty(world * largest, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, send, group=group)
    return torch.cat([buf[g * largest: g * largest + bounds[g + 1] - bounds[g]] for g in range(world)])


def product_bounds(Apos: torch.Tensor, Acrd: torch.Tensor, Bpos: torch.Tensor, parts: int) -> List[int]:
    """Row bounds of A that balance the number of scalar products of A B (entry (i, j) of A costs
    one product per stored entry of row j of B): block g starts at the first row whose running
    product count reaches g/parts of the total."""
    m = Apos.numel() - 1
    blen = (Bpos[1:] - Bpos[:-1]).to(torch.int64)
    per_entry = blen[Acrd.to(torch.int64)]
    run = torch.zeros(Acrd.numel() + 1, dtype=torch.int64, device=Acrd.device)
    run[1:] = torch.cumsum(per_entry, 0)
    row_run = run[Apos.to(torch.int64)]                  # products before each row
    total = int(row_run[-1])
    targets = torch.tensor([(total * g) // parts for g in range(parts)], dtype=torch.int64,
                           device=Acrd.device)
    b = torch.searchsorted(row_run.contiguous(), targets, right=False).tolist()
    return [min(int(x), m) for x in b] + [m]


def sharded_spgemm(Ablock: CsrBlock, Bpos, Bcrd, Bval, n: int, group=None,
                   spgemm_fn: Optional[Callable] = None):
    """This rank's rows of C = A B (both phases of the SpGEMM on the local row block, B held by
    every rank).  Returns (Cpos, Ccrd, Cval, offset, total): ``Cpos`` are the rows' pointers into
    the rank's own arrays (starting at 0); ``offset`` is what to add to make them pointers into
    the concatenation of all ranks' arrays (the stored entries of the ranks before this one) and
    ``total`` the entry count of the whole product — from one all-gather of the per-rank counts."""
    if spgemm_fn is None:
        from . import kernels as K
        cpos, ccrd, cval = K.spgemm_csr(Ablock.pos, Ablock.crd, Ablock.val, Bpos, Bcrd, Bval, n)
    else:
        cpos, ccrd, cval = spgemm_fn(Ablock, Bpos, Bcrd, Bval, n)
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    counts = torch.zeros(world, dtype=torch.int64, device=ccrd.device)
    mine = torch.tensor([ccrd.numel()], dtype=torch.int64, device=ccrd.device)
    if world > 1:
        dist.all_gather_into_tensor(counts, mine, group=group)
    else:
        counts[0] = mine[0]
    counts = counts.tolist()
    total = sum(counts)
    if total > 2**31 - 1:
        raise OverflowError(f"the product has {total} stored entries: global int32 row pointers overflow")
    return cpos, ccrd, cval, sum(counts[:rank]), total
