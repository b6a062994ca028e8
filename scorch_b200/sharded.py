"""Row-sharded SpMM and GCN layers over the GPUs of one box (one process per GPU).

The reference is single-process (its only parallelism is OpenMP inside one kernel,
csrc/spmm.h:2035-2077); this module is the multi-GPU form of the same products:

* rows of the sparse matrix are cut into contiguous blocks balanced by stored entries
  (``sb_partition_rows_by_nnz``); rank g owns block g and computes those output rows;
* the dense operand of a GCN layer is produced row-sharded by the previous layer, so every
  layer all-gathers it (NCCL over NVLink).  The gather is cut into column panels and issued on
  a side stream: the SpMM over panel p runs while panel p+1 is still in flight, and the local
  dense transform X·W (cuBLAS through torch) of later panels overlaps both;
* blocks have different row counts, so each rank's block is padded to the largest block in the
  gathered buffer and the matrix's column indices are remapped ONCE, at set-up, to that padded
  layout (column j of rank r's block -> r*max_rows + (j - start_r)).  Nothing is repacked at
  run time and the gathered panel lands in local HBM before any kernel reads it.

``spmm_fn`` lets the CPU tests (gloo, world size 2) run this host logic with the oracle's SpMM;
the default is the CUDA kernel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

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
class ShardedCsr:
    """One rank's row block of a CSR matrix, columns remapped to the padded gathered layout."""
    rank: int
    world: int
    bounds: List[int]          # world+1 row bounds of the global matrix
    max_rows: int              # rows per rank in the padded gathered layout
    pos: torch.Tensor          # int32 [rows_local + 1], rebased to 0
    crd: torch.Tensor          # int32 [nnz_local], remapped
    val: torch.Tensor
    n_global: int
    plan: object = None
    _buffers: dict = field(default_factory=dict)

    @property
    def rows(self) -> int:
        return self.bounds[self.rank + 1] - self.bounds[self.rank]

    @property
    def nnz(self) -> int:
        return int(self.crd.numel())

    @staticmethod
    def from_global(pos: torch.Tensor, crd: torch.Tensor, val: torch.Tensor, rank: int, world: int,
                    n_cols: Optional[int] = None) -> "ShardedCsr":
        m = pos.numel() - 1
        n_cols = m if n_cols is None else n_cols
        if n_cols != m:
            raise ValueError("sharded layers need a square matrix (features are sharded like rows)")
        bounds = row_bounds(pos, world)
        r0, r1 = bounds[rank], bounds[rank + 1]
        p0, p1 = int(pos[r0]), int(pos[r1])
        lpos = (pos[r0:r1 + 1] - p0).to(torch.int32).contiguous()
        lcrd = crd[p0:p1]
        max_rows = max(bounds[g + 1] - bounds[g] for g in range(world))
        if world > 1:
            starts = torch.tensor(bounds[:-1], dtype=torch.int64, device=crd.device)
            owner = torch.bucketize(lcrd.to(torch.int64), starts, right=True) - 1
            lcrd = (owner * max_rows + (lcrd.to(torch.int64) - starts[owner])).to(torch.int32)
        return ShardedCsr(rank, world, bounds, max_rows, lpos, lcrd.contiguous(),
                          val[p0:p1].contiguous(), m)

    def buffer(self, name: str, shape, device) -> torch.Tensor:
        key = (name, tuple(shape))
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.zeros(shape, dtype=torch.float32, device=device)
            self._buffers[key] = buf
        return buf


def _default_spmm(shard: ShardedCsr, B: torch.Tensor, out: torch.Tensor, relu: bool) -> None:
    from . import kernels as K
    if shard.plan is None:
        shard.plan = K.CsrPlan(shard.pos, shard.nnz)
    K.spmm_csr(shard.pos, shard.crd, shard.val, B, relu=relu, plan=shard.plan, out=out)


def _panels(k: int, widths) -> List[tuple]:
    """(first column, width) of each column panel; ``widths`` is an int or a sequence that is
    repeated/truncated to cover k columns."""
    if isinstance(widths, int):
        widths = [widths]
    out, c, i = [], 0, 0
    while c < k:
        w = min(int(widths[min(i, len(widths) - 1)]), k - c)
        out.append((c, w))
        c += w
        i += 1
    return out


class _Gatherer:
    """Issues one panel's all-gather on the communication stream and hands back the event the
    consumer has to wait for."""

    def __init__(self, shard: ShardedCsr, dev, group):
        self.shard, self.dev, self.group = shard, dev, group
        self.on_gpu = dev.type == "cuda"
        self.comm = None
        if self.on_gpu and shard.world > 1:
            self.comm = shard._buffers.get("comm_stream")
            if self.comm is None:
                # high priority: the gather's few CTAs are placed ahead of the SpMM's pending ones
                # (measured 2.5 % on the 8-GPU forward)
                self.comm = shard._buffers["comm_stream"] = torch.cuda.Stream(device=dev, priority=-1)
        self.main = torch.cuda.current_stream(dev) if self.on_gpu else None

    def gather(self, name: str, send: torch.Tensor):
        """Returns (gathered buffer, event or None)."""
        shard = self.shard
        if shard.world == 1:
            return send, None
        buf = shard.buffer(name, (shard.world * shard.max_rows, send.shape[1]), self.dev)
        if self.comm is None:
            dist.all_gather_into_tensor(buf, send, group=self.group)
            return buf, None
        produced = torch.cuda.Event()
        produced.record(self.main)
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(produced)
            dist.all_gather_into_tensor(buf, send, group=self.group)
            done = torch.cuda.Event()
            done.record(self.comm)
        return buf, done

    def wait(self, event) -> None:
        if event is not None:
            self.main.wait_event(event)


def sharded_layer(shard: ShardedCsr, x_local: torch.Tensor, weight: Optional[torch.Tensor],
                  relu: bool = False, panel=64, group=None,
                  spmm_fn: Optional[Callable] = None) -> torch.Tensor:
    """Rows [bounds[rank], bounds[rank+1]) of  act(A (X W))  (W = None: act(A X)).

    ``x_local`` holds this rank's rows of X.  Per column panel: local transform into the send
    buffer, all-gather into the padded (world*max_rows, panel) receive buffer on the
    communication stream, SpMM of the local row block over that panel as soon as it has arrived.
    """
    spmm_fn = spmm_fn or _default_spmm
    rows, dev = shard.rows, x_local.device
    k = weight.shape[1] if weight is not None else x_local.shape[1]
    panels = _panels(k, k if shard.world == 1 else panel)
    out = torch.empty((rows, k), dtype=torch.float32, device=dev)
    g = _Gatherer(shard, dev, group)
    pending = []
    for idx, (c, w) in enumerate(panels):
        send = shard.buffer(f"send{idx}", (shard.max_rows, w), dev)
        if weight is not None:
            torch.matmul(x_local, weight[:, c:c + w], out=send[:rows])
        else:
            send[:rows].copy_(x_local[:, c:c + w])
        pending.append(g.gather(f"recv{idx}", send))
    for idx, (c, w) in enumerate(panels):
        buf, ev = pending[idx]
        g.wait(ev)
        spmm_fn(shard, buf, out[:, c:c + w], relu)
    return out


def gcn_forward_sharded(shard: ShardedCsr, x_local: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor,
                        panel=(32, 32, 64), panel2=32, group=None,
                        spmm_fn: Optional[Callable] = None) -> torch.Tensor:
    """This rank's rows of  A_hat ReLU(A_hat X W1) W2  (reference caller: bench/bench_gcn.py:314-329).

    Both layers run as one pipeline so that as little communication as possible is exposed:
      * layer 1 is cut into column panels (a narrow first one shortens the pipeline fill); panel
        p's transform X W1[:, p] is all-gathered while the SpMM of panel p-1 runs;
      * as soon as a panel of H = ReLU(A_hat ...) is final, its contribution H_p W2[p, :] is
        accumulated into layer 2's send buffers, so after the last SpMM only a thin GEMM is left
        before layer 2's gathers can start;
      * layer 2 is cut into two panels so that the second gather overlaps the first SpMM.
    With one rank there is nothing to gather and every layer is a single full-width SpMM.
    """
    spmm_fn = spmm_fn or _default_spmm
    rows, dev, world = shard.rows, x_local.device, shard.world
    k1, k2 = W1.shape[1], W2.shape[1]
    if world == 1:
        panel, panel2 = k1, k2
    elif world == 2 and panel == (32, 32, 64) and panel2 == 32:
        panel, panel2 = 64, k2   # two ranks: the gather hides behind SpMM anyway; wider panels are cheaper
    p1, p2 = _panels(k1, panel), _panels(k2, panel2)
    g = _Gatherer(shard, dev, group)
    H = shard.buffer("hidden", (rows, k1), dev)
    out = torch.empty((rows, k2), dtype=torch.float32, device=dev)

    send2 = [shard.buffer(f"l2send{j}", (shard.max_rows, w), dev) for j, (_, w) in enumerate(p2)]
    pending, pending2 = [], []

    def produce(i):   # layer-1 transform of panel i and its gather
        c, w = p1[i]
        send = shard.buffer(f"l1send{i}", (shard.max_rows, w), dev)
        torch.matmul(x_local, W1[:, c:c + w], out=send[:rows])
        pending.append(g.gather(f"l1recv{i}", send))

    def consume(i):   # SpMM of panel i, then its contribution to layer 2's operands
        c, w = p1[i]
        buf, ev = pending[i]
        g.wait(ev)
        hp = H[:, c:c + w]
        spmm_fn(shard, buf, hp, True)
        last = i == len(p1) - 1
        for j, (c2, w2) in enumerate(p2):
            dst = send2[j][:rows]
            if i == 0:
                torch.matmul(hp, W2[c:c + w, c2:c2 + w2], out=dst)
            else:
                dst.addmm_(hp, W2[c:c + w, c2:c2 + w2])
            if last:
                pending2.append(g.gather(f"l2recv{j}", send2[j]))

    # transforms run `lookahead` panels ahead of the SpMMs on the main stream: the first SpMM is
    # issued when its gather is about to land instead of behind every transform
    lookahead = 2
    for i in range(len(p1)):
        produce(i)
        if i >= lookahead:
            consume(i - lookahead)
    for i in range(max(0, len(p1) - lookahead), len(p1)):
        consume(i)
    for j, (c2, w2) in enumerate(p2):
        buf, ev = pending2[j]
        g.wait(ev)
        spmm_fn(shard, buf, out[:, c2:c2 + w2], False)
    return out


def gather_rows(shard: ShardedCsr, local: torch.Tensor, group=None) -> torch.Tensor:
    """All ranks' row blocks concatenated in global row order (for checks and final outputs)."""
    if shard.world == 1:
        return local
    k = local.shape[1]
    send = torch.zeros((shard.max_rows, k), dtype=local.dtype, device=local.device)
    send[:shard.rows] = local
    buf = torch.empty((shard.world * shard.max_rows, k), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, send, group=group)
    parts = [buf[g * shard.max_rows: g * shard.max_rows + (shard.bounds[g + 1] - shard.bounds[g])]
             for g in range(shard.world)]
    return torch.cat(parts, 0)
