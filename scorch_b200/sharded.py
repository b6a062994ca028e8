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


def sharded_layer(shard: ShardedCsr, x_local: torch.Tensor, weight: Optional[torch.Tensor],
                  relu: bool = False, panel: int = 64, group=None,
                  spmm_fn: Optional[Callable] = None, timings: Optional[dict] = None) -> torch.Tensor:
    """Rows [bounds[rank], bounds[rank+1]) of  act(A (X W))  (W = None: act(A X)).

    ``x_local`` holds this rank's rows of X.  Per column panel: local transform into the send
    buffer, all-gather into the padded (world*max_rows, panel) receive buffer, SpMM of the local
    row block over that panel.
    """
    spmm_fn = spmm_fn or _default_spmm
    world, rows, dev = shard.world, shard.rows, x_local.device
    k = weight.shape[1] if weight is not None else x_local.shape[1]
    panel = min(panel, k)
    panels = [(c, min(panel, k - c)) for c in range(0, k, panel)]
    out = torch.empty((rows, k), dtype=torch.float32, device=dev)
    on_gpu = x_local.is_cuda
    comm = None
    if on_gpu and world > 1:
        comm = shard._buffers.get("comm_stream")
        if comm is None:
            comm = shard._buffers["comm_stream"] = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev) if on_gpu else None

    def mark(stream):
        if timings is None or not on_gpu:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream)
        return ev

    if timings is not None:
        timings.setdefault("events", []).append(("layer_start", mark(main)))
    recv, ready = [], []
    for idx, (c, w) in enumerate(panels):
        send = shard.buffer(f"send{idx}", (shard.max_rows, w), dev)
        if weight is not None:
            torch.matmul(x_local, weight[:, c:c + w], out=send[:rows])
        else:
            send[:rows].copy_(x_local[:, c:c + w])
        if timings is not None:
            timings["events"].append((f"transform{idx}_done", mark(main)))
        if world == 1:
            recv.append(send)
            ready.append(None)
            continue
        buf = shard.buffer(f"recv{idx}", (world * shard.max_rows, w), dev)
        if comm is not None:
            produced = torch.cuda.Event()
            produced.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(produced)
                if timings is not None:
                    timings["events"].append((f"gather{idx}_start", mark(comm)))
                dist.all_gather_into_tensor(buf, send, group=group)
                if timings is not None:
                    timings["events"].append((f"gather{idx}_done", mark(comm)))
                done = torch.cuda.Event()
                done.record(comm)
            ready.append(done)
        else:
            dist.all_gather_into_tensor(buf, send, group=group)
            ready.append(None)
        recv.append(buf)
    for idx, (c, w) in enumerate(panels):
        if ready[idx] is not None:
            main.wait_event(ready[idx])
        if timings is not None:
            timings["events"].append((f"spmm{idx}_start", mark(main)))
        spmm_fn(shard, recv[idx], out[:, c:c + w], relu)
        if timings is not None:
            timings["events"].append((f"spmm{idx}_done", mark(main)))
    return out


def gcn_forward_sharded(shard: ShardedCsr, x_local: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor,
                        panel: int = 64, group=None, spmm_fn: Optional[Callable] = None,
                        timings: Optional[dict] = None) -> torch.Tensor:
    """This rank's rows of  A_hat ReLU(A_hat X W1) W2  (reference caller: bench/bench_gcn.py:314-329).
    ``timings``: optional dict that receives ("name", cuda event) pairs marking each phase."""
    h = sharded_layer(shard, x_local, W1, relu=True, panel=panel, group=group, spmm_fn=spmm_fn,
                      timings=timings)
    return sharded_layer(shard, h, W2, relu=False, panel=panel, group=group, spmm_fn=spmm_fn,
                         timings=timings)


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
