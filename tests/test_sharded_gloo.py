"""Host logic of the row-sharded layers (partition, padded all-gather layout, column remap,
panel loop) on CPU ranks: world size 2 and 3 over gloo, the oracle standing in for the CUDA SpMM."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_spmm(shard, B, out, relu):
    from oracle import oracle as O
    r = O.spmm_csr_acc64(shard.pos.numpy(), shard.crd.numpy(), shard.val.numpy(),
                         B.contiguous().numpy(), None, relu)
    out.copy_(torch.from_numpy(r.astype(np.float32)))


def _worker(rank, world, port, n, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from scorch_b200 import sharded as S, workloads as W
        g = W.gcn_graph(n, mean_deg=6.0, max_deg=400, seed=0)
        X = W.randn_on((n, 24), seed=1)
        W1, W2 = W.glorot(24, 40, seed=0), W.glorot(40, 8, seed=1)
        shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, rank, world)
        r0, r1 = shard.bounds[rank], shard.bounds[rank + 1]
        out = S.gcn_forward_sharded(shard, X[r0:r1].contiguous(), W1, W2, panel=(8, 16), panel2=4,
                                    spmm_fn=_oracle_spmm)
        one = S.sharded_layer(shard, X[r0:r1].contiguous(), W1, relu=True, panel=16, spmm_fn=_oracle_spmm)
        assert one.shape == (r1 - r0, 40)
        full = S.gather_rows(shard, out)
        if rank == 0:
            torch.save({"out": full, "bounds": shard.bounds, "max_rows": shard.max_rows}, tmp)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_gcn_matches_single_process(tmp_path, world):
    from oracle import oracle as O
    from scorch_b200 import sharded as S, workloads as W
    n = 1500
    tmp = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(world, _free_port(), n, tmp), nprocs=world, join=True)
    got = torch.load(tmp)
    g = W.gcn_graph(n, mean_deg=6.0, max_deg=400, seed=0)
    X = W.randn_on((n, 24), seed=1)
    W1, W2 = W.glorot(24, 40, seed=0), W.glorot(40, 8, seed=1)
    pos, crd, val = g.pos.numpy(), g.crd.numpy(), g.val.numpy()
    h = O.spmm_csr_acc64(pos, crd, val, (X @ W1).numpy(), None, True).astype(np.float32)
    want = O.spmm_csr_acc64(pos, crd, val, (torch.from_numpy(h) @ W2).numpy())
    np.testing.assert_allclose(got["out"].numpy(), want, rtol=1e-4, atol=1e-5)
    # blocks are balanced by stored entries, contiguous and cover every row once
    b = got["bounds"]
    assert b[0] == 0 and b[-1] == n and all(b[i] <= b[i + 1] for i in range(world))
    nnz = np.diff(pos[np.array(b)])
    assert nnz.max() - nnz.min() <= 2 * np.diff(pos).max()
    assert got["max_rows"] == max(b[i + 1] - b[i] for i in range(world))


def test_row_bounds_host_matches_definition():
    from scorch_b200 import sharded as S
    pos = torch.tensor([0, 0, 5, 5, 9, 20, 21, 21, 30], dtype=torch.int32)
    b = S.row_bounds(pos, 3)
    # block g starts at the first row r with pos[r] >= g*nnz/3
    assert b == [0, 4, 4, 8] or b == [0, int(np.searchsorted(pos.numpy(), 10)), int(np.searchsorted(pos.numpy(), 20)), 8]
    assert S.row_bounds(pos, 1) == [0, 8]
