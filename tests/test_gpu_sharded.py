"""Row-sharded GCN forward on 2 GPUs (NCCL all-gather per layer, panel overlap) against the
single-GPU result and the float64 oracle.  Skipped on boxes with one GPU."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from scorch_b200 import sharded as S, workloads as W
        g = W.gcn_graph(n, mean_deg=30.0, max_deg=5000, seed=0).to("cuda")
        X = W.randn_on((n, 256), seed=1).cuda()
        W1, W2 = W.glorot(256, 256, seed=0).cuda(), W.glorot(256, 64, seed=1).cuda()
        shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, rank, world)
        r0, r1 = shard.bounds[rank], shard.bounds[rank + 1]
        for _ in range(2):  # twice: buffers and streams are reused across steps
            out = S.gcn_forward_sharded(shard, X[r0:r1].contiguous(), W1, W2)
        full = S.gather_rows(shard, out)
        torch.cuda.synchronize()
        if rank == 0:
            torch.save(full.cpu(), tmp)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_gcn_two_gpus(tmp_path, oracle):
    from scorch_b200 import pipelines as P, workloads as W
    n = 20000
    tmp = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, _free_port(), n, tmp), nprocs=2, join=True)
    got = torch.load(tmp)
    g = W.gcn_graph(n, mean_deg=30.0, max_deg=5000, seed=0)
    X = W.randn_on((n, 256), seed=1)
    W1, W2 = W.glorot(256, 256, seed=0), W.glorot(256, 64, seed=1)
    single = P.gcn_forward(g.pos.cuda(), g.crd.cuda(), g.val.cuda(), X.cuda(), W1.cuda(), W2.cuda()).cpu()
    torch.testing.assert_close(got, single, rtol=1e-4, atol=1e-5)
    pos, crd, val = g.pos.numpy(), g.crd.numpy(), g.val.numpy()
    h = np.maximum(oracle.spmm_csr_acc64(pos, crd, val, (X.double() @ W1.double()).float().numpy()), 0)
    want = oracle.spmm_csr_acc64(pos, crd, val, (h @ W2.double().numpy()).astype(np.float32))
    ok, err, bad = oracle.allclose_report(got.numpy(), want, 2e-3, 1e-4)
    assert ok, (err, bad)
