"""Row-sharded GCN forward: on 2 GPUs (NCCL all-gather per layer and row chunk, overlapped with
the SpMM of earlier chunks) against the single-GPU result and the float64 oracle (skipped on
boxes with one GPU), and the chunked accumulation on one GPU against the one-launch layers."""
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


@pytest.mark.parametrize("chunks", [1, 3, 8])
def test_chunked_gcn_one_gpu_matches_unchunked(oracle, chunks):
    """World size 1: the row block split into `chunks` sub-matrices, each layer accumulated
    chunk by chunk (heavy rows included), equals the two full-width SpMM launches."""
    from scorch_b200 import pipelines as P, sharded as S, workloads as W
    n = 30000
    g = W.gcn_graph(n, mean_deg=30.0, max_deg=9000, seed=1).to("cuda")
    X = W.randn_on((n, 256), seed=2).cuda()
    W1, W2 = W.glorot(256, 256, seed=0).cuda(), W.glorot(256, 64, seed=1).cuda()
    shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, 0, 1, chunks=chunks)
    tl = S.Timeline()
    for _ in range(2):
        out = S.gcn_forward_sharded(shard, X, W1, W2, timeline=tl)
    assert any(b.plan.segments > 0 for b in shard.blocks)   # heavy rows survive the split
    single = P.gcn_forward(g.pos, g.crd, g.val, X, W1, W2)
    torch.testing.assert_close(out, single, rtol=1e-4, atol=1e-5)
    phases = tl.summary()
    assert phases["spmm_layer1"] > 0 and phases["spmm_layer2"] > 0 and phases["dense_transform"] > 0
    # sampled rows of layer 1 against the float64 oracle on the library's own dense operand
    xw = torch.matmul(X, W1)
    h = shard._buffers[("hidden", (n, 256))]
    rows = torch.cat([torch.arange(0, n, 997), (g.pos[1:] - g.pos[:-1]).argmax().reshape(1).cpu()])
    pos, crd, val = g.pos.cpu().numpy(), g.crd.cpu().numpy(), g.val.cpu().numpy()
    xw_h = xw.cpu().numpy()
    for r in rows.tolist():
        b, e = pos[r], pos[r + 1]
        want = np.maximum((val[b:e, None].astype(np.float64) * xw_h[crd[b:e]].astype(np.float64)).sum(0), 0)
        ok, err, bad = oracle.allclose_report(h[r].cpu().numpy(), want, 1e-4, 1e-5)
        assert ok, (r, err, bad)


def test_replicated_operand_row_blocks(oracle):
    """Row blocks of a rectangular matrix against a dense operand every rank holds: the blocks'
    results stacked in rank order are the whole product (no communication involved)."""
    from scorch_b200 import kernels as K, sharded as S, workloads as W
    A = W.csr_uniform(3000, 5000, 0.01, seed=4).to("cuda")
    B = W.dense_normal(5000, 64, seed=5).cuda()
    whole = K.spmm_csr(A.pos, A.crd, A.val, B)
    parts = []
    for rank in range(3):
        blk, bounds = S.row_block(A.pos, A.crd, A.val, rank, 3)
        assert blk.rows == bounds[rank + 1] - bounds[rank]
        parts.append(S.sharded_spmm_replicated(blk, B))
    assert torch.equal(torch.cat(parts, 0), whole)
