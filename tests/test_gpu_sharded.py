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
        # the host-tensor front end: this rank's rows from pinned memory and back
        from scorch_b200 import pipelines as P
        host = P.HostGcnForward(g.pos, g.crd, g.val, W1, W2, rank, world)
        back = host(X[r0:r1].cpu().pin_memory())
        assert torch.allclose(back, out.cpu(), rtol=1e-4, atol=1e-5)
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


@pytest.mark.parametrize("chunks", [1, 3, 8, [1, 1, 2, 2, 2]])
def test_chunked_gcn_one_gpu_matches_unchunked(oracle, chunks):
    """World size 1: the row block split into `chunks` sub-matrices, each layer accumulated
    chunk by chunk (heavy rows included), equals the two full-width SpMM launches."""
    from scorch_b200 import pipelines as P, sharded as S, workloads as W
    n = 30000
    g = W.gcn_graph(n, mean_deg=30.0, max_deg=9000, seed=1).to("cuda")
    X = W.randn_on((n, 256), seed=2).cuda()
    W1, W2 = W.glorot(256, 256, seed=0).cuda(), W.glorot(256, 64, seed=1).cuda()
    shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, 0, 1, chunks=chunks,
                                     chunks2=8 if isinstance(chunks, list) else None)
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


@pytest.mark.parametrize("in_chunks,out_blocks", [(16, 16), (8, 8), (3, 5), (1, 1)])
def test_host_tensor_gcn_forward_overlaps_copies_and_matches(oracle, in_chunks, out_blocks):
    """Features in pinned host memory, result back there: chunked host-to-device copy feeding the
    accumulating first-layer passes, second layer in row blocks copied back as they finish."""
    from scorch_b200 import pipelines as P, workloads as W
    n = 20000
    g = W.gcn_graph(n, mean_deg=30.0, max_deg=5000, seed=0).to("cuda")
    X = W.randn_on((n, 256), seed=1)
    W1, W2 = W.glorot(256, 256, seed=0).cuda(), W.glorot(256, 64, seed=1).cuda()
    host = P.HostGcnForward(g.pos, g.crd, g.val, W1, W2, in_chunks=in_chunks, out_blocks=out_blocks)
    xh = X.pin_memory()
    out1 = host(xh).clone()
    out_h = torch.empty((n, 64), dtype=torch.float32).pin_memory()
    out2 = host(xh, out_h)                       # buffers and streams are reused across calls
    assert out2 is out_h and torch.equal(out1, out2)
    single = P.gcn_forward(g.pos, g.crd, g.val, X.cuda(), W1, W2).cpu()
    torch.testing.assert_close(out2, single, rtol=1e-4, atol=1e-5)
    pos, crd, val = (t.cpu().numpy() for t in (g.pos, g.crd, g.val))
    h = np.maximum(oracle.spmm_csr_acc64(pos, crd, val, (X.double() @ W1.cpu().double()).float().numpy()), 0)
    want = oracle.spmm_csr_acc64(pos, crd, val, (h @ W2.cpu().double().numpy()).astype(np.float32))
    ok, err, bad = oracle.allclose_report(out2.numpy(), want, 2e-3, 1e-4)
    assert ok, (err, bad)


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


def _spmv_spgemm_worker(rank, world, port, n, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from scorch_b200 import sharded as S, workloads as W
        A = W.powerlaw_square(n, mean_nnz=6.0, seed=2).to("cuda")
        x = W.randn_on((n,), seed=3).cuda()
        blk, bounds = S.row_block(A.pos, A.crd, A.val, rank, world)
        y = S.gather_vector(S.sharded_spmv(blk, x), bounds)
        pb = S.product_bounds(A.pos, A.crd, A.pos, world)
        ablk, _ = S.row_block(A.pos, A.crd, A.val, rank, world, bounds=pb)
        cpos, ccrd, cval, offset, total = S.sharded_spgemm(ablk, A.pos, A.crd, A.val, n)
        torch.cuda.synchronize()
        torch.save({"y": y.cpu(), "cpos": cpos.cpu(), "ccrd": ccrd.cpu(), "cval": cval.cpu(),
                    "offset": offset, "total": total}, f"{tmp}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_spmv_and_spgemm_two_gpus(tmp_path, oracle):
    from scorch_b200 import workloads as W
    n = 30000
    tmp = str(tmp_path / "out.pt")
    mp.spawn(_spmv_spgemm_worker, args=(2, _free_port(), n, tmp), nprocs=2, join=True)
    parts = [torch.load(f"{tmp}.{r}") for r in range(2)]
    A = W.powerlaw_square(n, mean_nnz=6.0, seed=2)
    x = W.randn_on((n,), seed=3)
    pos, crd, val = A.pos.numpy(), A.crd.numpy(), A.val.numpy()
    ok, err, bad = oracle.allclose_report(parts[0]["y"].numpy(), oracle.spmv_csr_acc64(pos, crd, val, x.numpy()),
                                          1e-4, 1e-5)
    assert ok, (err, bad)
    assert torch.equal(parts[0]["y"], parts[1]["y"])
    wpos, wcrd, _ = oracle.spgemm(pos, crd, val, pos, crd, val, n)
    gpos = np.concatenate([parts[0]["cpos"].numpy()[:-1] + parts[0]["offset"],
                           parts[1]["cpos"].numpy() + parts[1]["offset"]])
    assert np.array_equal(gpos, wpos) and parts[0]["total"] == len(wcrd)
    assert np.array_equal(np.concatenate([p["ccrd"].numpy() for p in parts]), wcrd)
    want = oracle.spgemm_values_acc64(pos, crd, val, pos, crd, val, n, wpos, wcrd)
    ok, err, bad = oracle.allclose_report(np.concatenate([p["cval"].numpy() for p in parts]), want, 1e-4, 1e-5)
    assert ok, (err, bad)


def test_sharded_spgemm_single_process_has_no_offset(oracle):
    from scorch_b200 import sharded as S, workloads as W
    A = W.powerlaw_square(4000, mean_nnz=5.0, seed=9).to("cuda")
    blk, bounds = S.row_block(A.pos, A.crd, A.val, 0, 1)
    cpos, ccrd, cval, offset, total = S.sharded_spgemm(blk, A.pos, A.crd, A.val, 4000)
    assert offset == 0 and total == ccrd.numel() and bounds == [0, 4000]
    wpos, wcrd, _ = oracle.spgemm(*(t.cpu().numpy() for t in (A.pos, A.crd, A.val, A.pos, A.crd, A.val)), 4000)
    assert np.array_equal(cpos.cpu().numpy(), wpos) and np.array_equal(ccrd.cpu().numpy(), wcrd)
