"""Host logic of the row-sharded layers (partition, padded all-gather layout, split of the row
block by operand row chunk, column remap, chunk loop with accumulation) on CPU ranks: world size
2 and 3 over gloo, the oracle standing in for the CUDA SpMM."""
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


def _oracle_spmm(block, B, out, relu, accumulate=False):
    from oracle import oracle as O
    r = O.spmm_csr_acc64(block.pos.numpy(), block.crd.numpy(), block.val.numpy(),
                         B.contiguous().numpy())
    if accumulate:
        r = r + out.numpy().astype(np.float64)
    if relu:
        r = np.maximum(r, 0)
    out.copy_(torch.from_numpy(r.astype(np.float32)))


def _worker(rank, world, port, n, chunks, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from scorch_b200 import sharded as S, workloads as W
        g = W.gcn_graph(n, mean_deg=6.0, max_deg=400, seed=0)
        X = W.randn_on((n, 24), seed=1)
        W1, W2 = W.glorot(24, 40, seed=0), W.glorot(40, 8, seed=1)
        shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, rank, world, chunks=chunks)
        want_chunks = chunks if isinstance(chunks, int) else len(chunks)
        assert shard.chunks == want_chunks and sum(b.nnz for b in shard.blocks) == shard.nnz
        assert sum(b.nnz for b in shard.splits[-1].blocks) == shard.nnz
        r0, r1 = shard.bounds[rank], shard.bounds[rank + 1]
        out = S.gcn_forward_sharded(shard, X[r0:r1].contiguous(), W1, W2, spmm_fn=_oracle_spmm)
        one = S.sharded_layer(shard, X[r0:r1].contiguous(), W1, relu=True, spmm_fn=_oracle_spmm)
        assert one.shape == (r1 - r0, 40)
        # the same forward without look-ahead, and its first layer alone (what the host-tensor front end calls)
        out0 = S.gcn_forward_sharded(shard, X[r0:r1].contiguous(), W1, W2, spmm_fn=_oracle_spmm, lookahead=0)
        assert torch.equal(out0, out)
        hid = S.gcn_forward_sharded(shard, X[r0:r1].contiguous(), W1, W2, spmm_fn=_oracle_spmm,
                                    first_layer_only=True)
        assert torch.equal(hid, one)
        full, full_one = S.gather_rows(shard, out), S.gather_rows(shard, one)
        if rank == 0:
            torch.save({"out": full, "one": full_one, "bounds": shard.bounds, "max_rows": shard.max_rows,
                        "offsets": shard.splits[0].offsets}, tmp)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 3), (3, 4), (2, [1, 1, 2, 3])])
def test_sharded_gcn_matches_single_process(tmp_path, world, chunks):
    from oracle import oracle as O
    from scorch_b200 import sharded as S, workloads as W
    n = 1500
    tmp = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(world, _free_port(), n, chunks, tmp), nprocs=world, join=True)
    got = torch.load(tmp)
    g = W.gcn_graph(n, mean_deg=6.0, max_deg=400, seed=0)
    X = W.randn_on((n, 24), seed=1)
    W1, W2 = W.glorot(24, 40, seed=0), W.glorot(40, 8, seed=1)
    pos, crd, val = g.pos.numpy(), g.crd.numpy(), g.val.numpy()
    h = O.spmm_csr_acc64(pos, crd, val, (X @ W1).numpy(), None, True).astype(np.float32)
    want = O.spmm_csr_acc64(pos, crd, val, (torch.from_numpy(h) @ W2).numpy())
    np.testing.assert_allclose(got["out"].numpy(), want, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(got["one"].numpy(), h, rtol=1e-4, atol=1e-5)
    # blocks are balanced by stored entries, contiguous and cover every row once
    b = got["bounds"]
    assert b[0] == 0 and b[-1] == n and all(b[i] <= b[i + 1] for i in range(world))
    nnz = np.diff(pos[np.array(b)])
    assert nnz.max() - nnz.min() <= 2 * np.diff(pos).max()
    largest = max(b[i + 1] - b[i] for i in range(world))
    off = got["offsets"]
    assert got["max_rows"] == largest == off[-1] and off[0] == 0 and off == sorted(off)
    if not isinstance(chunks, int):   # pieces in the requested proportions (to rounding)
        sizes = np.diff(off)
        assert np.all(np.abs(sizes - largest * np.array(chunks) / sum(chunks)) <= 1)


def test_chunk_split_single_process_keeps_every_entry():
    """One rank, several chunks: each sub-matrix holds the entries of its column range with
    columns renumbered from the chunk's first row, ascending within a row."""
    from scorch_b200 import sharded as S, workloads as W
    n = 700
    g = W.gcn_graph(n, mean_deg=5.0, max_deg=200, seed=3)
    shard = S.ShardedCsr.from_global(g.pos, g.crd, g.val, 0, 1, chunks=4, chunks2=[1, 2, 4])
    assert [sp.chunks for sp in shard.splits] == [4, 3]
    want = g.torch_csr().to_dense()
    for split in shard.splits:
        dense = torch.zeros((n, n), dtype=torch.float32)
        for c, blk in enumerate(split.blocks):
            lens = (blk.pos[1:] - blk.pos[:-1]).long()
            rows = torch.repeat_interleave(torch.arange(n), lens)
            assert blk.nnz == 0 or int(blk.crd.max()) < split.rows_of(c)
            d = (blk.crd[1:] - blk.crd[:-1])[rows[1:] == rows[:-1]]
            assert bool((d > 0).all())
            dense[rows, blk.crd.long() + split.offsets[c]] += blk.val
        assert torch.equal(dense, want)


def test_chunk_offsets():
    from scorch_b200 import sharded as S
    assert S.chunk_offsets(100, 4) == [0, 25, 50, 75, 100]
    assert S.chunk_offsets(10, [1, 1, 2]) == [0, 3, 5, 10]
    assert S.chunk_offsets(2, 4) == [0, 1, 1, 2, 2]          # more pieces than rows: empty pieces
    assert S.chunk_offsets(7, 1) == [0, 7]
    with pytest.raises(ValueError):
        S.chunk_offsets(7, [1, 0])


def test_row_bounds_host_matches_definition():
    from scorch_b200 import sharded as S
    pos = torch.tensor([0, 0, 5, 5, 9, 20, 21, 21, 30], dtype=torch.int32)
    b = S.row_bounds(pos, 3)
    # block g starts at the first row r with pos[r] >= g*nnz/3
    assert b == [0, 4, 4, 8] or b == [0, int(np.searchsorted(pos.numpy(), 10)), int(np.searchsorted(pos.numpy(), 20)), 8]
    assert S.row_bounds(pos, 1) == [0, 8]


def _spmv_spgemm_worker(rank, world, port, n, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from scorch_b200 import sharded as S, workloads as W
        A = W.powerlaw_square(n, mean_nnz=5.0, seed=2)
        x = W.randn_on((n,), seed=3)
        # SpMV: rows balanced by stored entries, x replicated, y gathered
        blk, bounds = S.row_block(A.pos, A.crd, A.val, rank, world)
        spmv = lambda b, v: torch.from_numpy(O.spmv_csr(b.pos.numpy(), b.crd.numpy(), b.val.numpy(), v.numpy()))
        y = S.gather_vector(S.sharded_spmv(blk, x, spmv_fn=spmv), bounds)
        # SpGEMM: rows balanced by products, B replicated, pointers offset by the ranks before
        pb = S.product_bounds(A.pos, A.crd, A.pos, world)
        ablk, _ = S.row_block(A.pos, A.crd, A.val, rank, world, bounds=pb)

        def spgemm(b, Bp, Bc, Bv, nn):
            p, c, v = O.spgemm(b.pos.numpy(), b.crd.numpy(), b.val.numpy(), Bp.numpy(), Bc.numpy(), Bv.numpy(), nn)
            return torch.from_numpy(p), torch.from_numpy(c), torch.from_numpy(v)
        cpos, ccrd, cval, offset, total = S.sharded_spgemm(ablk, A.pos, A.crd, A.val, n, spgemm_fn=spgemm)
        torch.save({"y": y, "pb": pb, "cpos": cpos, "ccrd": ccrd, "cval": cval, "offset": offset,
                    "total": total, "unit_range": S.unit_range(32, rank, world)}, f"{tmp}.{rank}")
    finally:
        dist.destroy_process_group()


def test_sharded_spmv_and_spgemm_match_single_process(tmp_path):
    from oracle import oracle as O
    from scorch_b200 import workloads as W
    n, world = 1200, 2
    tmp = str(tmp_path / "out.pt")
    mp.spawn(_spmv_spgemm_worker, args=(world, _free_port(), n, tmp), nprocs=world, join=True)
    parts = [torch.load(f"{tmp}.{r}") for r in range(world)]
    A = W.powerlaw_square(n, mean_nnz=5.0, seed=2)
    x = W.randn_on((n,), seed=3)
    pos, crd, val = A.pos.numpy(), A.crd.numpy(), A.val.numpy()
    want_y = O.spmv_csr(pos, crd, val, x.numpy())
    for p in parts:
        assert np.array_equal(p["y"].numpy(), want_y)
    wpos, wcrd, wval = O.spgemm(pos, crd, val, pos, crd, val, n)
    pb = parts[0]["pb"]
    assert pb[0] == 0 and pb[-1] == n and parts[1]["pb"] == pb
    # the ranks' arrays concatenated, pointers offset, are the whole product bit for bit
    gpos = np.concatenate([parts[0]["cpos"].numpy()[:-1] + parts[0]["offset"],
                           parts[1]["cpos"].numpy() + parts[1]["offset"]])
    assert parts[0]["offset"] == 0 and parts[1]["offset"] == parts[0]["ccrd"].numel()
    assert parts[0]["total"] == parts[1]["total"] == len(wcrd)
    assert np.array_equal(gpos, wpos)
    assert np.array_equal(np.concatenate([p["ccrd"].numpy() for p in parts]), wcrd)
    assert np.array_equal(np.concatenate([p["cval"].numpy() for p in parts]), wval)
    # products are balanced: each block within one row's worth of half the total
    lens = np.diff(pos)
    prods = np.concatenate([[0], np.cumsum(lens[crd])])[pos]
    assert abs((prods[pb[1]] - prods[0]) - prods[-1] / 2) <= lens[crd].max() * lens.max()
    assert [p["unit_range"] for p in parts] == [(0, 16), (16, 32)]
