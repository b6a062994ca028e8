"""The reference-facing front end (scorch_b200.matmul / einsum / spmm_bias_act and the legacy COO
symbols) on host tensors, end to end through the CUDA kernels, against dense torch products —
the oracle style of the reference's own tests (tests/test_scorch/test_matmul_dispatch.py,
test_kernels_comprehensive.py, test_compile.py)."""
from __future__ import annotations

import warnings

import numpy as np
import pytest
import torch

import scorch_b200 as scorch
from scorch_b200 import scorch_ops
from scorch_b200.stensor import STensor

pytestmark = pytest.mark.gpu
warnings.filterwarnings("ignore", message=".*Sparse CSR tensor support.*")
warnings.filterwarnings("ignore", message=".*Sparse invariant checks.*")


def sparse_dense(m, n, density, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    d = torch.rand((m, n), generator=g)
    d = torch.where(torch.rand((m, n), generator=g) < density, d + 0.1, torch.zeros(()))
    return d.to(dtype)


def test_matmul_csr_dense_returns_host_tensor_and_time_dict():
    A, B = sparse_dense(200, 150, 0.1, 0), torch.rand(150, 24)
    t = {}
    C = scorch.matmul(A.to_sparse_csr(), B, format="dd", time_dict=t)
    assert isinstance(C, torch.Tensor) and not C.is_cuda and "eval_time" in t
    torch.testing.assert_close(C, A @ B, rtol=1e-4, atol=1e-5)
    # device operands stay on the device
    Cd = scorch.matmul(STensor.from_torch(A.to_sparse_csr()).cuda(), B.cuda())
    assert Cd.is_cuda
    torch.testing.assert_close(Cd.cpu(), A @ B, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float64, torch.int32, torch.int64])
def test_matmul_typed_registry_paths(dtype):
    A = (sparse_dense(60, 50, 0.2, 1) * 7).to(dtype)
    B = (torch.rand(50, 9) * 5).to(dtype)
    x = (torch.rand(50) * 5).to(dtype)
    C = scorch.matmul(A.to_sparse_csr(), B)
    y = scorch.matmul(A.to_sparse_csr(), x)
    if dtype.is_floating_point:
        torch.testing.assert_close(C, A @ B)
        torch.testing.assert_close(y, A @ x)
    else:
        assert torch.equal(C, A @ B) and torch.equal(y, A @ x)


def test_matmul_csr_csr_returns_sparse_stensor_with_sorted_columns():
    A, B = sparse_dense(120, 90, 0.08, 2), sparse_dense(90, 110, 0.08, 3)
    C = scorch.matmul(A.to_sparse_csr(), B.to_sparse_csr())
    assert isinstance(C, STensor) and str(C.format) == "d,s" and C.shape == (120, 110)
    pos, crd = C.index.mode_indices[1]
    assert pos.dtype == torch.int32 and crd.dtype == torch.int32
    for i in range(120):
        row = crd[pos[i]:pos[i + 1]]
        assert (row[1:] > row[:-1]).all()
    torch.testing.assert_close(C.to_torch().to_dense(), A @ B, rtol=1e-4, atol=1e-5)
    # two torch COO operands are converted to CSR first, like the reference (ops.py:256-258)
    C2 = scorch.matmul(A.to_sparse_coo(), B.to_sparse_coo())
    torch.testing.assert_close(C2.to_torch().to_dense(), A @ B, rtol=1e-4, atol=1e-5)


def test_spmv_through_matmul_and_einsum():
    A, x = sparse_dense(300, 280, 0.05, 4), torch.rand(280)
    torch.testing.assert_close(scorch.matmul(A.to_sparse_csr(), x), A @ x, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(scorch.einsum("ij,j->i", A.to_sparse_csr(), x), A @ x, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(scorch.einsum("ij,jk->ik", A.to_sparse_csr(), torch.eye(280)), A,
                               rtol=1e-4, atol=1e-5)


def test_legacy_coo_symbols():
    A, B = sparse_dense(70, 60, 0.1, 5), torch.rand(60, 12)
    coo = A.to_sparse_coo().coalesce()
    row, col = coo.indices()[0].int(), coo.indices()[1].int()
    r = scorch_ops.spmm_coo_float([70, 12], [70, 60], [[row], [col]], coo.values(), [60, 12], [[], []], B.flatten())
    torch.testing.assert_close(r.storage.value.view(70, 12), A @ B, rtol=1e-4, atol=1e-5)
    # through the front end: a COO STensor times a dense matrix resolves to spmm_coo_float
    C = scorch.matmul(STensor.from_coo(coo), B)
    torch.testing.assert_close(C, A @ B, rtol=1e-4, atol=1e-5)
    B2 = sparse_dense(60, 80, 0.1, 6).to_sparse_coo().coalesce()
    r = scorch_ops.spmspm_coo_float([70, 80], [70, 60], [[row], [col]], coo.values(), [60, 80],
                                    [[B2.indices()[0].int()], [B2.indices()[1].int()]], B2.values())
    rr, cc = r.storage.index.mode_indices[0][0], r.storage.index.mode_indices[1][0]
    got = torch.sparse_coo_tensor(torch.stack([rr, cc]).long(), r.storage.value, (70, 80)).to_dense()
    torch.testing.assert_close(got, A @ B2.to_dense(), rtol=1e-4, atol=1e-5)
    key = rr.long() * 80 + cc.long()
    assert (key[1:] > key[:-1]).all()  # rows ascending, columns ascending within a row


@pytest.mark.parametrize("relu", [False, True])
def test_fused_bias_activation_layer(relu):
    # what @scorch.compile reaches for relu(A @ B + bias) (reference tests/test_scorch/test_compile.py:70-127)
    A, B, bias = sparse_dense(90, 70, 0.1, 7) - 0.3, torch.rand(70, 16) - 0.5, torch.rand(16) - 0.5
    A = torch.where(A > -0.25, A, torch.zeros(()))
    got = scorch.spmm_bias_act(A.to_sparse_csr(), B, bias, relu)
    want = A @ B + bias
    torch.testing.assert_close(got, want.relu() if relu else want, rtol=1e-4, atol=1e-5)


def test_sddmm_coo_and_csr_masks_vs_dense():
    # reference tests/test_scorch/test_kernels_comprehensive.py:330-411
    M, Q, K = sparse_dense(50, 40, 0.2, 8), torch.rand(50, 32), torch.rand(40, 32)
    want = M * (Q @ K.t())
    for mask in (M.to_sparse_coo(), M.to_sparse_csr()):
        for expr, Kop in (("ij,ik,jk->ij", K), ("ij,ik,kj->ij", K.t().contiguous())):
            r = scorch.einsum(expr, mask, Q, Kop)
            assert str(r.format) == "o,o"
            torch.testing.assert_close(r.to_torch().to_dense(), want, rtol=1e-4, atol=1e-5)


def test_unsupported_patterns_raise_instead_of_falling_back():
    with pytest.raises(NotImplementedError):
        scorch.matmul(sparse_dense(8, 8, 0.5, 9).to_sparse_csr(), torch.rand(8, 4), format="ds")
    with pytest.raises(NotImplementedError):
        scorch.einsum("ij,ij->ij", sparse_dense(8, 8, 0.5, 9).to_sparse_csr(), torch.rand(8, 8))
