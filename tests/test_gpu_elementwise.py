"""Element-wise product and sum of two sparse matrices (the first of the patterns the reference
compiles rather than dispatches to a prebuilt kernel): golden vectors from the reference's own
``einsum("ij,ij->ij")`` / ``A + B``, the numpy oracle on random inputs with hub rows and empty
rows, every value type, and the front end for compressed and coordinate operands."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def random_csr(m, n, lens, seed, dtype=np.float32):
    rng = np.random.default_rng(seed)
    lens = np.minimum(np.asarray(lens, np.int64), n)
    pos = np.zeros(m + 1, np.int64)
    np.cumsum(lens, out=pos[1:])
    crd = np.empty(pos[-1], np.int32)
    for i in range(m):
        if lens[i]:
            crd[pos[i]:pos[i + 1]] = np.sort(rng.choice(n, size=lens[i], replace=False))
    val = rng.integers(-9, 10, size=pos[-1]).astype(dtype) if np.dtype(dtype).kind == "i" \
        else rng.standard_normal(pos[-1]).astype(dtype)
    return pos.astype(np.int32), crd, val


@pytest.mark.parametrize("op", ["mul", "add"])
def test_elementwise_golden_from_the_reference(golden, op):
    from scorch_b200 import kernels as K
    g = golden.case("ewise_f32")
    assert str(g[f"{op}_format"][0]) == "d,s"
    cpos, ccrd, cval = K.csr_ewise(op, dev(g["Apos"]), dev(g["Acrd"]), dev(g["Aval"]), dev(g["Bpos"]),
                                   dev(g["Bcrd"]), dev(g["Bval"]))
    assert np.array_equal(cpos.cpu().numpy(), g[f"{op}_pos"])
    assert np.array_equal(ccrd.cpu().numpy(), g[f"{op}_crd"])
    np.testing.assert_allclose(cval.cpu().numpy(), g[f"{op}_val"], rtol=1e-6, atol=0)


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64])
@pytest.mark.parametrize("op", ["mul", "add"])
def test_elementwise_vs_oracle(oracle, op, dtype):
    from scorch_b200 import kernels as K
    m, n = 300, 500
    la = np.random.default_rng(1).poisson(8, size=m)
    lb = np.random.default_rng(2).poisson(8, size=m)
    la[[0, 7]] = 0
    lb[[0, 9]] = 0
    la[20], lb[20] = 400, 450          # long rows with many common columns
    la[21], lb[21] = 300, 0
    Ap, Ac, Av = random_csr(m, n, la, seed=3, dtype=dtype)
    Bp, Bc, Bv = random_csr(m, n, lb, seed=4, dtype=dtype)
    cpos, ccrd, cval = K.csr_ewise(op, dev(Ap), dev(Ac), dev(Av), dev(Bp), dev(Bc), dev(Bv))
    wpos, wcrd, wval = oracle.csr_ewise(op, Ap, Ac, Av, Bp, Bc, Bv)
    assert np.array_equal(cpos.cpu().numpy(), wpos)
    assert np.array_equal(ccrd.cpu().numpy(), wcrd)
    assert np.array_equal(cval.cpu().numpy(), wval)    # one multiply or add per entry: bit-exact


def test_elementwise_keeps_cancelled_sums_and_handles_empty_matrices():
    from scorch_b200 import kernels as K
    pos = np.array([0, 2, 2], np.int32)
    crd = np.array([1, 3], np.int32)
    a, b = np.array([2.0, 1.0], np.float32), np.array([-2.0, 5.0], np.float32)
    cpos, ccrd, cval = K.csr_ewise("add", dev(pos), dev(crd), dev(a), dev(pos), dev(crd), dev(b))
    assert cpos.tolist() == [0, 2, 2] and ccrd.tolist() == [1, 3] and cval.tolist() == [0.0, 6.0]
    z = np.zeros(3, np.int32)
    e = np.zeros(0, np.int32)
    for op in ("mul", "add"):
        cpos, ccrd, cval = K.csr_ewise(op, dev(z), dev(e), dev(e.astype(np.float32)), dev(z), dev(e),
                                       dev(e.astype(np.float32)))
        assert cpos.tolist() == [0, 0, 0] and ccrd.numel() == 0 and cval.numel() == 0


@pytest.mark.parametrize("fmt", ["csr", "coo"])
def test_front_end_einsum_and_add(fmt):
    """``einsum("ij,ij->ij")`` and ``+`` on host tensors, like the reference's tests
    (tests/test_scorch/test_kernels_comprehensive.py:119-200): compare with dense torch."""
    import scorch_b200 as scorch
    g = torch.Generator().manual_seed(100)
    a = torch.rand(25, 25, generator=g) * (torch.rand(25, 25, generator=g) < 0.3)
    b = torch.rand(25, 25, generator=g) * (torch.rand(25, 25, generator=g) < 0.3)
    to = (lambda t: t.to_sparse_csr()) if fmt == "csr" else (lambda t: t.to_sparse_coo())
    a_st, b_st = scorch.STensor.from_torch(to(a)), scorch.STensor.from_torch(to(b))
    prod = scorch.einsum("ij,ij->ij", a_st, b_st, format="ds" if fmt == "csr" else "oo")
    total = a_st + b_st
    assert str(prod.format) == str(total.format) == ("d,s" if fmt == "csr" else "o,o")
    assert not prod.values.is_cuda
    assert torch.allclose(prod.to_torch().to_dense(), a * b, atol=1e-6)
    assert torch.allclose(total.to_torch().to_dense(), a + b, atol=1e-6)
    assert total.nnz() == int(((a != 0) | (b != 0)).sum()) and prod.nnz() == int(((a != 0) & (b != 0)).sum())
    with pytest.raises(NotImplementedError):
        scorch.einsum("ij,ij->ij", a_st, scorch.STensor.from_torch(b), format="ds")
