"""Device-side CSR validation: the first violation of what the kernels assume about their inputs
is named (smallest row, then entry), reading nothing outside pos[0..m] and crd[0..nnz); with
SCORCH_B200_VALIDATE=1 the front end refuses an invalid operand before any kernel reads it."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a, dt=np.int32):
    return torch.from_numpy(np.asarray(a, dt)).cuda()


POS = [0, 2, 2, 5, 6]
CRD = [1, 4, 0, 2, 3, 4]


def test_valid_matrices_pass():
    from scorch_b200 import kernels as K, workloads as W
    assert K.csr_validate(dev(POS), dev(CRD), 5) is None
    assert K.csr_validate(dev([0]), dev([]), 3) is None                       # no rows
    assert K.csr_validate(dev([0, 0, 0]), dev([]), 3) is None                 # no entries
    A = W.powerlaw_square(20000, mean_nnz=8.0, seed=2)
    assert K.csr_validate(A.pos.cuda(), A.crd.cuda(), 20000) is None


@pytest.mark.parametrize("pos,crd,n,sorted_unique,want", [
    ([1, 2, 2, 5, 6], CRD, 5, True, ("pos[0] is not 0", 0, 0, 1)),
    ([0, 2, 2, 5, 5], CRD, 5, True, ("pos[m] is not nnz", 4, 0, 5)),
    ([0, 2, 9, 5, 6], CRD, 5, True, ("row pointer out of [0, nnz]", 2, 0, 9)),
    ([0, 2, 1, 5, 6], CRD, 5, True, ("row pointers decrease", 1, 0, 1)),
    ([0, 3, 2, 5, 6], CRD, 5, True, ("row pointers decrease", 1, 0, 2)),
    (POS, [1, 4, 0, 2, 5, 4], 5, True, ("column index out of range", 2, 4, 5)),
    (POS, [1, -4, 0, 2, 3, 4], 5, True, ("column index out of range", 0, 1, -4)),
    (POS, [1, 4, 0, 3, 3, 4], 5, True, ("columns of a row not strictly ascending", 2, 4, 3)),
    (POS, [4, 1, 0, 2, 3, 9], 5, True, ("columns of a row not strictly ascending", 0, 1, 1)),   # the first of two
])
def test_first_violation_is_named(pos, crd, n, sorted_unique, want):
    from scorch_b200 import kernels as K
    assert K.csr_validate(dev(pos), dev(crd), n, sorted_unique) == want


def test_unsorted_rows_are_accepted_when_order_is_not_required():
    from scorch_b200 import kernels as K
    assert K.csr_validate(dev(POS), dev([4, 1, 0, 3, 3, 2]), 5, sorted_unique=False) is None
    assert K.csr_validate(dev(POS), dev([4, 1, 0, 3, 3, 7]), 5, sorted_unique=False) == (
        "column index out of range", 3, 5, 7)


def test_front_end_refuses_invalid_operands_when_asked(monkeypatch):
    from scorch_b200 import kernels as K
    B = torch.ones((5, 8), device="cuda")
    val = torch.ones(6, device="cuda")
    good = K.spmm_csr(dev(POS), dev(CRD), val, B)
    monkeypatch.setenv("SCORCH_B200_VALIDATE", "1")
    assert torch.equal(K.spmm_csr(dev(POS), dev(CRD), val, B), good)
    with pytest.raises(ValueError, match="column index out of range"):
        K.spmm_csr(dev(POS), dev([1, 4, 0, 2, 3, 5]), val, B)            # never reaches the kernel
    with pytest.raises(ValueError, match="row pointers decrease"):
        K.spmv_csr(dev([0, 3, 2, 5, 6]), dev(CRD), val, torch.ones(5, device="cuda"))
    with pytest.raises(ValueError, match="not strictly ascending"):
        K.spgemm_csr(dev(POS), dev([4, 1, 0, 2, 3, 4]), val, dev([0, 1, 2, 3, 4, 5]), dev([0, 1, 2, 3, 4]),
                     torch.ones(5, device="cuda"), 5)
