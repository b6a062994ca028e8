"""The allocation-free SpMV entry point (sb_spmv_csr_f32_static) against the regular one.

Who needs it: code that runs on a GPU whose memory it does not own — a plugin inside another
runtime's arena, a service that may not touch the allocator once it is up — cannot hand the
library a scratch buffer for the partial sums of rows cut by tile borders, and cannot let it call
cudaMalloc either.  The static entry keeps that scratch in an array inside the library image,
shared by all calls: the tests run different matrices back to back to show that nothing a call
leaves in the array reaches the next one.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _matrix(m, n, lens, seed):
    rng = np.random.default_rng(seed)
    lens = np.minimum(np.asarray(lens, np.int64), n)
    pos = np.zeros(m + 1, np.int64)
    np.cumsum(lens, out=pos[1:])
    crd = np.empty(pos[-1], np.int32)
    for i in range(m):
        if lens[i]:
            crd[pos[i]:pos[i + 1]] = np.sort(rng.choice(n, size=lens[i], replace=False))
    val = (rng.standard_normal(pos[-1]) / np.sqrt(np.repeat(np.maximum(lens, 1), lens))).astype(np.float32)
    x = rng.standard_normal(n).astype(np.float32)
    return [torch.from_numpy(a).cuda() for a in (pos.astype(np.int32), crd, val, x)]


def _static_spmv(pos, crd, val, x):
    from scorch_b200 import _lib
    L = _lib.lib()
    y = torch.full((pos.numel() - 1,), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(L.sb_spmv_csr_f32_static(pos.numel() - 1, x.numel(), crd.numel(), pos.data_ptr(),
                                        crd.data_ptr(), val.data_ptr(), x.data_ptr(), y.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream))
    return y


def test_static_spmv_matches_regular_entry_on_two_calls_in_a_row():
    from scorch_b200 import kernels as K
    from scorch_b200._lib import HEAVY_ROW_NNZ as T
    # first call: many rows cut by tile borders, so the shared array is left full of partial sums
    lens1 = np.random.default_rng(0).poisson(10, size=4000)
    lens1[[3, 900, 901, 3999]] = [6 * T + 5, T + 1, 2 * T, 3 * T - 7]
    a1 = _matrix(4000, 20000, lens1, seed=1)
    # second call: a different, smaller structure with other heavy rows and an empty tail row
    lens2 = np.random.default_rng(2).poisson(3, size=1500)
    lens2[[0, 700]] = [2 * T + 9, T + 2]
    lens2[-1] = 0
    a2 = _matrix(1500, 9000, lens2, seed=3)

    # third matrix: thousands of empty rows (more than a tile's worth of entries would span)
    # between two rows that tile borders cut, and empty rows at both ends
    lens3 = np.zeros(9000, np.int64)
    lens3[[5, 6, 8000, 8001]] = [3000, 2500, 4100, 7]
    a3 = _matrix(9000, 30000, lens3, seed=5)

    want1, want2, want3 = K.spmv_csr(*a1), K.spmv_csr(*a2), K.spmv_csr(*a3)
    got1 = _static_spmv(*a1)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    got2 = _static_spmv(*a2)
    got3 = _static_spmv(*a3)
    got1_again = _static_spmv(*a1)
    torch.cuda.synchronize()
    # nothing was allocated by the calls themselves (y comes from torch's cached pool)
    assert torch.cuda.mem_get_info()[0] == free_before
    # same kernels, same fixed-order sums: the results agree to the last bit, and well inside
    # the suite's tolerance
    for got, want in ((got1, want1), (got2, want2), (got3, want3), (got1_again, want1)):
        assert torch.isfinite(got).all()
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
        assert torch.equal(got, want)


def test_static_spmv_rejects_sizes_beyond_the_builtin_scratch():
    from scorch_b200 import _lib
    L = _lib.lib()
    one = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = L.sb_spmv_csr_f32_static(2, 2, _lib.STATIC_SPMV_MAX_NNZ + 1, one.data_ptr(), one.data_ptr(),
                                  one.data_ptr(), one.data_ptr(), one.data_ptr(), None)
    assert rc == 5 and b"exceeds" in L.sb_last_error()
    # argument errors are reported as such, whatever the size
    rc = L.sb_spmv_csr_f32_static(2, 2, _lib.STATIC_SPMV_MAX_NNZ + 1, None, one.data_ptr(),
                                  one.data_ptr(), one.data_ptr(), one.data_ptr(), None)
    assert rc == 1 and b"pos is null" in L.sb_last_error()
