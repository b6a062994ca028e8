"""The bulk-copy SpMM kernel for wide dense operands (operand rows staged through shared memory by
cp.async.bulk + mbarrier) against the float64 oracle, beside the gather kernel on the same
inputs, selected through the environment (a process of its own) and through the library call;
and the L2 gather-rate probe."""
from __future__ import annotations

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys
import numpy as np, torch
sys.path.insert(0, %(root)r)
from oracle import oracle as O
from scorch_b200 import kernels as K, _lib

def csr(m, n, lens, seed):
    rng = np.random.default_rng(seed)
    pos = np.zeros(m + 1, np.int64); np.cumsum(lens, out=pos[1:])
    crd = np.empty(pos[-1], np.int32)
    for i in range(m):
        if lens[i]:
            crd[pos[i]:pos[i + 1]] = np.sort(rng.choice(n, size=lens[i], replace=False))
    val = (rng.standard_normal(pos[-1]) / np.sqrt(np.repeat(np.maximum(lens, 1), lens))).astype(np.float32)
    return pos.astype(np.int32), crd, val

rng = np.random.default_rng(0)
for m, n, k in ((700, 900, 512), (333, 2000, 1000), (64, 300, 4096), (5000, 4000, 768)):
    lens = rng.integers(0, 70, size=m)
    lens[[0, 3, m - 1]] = [0, 32, 0]
    lens[5] = 200                      # several chunks for one row
    if m > 4000:
        lens[:] = 32                   # the shape of the top-k activations: one full chunk per row
    pos, crd, val = csr(m, n, lens, seed=k)
    B = rng.standard_normal((n, k)).astype(np.float32)
    bias = rng.standard_normal(k).astype(np.float32)
    d = lambda a: torch.from_numpy(a).cuda()
    for b_, relu in ((None, False), (bias, True)):
        got = K.spmm_csr(d(pos), d(crd), d(val), d(B), bias=None if b_ is None else d(b_), relu=relu)
        want = O.spmm_csr_acc64(pos, crd, val, B, b_, relu)
        ok, err, bad = O.allclose_report(got.cpu().numpy(), want, 1e-4, 1e-5)
        assert ok, (m, n, k, err, bad)
        again = K.spmm_csr(d(pos), d(crd), d(val), d(B), bias=None if b_ is None else d(b_), relu=relu)
        assert torch.equal(got, again)
torch.cuda.synchronize()
assert _lib.lib().sb_spmm_wide_status() == 0
print("WIDE_OK")
"""


@pytest.mark.parametrize("mode", ["tma", "gather"])
def test_wide_spmm_kernel_choice_matches_oracle(mode):
    env = dict(os.environ, SCORCH_B200_SPMM_WIDE=mode)
    r = subprocess.run([sys.executable, "-c", SCRIPT % {"root": ROOT}], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0 and "WIDE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_l2_gather_probe_runs_and_reports_a_rate():
    import torch
    from scorch_b200 import _lib
    L = _lib.lib()
    rows, warps, gathers = 32768, 148 * 64, 256
    panel = torch.randn((rows, 256), device="cuda", dtype=torch.float32)
    out = torch.zeros(warps, device="cuda", dtype=torch.float32)
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        _lib.check(L.sb_probe_l2_gather(panel.data_ptr(), rows, gathers, warps, out.data_ptr(), st))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    _lib.check(L.sb_probe_l2_gather(panel.data_ptr(), rows, gathers, warps, out.data_ptr(), st))
    b.record()
    b.synchronize()
    gbps = warps * gathers * 1024 / (a.elapsed_time(b) * 1e-3) / 1e9
    assert 1000 < gbps < 200_000, gbps
    assert L.sb_probe_l2_gather(None, rows, gathers, warps, out.data_ptr(), st) == 1


def test_wide_kernel_selected_by_call_agrees_with_gather_kernel():
    import numpy as np
    import torch
    from scorch_b200 import kernels as K, _lib, workloads as W
    L = _lib.lib()
    A = W.sae_activations(512, 8192, 32, seed=3, device="cuda")
    Wd = W.sae_decoder(8192, 2048, seed=4, device="cuda")
    before = L.sb_spmm_wide_select(1)
    try:
        tma = K.spmm_csr(A.pos, A.crd, A.val, Wd)
        assert L.sb_spmm_wide_select(0) == 1
        gather = K.spmm_csr(A.pos, A.crd, A.val, Wd)
    finally:
        L.sb_spmm_wide_select(before)
    torch.cuda.synchronize()
    assert L.sb_spmm_wide_status() == 0
    # one sequential fp32 sum per output element in both kernels, in different orders
    torch.testing.assert_close(tma, gather, rtol=1e-5, atol=1e-6)
