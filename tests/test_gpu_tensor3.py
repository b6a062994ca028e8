"""TTM and MTTKRP of a compressed-fibre 3-D tensor through ``einsum`` (their per-entry work runs in
the SpMM kernel) against the reference's own results (golden) and the float64 oracle."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "hotpath_golden.npz"))
RTOL, ATOL = 1e-4, 1e-5


def golden_tensor(fmt, device):
    from scorch_b200.stensor import STensor, TensorIndex, TensorStorage
    p = f"tensor3_{fmt}."
    t = lambda k: torch.from_numpy(GOLD[p + k]).to(device)
    lv0 = [t("pos0"), t("crd0")] if p + "pos0" in GOLD.files else []
    idx = TensorIndex([lv0, [t("pos1"), t("crd1")], [t("pos2"), t("crd2")]], str(GOLD[p + "format"][0]))
    return STensor(tuple(int(x) for x in GOLD[p + "shape"]), TensorStorage(idx, t("val"))), p


@pytest.mark.parametrize("device", ["cuda", "cpu"])
@pytest.mark.parametrize("fmt", ["dss", "sss"])
def test_ttm_and_mttkrp_match_the_reference(fmt, device):
    import scorch_b200 as scorch
    a, p = golden_tensor(fmt, device)
    Bkm, Bjm = (torch.from_numpy(GOLD[p + k]).to(device) for k in ("B_km", "B_jm"))
    c = scorch.einsum("ijk,km->ijm", a, Bkm, format="ddd")
    assert str(c.format) == "d,d,d" and c.values.device.type == device
    np.testing.assert_allclose(c.to_torch().cpu().numpy(), GOLD[p + "ttm"], rtol=RTOL, atol=ATOL)
    d = scorch.einsum("ijk,jm,km->im", a, Bjm, Bkm, format="dd")
    np.testing.assert_allclose(d.to_torch().cpu().numpy(), GOLD[p + "mttkrp"], rtol=RTOL, atol=ATOL)
    with pytest.raises(NotImplementedError):
        scorch.einsum("ijk,km->ijm", a, Bkm, format="dds")


@pytest.mark.parametrize("fmt", ["dss", "sss"])
@pytest.mark.parametrize("shape,m,density", [((40, 30, 50), 64, 0.05), ((5, 300, 2000), 256, 0.02), ((64, 1, 7), 3, 0.5)])
def test_random_tensors_vs_oracle(oracle, fmt, shape, m, density):
    import scorch_b200 as scorch
    from scorch_b200 import tensor3
    rng = np.random.default_rng(shape[0] + m)
    dense = (rng.standard_normal(shape) * (rng.random(shape) < density)).astype(np.float32)
    dense[shape[0] // 2] = 0
    st = tensor3.csf3_from_dense(torch.from_numpy(dense).cuda(), fmt)
    lv = [[x.cpu().numpy() for x in level] for level in st.index.mode_indices]
    val = st.values.cpu().numpy()
    B = rng.standard_normal((shape[2], m)).astype(np.float32)
    Bj = rng.standard_normal((shape[1], m)).astype(np.float32)
    got = scorch.einsum("ijk,km->ijm", st, torch.from_numpy(B).cuda()).to_torch().cpu().numpy()
    ok, err, bad = oracle.allclose_report(got, oracle.ttm_acc64(shape, lv, val, B), RTOL, ATOL)
    assert ok, (err, bad)
    got = scorch.einsum("ijk,jm,km->im", st, torch.from_numpy(Bj).cuda(), torch.from_numpy(B).cuda())
    ok, err, bad = oracle.allclose_report(got.to_torch().cpu().numpy(), oracle.mttkrp_acc64(shape, lv, val, Bj, B),
                                          RTOL, 4 * ATOL)
    assert ok, (err, bad)
    # a dense tensor takes the library route and gives the same numbers
    dn = scorch.einsum("ijk,km->ijm", torch.from_numpy(dense).cuda(), torch.from_numpy(B).cuda())
    np.testing.assert_allclose(dn.to_torch().cpu().numpy(), oracle.ttm_acc64(shape, lv, val, B), rtol=1e-3, atol=1e-3)
