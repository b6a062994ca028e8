"""Host-side mirror of the reference interface: container layout, dispatch registry, exported
symbol names.  Follows the reference's tests/test_scorch/test_prebuilt_kernel_registry.py and
test_matmul_dispatch.py in what it asserts."""
from __future__ import annotations

import inspect
import warnings

import pytest
import torch

import scorch_b200 as scorch
from scorch_b200 import ops, scorch_ops
from scorch_b200.stensor import STensor, parse_format

warnings.filterwarnings("ignore", message=".*Sparse CSR tensor support.*")


def _csr(m=6, n=5, dtype=torch.float32):
    d = torch.arange(m * n, dtype=torch.float32).reshape(m, n)
    d[d % 3 != 0] = 0
    return d.to(dtype).to_sparse_csr()


def test_stensor_layout_matches_reference():
    a = STensor.from_torch(_csr())
    assert str(a.format) == "d,s" and a.dim() == 2
    assert a.index.mode_indices[0] == [] and len(a.index.mode_indices[1]) == 2
    assert all(t.dtype == torch.int32 for t in a.index.mode_indices[1])  # storage.py:46-51
    d = STensor.from_torch(torch.ones(3, 4))
    assert str(d.format) == "d,d" and d.values.shape == (12,) and d.index.mode_indices == [[], []]
    c = STensor.from_torch(_csr().to_sparse_coo())
    assert str(c.format) == "o,o" and len(c.index.mode_indices[0]) == 1
    v = STensor.from_torch(torch.ones(4))
    assert str(v.format) == "d"
    assert torch.equal(a.to_torch().to_dense(), _csr().to_dense())


def test_parse_format_forms():
    assert str(parse_format("ds")) == "d,s" == str(parse_format("d,s")) == str(parse_format(["d", "s"]))
    assert parse_format("dd").is_dense() and not parse_format("ds").is_dense()


@pytest.mark.parametrize("dtype,name", [(torch.float32, "spmm_csr_float_v2"),
                                        (torch.float64, "prebuilt_spmm_csr_f64"),
                                        (torch.int32, "prebuilt_spmm_csr_i32"),
                                        (torch.int64, "prebuilt_spmm_csr_i64")])
def test_registry_spmm_symbols(dtype, name):
    a = STensor.from_torch(_csr(dtype=dtype))
    b = STensor.from_torch(torch.ones(5, 3, dtype=dtype))
    r = ops.resolve_prebuilt_matmul(a, b, output_format="dd")
    assert r is not None and r.symbol_name == name and str(r.output_format) == "d,d"


def test_registry_spgemm_spmv_and_misses():
    a = STensor.from_torch(_csr())
    b = STensor.from_torch(_csr(5, 6))
    r = ops.resolve_prebuilt_matmul(a, b)
    assert r.symbol_name == "prebuilt_spmspm_csr_f32" and str(r.output_format) == "d,s"
    # a different requested output format skips the prebuilt kernel
    # (reference tests/test_scorch/test_prebuilt_kernel_registry.py:41-51)
    assert ops.resolve_prebuilt_matmul(a, b, output_format="dd") is None
    x = STensor.from_torch(torch.ones(5))
    assert ops.resolve_prebuilt_matmul(a, x).symbol_name == "prebuilt_spmv_csr_f32"
    # dtype mismatch -> no prebuilt (prebuilt_kernels.py:109-110)
    assert ops.resolve_prebuilt_matmul(a, STensor.from_torch(torch.ones(5, 2, dtype=torch.float64))) is None
    assert ops.resolve_prebuilt_fused("d,s", "d,d", ("add", "relu"), torch.float32) is scorch_ops.spmm_csr_bias_relu_float
    assert ops.resolve_prebuilt_fused("d,s", "d,d", ("add",), torch.float32) is scorch_ops.spmm_csr_bias_float
    assert ops.resolve_prebuilt_fused("d,s", "d,d", ("mul",), torch.float32) is None


def test_scorch_ops_exports_every_reference_symbol_with_reference_keywords():
    assert len(scorch_ops.REFERENCE_SYMBOLS) == 38
    for n in scorch_ops.REFERENCE_SYMBOLS:
        assert hasattr(scorch_ops, n), n
    base = ["result_shape", "A_shape", "A_mode_indices", "A_values", "B_shape", "B_mode_indices", "B_values"]
    sig = lambda f: list(inspect.signature(f).parameters)
    assert sig(scorch_ops.spmm_csr_float_v2) == base + ["tile_size"]
    assert inspect.signature(scorch_ops.spmm_csr_float_v2).parameters["tile_size"].default == 256
    assert inspect.signature(scorch_ops.prebuilt_spmm_csr_f32).parameters["tile_size"].default == 32
    assert sig(scorch_ops.prebuilt_spmv_csr_f32) == base == sig(scorch_ops.prebuilt_spmspm_csr_i64)
    assert sig(scorch_ops.spmm_csr_bias_relu_float) == base + ["bias"]
    assert sig(scorch_ops.spmm_csr_float_tiled_i_k) == base + ["i_tile_size", "k_tile_size"]
    assert sig(scorch_ops.sddmm_coo_float_prebuilt) == [
        "result_shape", "S_shape", "S_mode_indices", "S_values", "A_shape", "A_mode_indices",
        "A_values", "B_shape", "B_mode_indices", "B_values"]


def test_dense_dense_goes_to_torch_and_unknown_patterns_raise():
    a, b = torch.ones(3, 4), torch.ones(4, 2)
    assert torch.equal(scorch.matmul(a, b), a @ b)
    with pytest.raises(NotImplementedError):
        scorch.einsum("ijk,jk->i", torch.ones(2, 2, 2), torch.ones(2, 2))
    assert scorch.float32 is torch.float32  # falls through to torch like the reference package


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_sparse_matmul_without_gpu_fails_loudly():
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        scorch.matmul(_csr(), torch.ones(5, 2))
    from scorch_b200 import kernels
    with pytest.raises(TypeError, match="CUDA tensor"):
        kernels.spmv_csr(torch.zeros(2, dtype=torch.int32), torch.zeros(0, dtype=torch.int32),
                         torch.zeros(0), torch.zeros(1))


def test_all_ones_mask_check_is_cached_until_the_tensor_is_written():
    """The one-call attention path drops mask values that are all exactly 1.0; the check is
    remembered on the tensor object and redone after an in-place write."""
    from scorch_b200 import kernels as K
    v = torch.ones(100)
    assert K._mask_is_all_ones(v) is True
    assert v._sb_all_ones[1] is True
    v[3] = 0.5                      # in-place write bumps the version: the cache entry is stale
    assert K._mask_is_all_ones(v) is False
    v[3] = 1.0
    assert K._mask_is_all_ones(v) is True
    assert K._mask_is_all_ones(torch.full((4,), 1.0 + 1e-6)) is False


def test_host_attention_chunk_bounds():
    """Chunks of the host-tensor attention front end: cover every unit once, in order, shrinking
    towards the end; degenerate sizes give empty chunks, never a gap."""
    from scorch_b200.pipelines import chunk_bounds
    assert chunk_bounds(32, 4) == [0, 14, 24, 30, 32]
    assert chunk_bounds(32, 4, shrink=False) == [0, 8, 16, 24, 32]
    for units in (1, 2, 3, 5, 8, 31, 32, 100):
        for chunks in (1, 2, 3, 4, 8):
            for shrink in (True, False):
                b = chunk_bounds(units, chunks, shrink)
                assert len(b) == chunks + 1 and b[0] == 0 and b[-1] == units
                assert all(x <= y for x, y in zip(b, b[1:]))
                sizes = [y - x for x, y in zip(b, b[1:])]
                if shrink and units >= 4 * chunks:
                    assert all(x >= y for x, y in zip(sizes, sizes[1:]))
