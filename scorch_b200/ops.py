"""``matmul`` / ``einsum`` front end for the patterns the sparse hot path covers, with the
reference's dispatch rules, keyword arguments and return conventions.

Reference: src/scorch/ops.py:248-423 (matmul, einsum SDDMM dispatch) and the registry in
src/scorch/prebuilt_kernels.py:37-224.  Where the reference would fall through to its
einsum->CIN->LLIR compiler (any pattern without a prebuilt kernel) this module raises
``NotImplementedError``: the compiler is not part of this package — only its output for SpMM,
SDDMM, SpMV and SpGEMM is, as CUDA kernels.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Callable, List, Mapping, Optional, Sequence, Tuple, Union

import torch

from . import scorch_ops as native_ops
from .stensor import STensor, TensorFormat, TensorIndex, parse_format


@dataclass(frozen=True)
class PrebuiltMatmulSpec:
    lhs_rank: int
    rhs_rank: int
    lhs_format: str
    rhs_format: str
    output_format: str
    symbol_by_dtype: Mapping[torch.dtype, Sequence[str]]


@dataclass(frozen=True)
class ResolvedPrebuiltKernel:
    fn: Callable[..., Any]
    output_format: TensorFormat
    symbol_name: str


# Same table as the reference (src/scorch/prebuilt_kernels.py:37-93).
_MATMUL_PREBUILT_SPECS: List[PrebuiltMatmulSpec] = [
    PrebuiltMatmulSpec(2, 2, "d,s", "d,d", "dd", {
        torch.float32: ("spmm_csr_float_v2", "prebuilt_spmm_csr_f32", "spmm_csr_float"),
        torch.float64: ("prebuilt_spmm_csr_f64", "spmm_csr_double"),
        torch.int32: ("prebuilt_spmm_csr_i32",),
        torch.int64: ("prebuilt_spmm_csr_i64",)}),
    PrebuiltMatmulSpec(2, 2, "d,s", "d,s", "ds", {
        torch.float32: ("prebuilt_spmspm_csr_f32", "spmspm_csr_float"),
        torch.float64: ("prebuilt_spmspm_csr_f64",),
        torch.int32: ("prebuilt_spmspm_csr_i32",),
        torch.int64: ("prebuilt_spmspm_csr_i64",)}),
    PrebuiltMatmulSpec(2, 2, "o,o", "o,o", "oo", {torch.float32: ("spmspm_coo_float",)}),
    PrebuiltMatmulSpec(2, 2, "o,o", "d,d", "dd", {torch.float32: ("spmm_coo_float",)}),
    PrebuiltMatmulSpec(2, 1, "d,s", "d", "d", {
        torch.float32: ("prebuilt_spmv_csr_f32",),
        torch.float64: ("prebuilt_spmv_csr_f64",),
        torch.int32: ("prebuilt_spmv_csr_i32",),
        torch.int64: ("prebuilt_spmv_csr_i64",)}),
]

_FUSED_PREBUILT_SPECS = {
    ("d,s", "d,d", ("add", "relu"), torch.float32): "spmm_csr_bias_relu_float",
    ("d,s", "d,d", ("add",), torch.float32): "spmm_csr_bias_float",
}


def resolve_prebuilt_matmul(a: STensor, b: STensor, output_format=None
                            ) -> Optional[ResolvedPrebuiltKernel]:
    """Reference: resolve_prebuilt_matmul, src/scorch/prebuilt_kernels.py:104-137."""
    if a.values.dtype != b.values.dtype:
        return None
    requested = str(parse_format(output_format)) if output_format is not None else None
    for spec in _MATMUL_PREBUILT_SPECS:
        if a.dim() != spec.lhs_rank or b.dim() != spec.rhs_rank:
            continue
        if str(a.format) != spec.lhs_format or str(b.format) != spec.rhs_format:
            continue
        if requested is not None and requested != str(parse_format(spec.output_format)):
            continue
        for name in spec.symbol_by_dtype.get(a.values.dtype, ()):
            fn = getattr(native_ops, name, None)
            if fn is not None:
                return ResolvedPrebuiltKernel(fn, parse_format(spec.output_format), name)
    return None


def resolve_prebuilt_fused(a_format: str, b_format: str, post_op_kinds: Tuple[str, ...],
                           dtype: torch.dtype):
    """Reference: resolve_prebuilt_fused, src/scorch/prebuilt_kernels.py:176-195."""
    name = _FUSED_PREBUILT_SPECS.get((a_format, b_format, tuple(post_op_kinds), dtype))
    return getattr(native_ops, name, None) if name else None


def execute_prebuilt_binary_kernel(kernel_fn, a: STensor, b: STensor, time_dict=None):
    """Reference: execute_prebuilt_binary_kernel, src/scorch/prebuilt_kernels.py:198-224."""
    if b.dim() == 2:
        result_shape: Tuple[int, ...] = (a.shape[0], b.shape[1])
    elif b.dim() == 1:
        result_shape = (a.shape[0],)
    else:
        raise ValueError(f"Unsupported RHS rank for prebuilt matmul kernel: {b.dim()}")
    args: list = [result_shape]
    for t in (a, b):
        args += [t.shape, t.index.mode_indices, t.values]
    start = time.time()
    result = kernel_fn(*args)
    if time_dict is not None:
        if result.storage.value.is_cuda:
            torch.cuda.current_stream().synchronize()
        time_dict["eval_time"] = time.time() - start
    return result, result_shape


def _wrap(result_cpp, shape, fmt) -> STensor:
    return STensor(shape=shape, index=TensorIndex(result_cpp.storage.index.mode_indices, fmt),
                   value=result_cpp.storage.value)


def matmul(a: Union[torch.Tensor, STensor], b: Union[torch.Tensor, STensor], **kwargs: Any
           ) -> Union[torch.Tensor, STensor]:
    """Matrix product with the reference's dispatch (src/scorch/ops.py:248-372)."""
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor):
        a_sp = a.layout != torch.strided
        b_sp = b.layout != torch.strided
        if a.layout == torch.sparse_coo and b.layout == torch.sparse_coo:
            a, b = a.to_sparse_csr(), b.to_sparse_csr()
        if not (a_sp or b_sp):
            return torch.matmul(a, b)
    if isinstance(a, torch.Tensor):
        a = STensor.from_torch(a)
    if isinstance(b, torch.Tensor):
        b = STensor.from_torch(b)

    time_dict = kwargs.get("time_dict")
    requested = kwargs.get("format", kwargs.get("output_format"))

    if a.format.is_dense() and b.format.is_dense():
        start = time.time()
        out = torch.matmul(a.to_torch(), b.to_torch())
        if time_dict is not None:
            time_dict["eval_time"] = time.time() - start
        if requested is None or parse_format(requested).is_dense():
            return out
        raise NotImplementedError("sparse output of a dense x dense product needs the reference's "
                                  "compiler, which this package does not contain")

    # sparse 2-D operands stored in the other mode order are re-laid-out to the canonical one
    # before dispatch, on the device (reference: src/scorch/ops.py:299-303,333-346)
    if a.dim() == 2 and not a.format.is_dense() and a.index.mode_order != [0, 1]:
        a = a.copy().change_mode_order([0, 1])
    if b.dim() == 2 and a.dim() == 2 and b.index.mode_order != [0, 1] and not (
            a.format.is_dense() and b.format.is_dense()):
        b = b.copy().change_mode_order([0, 1])

    resolved = resolve_prebuilt_matmul(a, b, output_format=requested)
    if resolved is None:
        raise NotImplementedError(
            f"no B200 kernel for matmul({a.format} rank {a.dim()}, {b.format} rank {b.dim()}, "
            f"dtypes {a.dtype}/{b.dtype}, output {requested}); the reference would JIT-compile it")
    result_cpp, shape = execute_prebuilt_binary_kernel(resolved.fn, a, b, time_dict=time_dict)
    result = _wrap(result_cpp, shape, resolved.output_format)
    return result.to_torch() if result.format.is_dense() else result


_SDDMM_EXPRS = ("ij,ik,jk->ij", "ij,ik,kj->ij")


def einsum(expression: str, *tensors: Union[torch.Tensor, STensor], **kwargs: Any):
    """Einsum for the expressions the hot path covers (reference: src/scorch/ops.py:375-819).

    * ``"ij,ik,jk->ij"`` / ``"ij,ik,kj->ij"`` with a COO or CSR mask and dense Q, K -> SDDMM.
      A COO mask gives a result sharing the mask's coordinates (prebuilt route, ops.py:396-423);
      a CSR mask gives an all-COO result with fresh int32 coordinates in mask order, which is
      what the reference's compiler emits (ops.py:638-664).
    * ``"ij,jk->ik"`` -> ``matmul``;  ``"ij,j->i"`` -> SpMV;  ``"ij,ij->ij"`` -> element-wise product.
    * ``"ijk,km->ijm"`` (TTM) and ``"ijk,jm,km->im"`` (MTTKRP) with a ``d,s,s`` / ``s,s,s`` (or dense)
      3-D tensor and dense matrices -> dense result (``tensor3``).
    """
    ts = tuple(STensor.from_torch(t) if isinstance(t, torch.Tensor) else t for t in tensors)
    expr = expression.replace(" ", "")
    if expr in _SDDMM_EXPRS and len(ts) == 3:
        S, A, B = ts
        if not (str(A.format) == "d,d" and str(B.format) == "d,d" and S.dtype == torch.float32):
            raise NotImplementedError("SDDMM needs a float32 sparse mask and dense Q, K")
        if expr == "ij,ik,kj->ij":
            # the reference transposes the third operand physically before the kernel
            # (ops.py:534-540), so the kernel always sees K as (j, k) row-major
            Bt = B.to_torch().t().contiguous()
            B = STensor.from_torch(Bt)
        args = (S.shape, S.shape, S.index.mode_indices, S.values, A.shape, A.index.mode_indices,
                A.values, B.shape, B.index.mode_indices, B.values)
        if str(S.format) == "o,o":
            r = native_ops.sddmm_coo_float_prebuilt(*args)
            return _wrap(r, S.shape, S.format)
        if str(S.format) == "d,s":
            r = native_ops.sddmm_csr_float(*args)
            return _wrap(r, S.shape, "o,o")
        raise NotImplementedError(f"SDDMM mask format {S.format}")
    if expr == "ij,ij->ij" and len(ts) == 2:
        return elementwise("mul", ts[0], ts[1], **kwargs)
    if expr == "ij,jk->ik" and len(ts) == 2:
        return matmul(ts[0], ts[1], **kwargs)
    if expr == "ij,j->i" and len(ts) == 2:
        return matmul(ts[0], ts[1], **kwargs)
    if expr in ("ijk,km->ijm", "ijk,jm,km->im"):
        # TTM / MTTKRP of a compressed-fibre tensor: CSR x dense products over its fibre matrix
        from . import tensor3
        requested = kwargs.get("format", kwargs.get("output_format"))
        if requested is not None and not parse_format(requested).is_dense():
            raise NotImplementedError("3-D contractions produce dense results")
        r = tensor3.contract(expr, ts[0], *ts[1:])
        if r is not None:
            return STensor.from_torch(r[0])
    raise NotImplementedError(
        f"einsum expression {expression!r} is outside the sparse hot path (SpMM, SDDMM, SpMV, "
        "SpGEMM); the reference would JIT-compile it")


def elementwise(op: str, a: Union[torch.Tensor, STensor], b: Union[torch.Tensor, STensor], **kwargs: Any
                ) -> STensor:
    """``"mul"``: C[i,j] = A[i,j] * B[i,j];  ``"add"``: C = A + B, for two sparse matrices of the same
    shape in the same format, compressed (``d,s``) or coordinate (``o,o``); the result has that
    format, its structure the intersection / union of the operands' (the reference compiles a merge
    loop for these, src/scorch/ops.py:375-819; tests/test_scorch/test_kernels_comprehensive.py:119-200).
    Host operands are moved to the GPU for the kernel and the result comes back to the host."""
    from . import kernels as K
    a = STensor.from_torch(a) if isinstance(a, torch.Tensor) else a
    b = STensor.from_torch(b) if isinstance(b, torch.Tensor) else b
    fa, fb = str(a.format), str(b.format)
    requested = kwargs.get("format", kwargs.get("output_format"))
    if a.shape != b.shape or a.dim() != 2:
        raise ValueError("element-wise operands must be matrices of the same shape")
    if fa != fb or fa not in ("d,s", "o,o") or a.dtype != b.dtype or (
            requested is not None and str(parse_format(requested)) != fa):
        raise NotImplementedError(
            f"no B200 kernel for element-wise {op} of {fa} and {fb} operands ({a.dtype}/{b.dtype}, output "
            f"{requested}); the reference would JIT-compile it")
    for t in (a, b):
        if t.index.mode_order != [0, 1]:
            raise NotImplementedError("element-wise operands must be in the default mode order")
    host = not a.values.is_cuda
    dev = torch.device("cuda", torch.cuda.current_device()) if host else a.values.device
    up = lambda t: t.to(dev)

    def csr_of(t):
        if str(t.format) == "d,s":
            return up(t.index.mode_indices[1][0]), up(t.index.mode_indices[1][1])
        return (K.coo_rows_to_csr_pos(up(t.index.mode_indices[0][0]), t.shape[0]),
                up(t.index.mode_indices[1][0]))
    (apos, acrd), (bpos, bcrd) = csr_of(a), csr_of(b)
    start = time.time()
    cpos, ccrd, cval = K.csr_ewise(op, apos, acrd, up(a.values), bpos, bcrd, up(b.values))
    time_dict = kwargs.get("time_dict")
    if time_dict is not None:
        torch.cuda.current_stream().synchronize()
        time_dict["eval_time"] = time.time() - start
    back = (lambda t: t.cpu()) if host else (lambda t: t)
    if fa == "d,s":
        idx = TensorIndex([[], [back(cpos), back(ccrd)]], "d,s")
    else:
        idx = TensorIndex([[back(K.csr_pos_to_coo_rows(cpos, ccrd.numel()))], [back(ccrd)]], "o,o")
    return STensor(shape=a.shape, index=idx, value=back(cval))


def add(a: Union[torch.Tensor, STensor], b: Union[torch.Tensor, STensor], **kwargs: Any) -> STensor:
    """A + B for two sparse matrices (what ``STensor.__add__`` of the reference computes)."""
    return elementwise("add", a, b, **kwargs)


def spmm_bias_act(a: Union[torch.Tensor, STensor], b: torch.Tensor, bias: torch.Tensor,
                  relu: bool) -> torch.Tensor:
    """Fused ``act(A @ B + bias)`` — the kernel ``@scorch.compile`` reaches for a GCN layer
    (reference: src/scorch/trace.py:232-301 -> csrc/spmm.h:28-89)."""
    if isinstance(a, torch.Tensor):
        a = STensor.from_torch(a)
    bs = STensor.from_torch(b)
    fn = resolve_prebuilt_fused(str(a.format), str(bs.format), ("add", "relu") if relu else ("add",),
                                a.dtype)
    if fn is None:
        raise NotImplementedError("fused SpMM+bias needs a float32 CSR x dense product")
    shape = (a.shape[0], b.shape[1])
    r = fn(shape, a.shape, a.index.mode_indices, a.values, bs.shape, bs.index.mode_indices,
           bs.values, bias)
    return r.storage.value.view(shape)
