"""Contractions of a 3-D sparse tensor with dense matrices on the SpMM kernel.

The reference compiles these from einsum expressions (src/scorch/ops.py:375-819; exercised with
dense operands in tests/test_scorch/test_kernels_comprehensive.py:418-482); for a tensor stored in
its compressed-fibre formats ``d,s,s`` / ``s,s,s`` (level 1 compresses j under i, level 2
compresses k under the (i, j) fibre) both contractions reduce to CSR x dense products over the
*fibre matrix* — one row per stored (i, j) fibre, the fibre's k entries as its columns, which is
exactly what level 2 of the format stores as ``[pos, crd]`` + values:

* TTM     ``"ijk,km->ijm"``      C[i, j, :] = sum_k A[i, j, k] B[k, :]
          = rows of  (fibre matrix) B  scattered to their (i, j) positions;
* MTTKRP  ``"ijk,jm,km->im"``    D[i, :] = sum_{j,k} A[i, j, k] B[j, :] * C[k, :]
          = sum over the fibres of row i of  B[j_f, :] * ((fibre matrix) C)[f, :]
          (the k sum is shared by the whole fibre), a second CSR x dense product with level 1's
          ``pos`` as row pointers.

So the per-entry work runs in ``sb_spmm_csr_*``; index expansion and the row scatter are device
torch ops.  Dense 3-D operands go through the library GEMM (they are not sparse work).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .stensor import STensor, TensorIndex, TensorStorage

CSF3_FORMATS = ("d,s,s", "s,s,s")


def csf3_from_dense(t: torch.Tensor, fmt: str = "dss") -> STensor:
    """Dense (I, J, K) tensor -> ``d,s,s`` or ``s,s,s`` STensor with the reference's arrays
    (STensor.to_sparse, src/scorch/stensor.py:607+): coordinates in lexicographic order, a fibre
    per stored (i, j) pair, for ``s,s,s`` only the i slices that hold entries."""
    fmt = fmt.replace(",", "")
    if t.dim() != 3 or fmt not in ("dss", "sss"):
        raise ValueError("csf3_from_dense takes a 3-D tensor and the format 'dss' or 'sss'")
    I, J, K = t.shape
    dev = t.device
    nz = t.nonzero()                                   # lexicographic (i, j, k)
    vals = t[nz[:, 0], nz[:, 1], nz[:, 2]].contiguous()
    fib = nz[:, 0] * J + nz[:, 1]
    fibres, counts = torch.unique_consecutive(fib, return_counts=True)
    pos2 = torch.zeros(fibres.numel() + 1, dtype=torch.int64, device=dev)
    pos2[1:] = torch.cumsum(counts, 0)
    fi, fj = fibres // J, fibres % J
    crd2 = nz[:, 2]
    if fmt == "dss":
        per_i = torch.bincount(fi, minlength=I)
        pos1 = torch.zeros(I + 1, dtype=torch.int64, device=dev)
        pos1[1:] = torch.cumsum(per_i, 0)
        levels = [[], [pos1, fj], [pos2, crd2]]
    else:
        rows, per_row = torch.unique_consecutive(fi, return_counts=True)
        pos1 = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=dev)
        pos1[1:] = torch.cumsum(per_row, 0)
        pos0 = torch.tensor([0, rows.numel()], dtype=torch.int64, device=dev)
        levels = [[pos0, rows], [pos1, fj], [pos2, crd2]]
    idx = TensorIndex(levels, ",".join(fmt))
    return STensor((I, J, K), TensorStorage(idx, vals))


def csf3_to_dense(a: STensor) -> torch.Tensor:
    """``d,s,s`` / ``s,s,s`` STensor -> dense (I, J, K) tensor (checks and small cases)."""
    I, J, K = a.shape
    slices, pos1, crd1, pos2, crd2 = _levels(a)
    dev = a.values.device
    fib_of_entry = _expand(pos2, crd2.numel())
    row_of_fibre = _expand(pos1, crd1.numel())
    i_of_fibre = row_of_fibre if slices is None else slices.long()[row_of_fibre]
    out = torch.zeros((I, J, K), dtype=a.values.dtype, device=dev)
    out[i_of_fibre[fib_of_entry], crd1.long()[fib_of_entry], crd2.long()] = a.values
    return out


def _expand(pos: torch.Tensor, n: int) -> torch.Tensor:
    """Row index of each of the n entries described by row pointers ``pos`` (int64)."""
    lens = (pos[1:] - pos[:-1]).long()
    return torch.repeat_interleave(torch.arange(lens.numel(), device=pos.device), lens, output_size=n)


def _levels(a: STensor):
    f = str(a.format)
    if f not in CSF3_FORMATS or a.dim() != 3:
        raise NotImplementedError(f"3-D contractions take a d,s,s or s,s,s tensor, not {f!r}")
    if a.index.mode_order != [0, 1, 2]:
        raise NotImplementedError("3-D contractions need the default mode order")
    lv = a.index.mode_indices
    slices = None if f == "d,s,s" else lv[0][1]
    return slices, lv[1][0], lv[1][1], lv[2][0], lv[2][1]


def _on_device(a: STensor, *dense: torch.Tensor):
    host = not a.values.is_cuda
    dev = torch.device("cuda", torch.cuda.current_device()) if host else a.values.device
    return host, a.to(dev), tuple(d.to(dev).contiguous() for d in dense)


def ttm(a: STensor, b: torch.Tensor) -> torch.Tensor:
    """C[i, j, :] = sum_k A[i, j, k] B[k, :] for a compressed-fibre A; dense (I, J, M) result."""
    from . import kernels as K
    I, J, Kdim = a.shape
    if b.dim() != 2 or b.shape[0] != Kdim:
        raise ValueError("TTM needs B of shape (K, M)")
    host, a, (b,) = _on_device(a, b)
    slices, pos1, crd1, pos2, crd2 = _levels(a)
    M = b.shape[1]
    out = torch.zeros((I * J, M), dtype=a.values.dtype, device=b.device)
    fibres = crd1.numel()
    if fibres:
        per_fibre = K.spmm_csr(pos2, crd2, a.values, b)                   # (fibres, M)
        row_of_fibre = _expand(pos1, fibres)
        i_of_fibre = row_of_fibre if slices is None else slices.long()[row_of_fibre]
        out.index_copy_(0, i_of_fibre * J + crd1.long(), per_fibre)
    out = out.view(I, J, M)
    return out.cpu() if host else out


def mttkrp(a: STensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """D[i, :] = sum_{j,k} A[i, j, k] B[j, :] * C[k, :] for a compressed-fibre A; dense (I, M)."""
    from . import kernels as K
    I, J, Kdim = a.shape
    if b.dim() != 2 or c.dim() != 2 or b.shape[0] != J or c.shape[0] != Kdim or b.shape[1] != c.shape[1]:
        raise ValueError("MTTKRP needs B of shape (J, M) and C of shape (K, M)")
    host, a, (b, c) = _on_device(a, b, c)
    slices, pos1, crd1, pos2, crd2 = _levels(a)
    M = b.shape[1]
    fibres = crd1.numel()
    out = torch.zeros((I, M), dtype=a.values.dtype, device=b.device)
    if fibres:
        per_fibre = K.spmm_csr(pos2, crd2, a.values, c)                   # sum_k A[f, k] C[k, :]
        per_fibre.mul_(b[crd1.long()])                                    # times B[j_f, :]
        ones = torch.ones(fibres, dtype=a.values.dtype, device=b.device)
        ident = torch.arange(fibres, dtype=torch.int32, device=b.device)
        rows = K.spmm_csr(pos1, ident, ones, per_fibre)                   # sum over the fibres of a slice
        if slices is None:
            out = rows
        else:
            out.index_copy_(0, slices.long(), rows)
    return out.cpu() if host else out


def contract(expr: str, a: STensor, *dense: STensor) -> Optional[Tuple[torch.Tensor, Tuple[int, ...]]]:
    """``einsum`` hook: the dense result and its shape for the expressions above, None otherwise."""
    if a.dim() != 3 or any(isinstance(d, STensor) and not d.format.is_dense() for d in dense):
        return None
    mats = [d.to_torch() if isinstance(d, STensor) else d for d in dense]
    if a.format.is_dense():
        # dense operands: library GEMMs on the GPU (not sparse work, but the same call shape)
        host, a_dev, mats_dev = _on_device(a, *mats)
        t = a_dev.to_torch()
        if expr == "ijk,km->ijm" and len(mats) == 1:
            out = torch.matmul(t.reshape(-1, t.shape[2]), mats_dev[0]).view(t.shape[0], t.shape[1], -1)
        elif expr == "ijk,jm,km->im" and len(mats) == 2:
            out = torch.einsum("ijk,jm,km->im", t, mats_dev[0], mats_dev[1])
        else:
            return None
        out = out.cpu() if host else out
        return out, tuple(out.shape)
    if expr == "ijk,km->ijm" and len(mats) == 1:
        out = ttm(a, mats[0])
    elif expr == "ijk,jm,km->im" and len(mats) == 2:
        out = mttkrp(a, mats[0], mats[1])
    else:
        return None
    return out, tuple(out.shape)
