"""The two application-level callers of the kernels that the benchmark configurations name, kept
on the device end to end.

* ``sparse_attention`` — per (batch, head): S = SDDMM(mask, Q, K), row softmax over the stored
  entries, O = SpMM(S, V).  Reference caller: bench/bench_sparse_transformer.py:304-382, which
  loops over heads in Python and does the softmax with torch scatter ops; here all heads go
  through one batched launch per stage.
* ``gcn_forward`` — H = ReLU(A_hat (X W1)), out = A_hat (H W2), transform first like the
  reference's bench (bench/bench_gcn.py:314-329).  The dense X·W products are cuBLAS calls
  through torch (outside the sparse path); the two A_hat products are the SpMM kernel, the first
  with the fused ReLU epilogue.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K


def sparse_attention(pos: torch.Tensor, crd: torch.Tensor, mask_val: Optional[torch.Tensor],
                     Q: torch.Tensor, Kmat: torch.Tensor, V: torch.Tensor, scale: float = 1.0,
                     plan: Optional[K.CsrPlan] = None, scores_out: Optional[list] = None
                     ) -> torch.Tensor:
    """Q, K, V: (units, seq, d) with units = batch*heads.  Returns O (units, seq, d)."""
    s = K.sddmm_csr(pos, crd, mask_val, Q, Kmat)          # (units, nnz)
    K.csr_row_softmax(pos, s, scale=scale, out=s)         # in place
    if scores_out is not None:
        scores_out.append(s)
    return K.spmm_csr(pos, crd, s, V, plan=plan)


def gcn_forward(pos, crd, val, X, W1, W2, plan: Optional[K.CsrPlan] = None) -> torch.Tensor:
    xw = torch.matmul(X, W1)
    h = K.spmm_csr(pos, crd, val, xw, relu=True, plan=plan)
    hw = torch.matmul(h, W2)
    return K.spmm_csr(pos, crd, val, hw, plan=plan)
