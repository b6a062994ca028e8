"""Minimal mirror of the reference's sparse tensor container — only what the hot path needs.

Reference: src/scorch/stensor.py (STensor), src/scorch/storage.py (TensorStorage/TensorIndex,
indices forced to int32 at :46-51), src/scorch/format.py (level types d/s/o).  The array layout
is the reference's: a dense level stores nothing, a compressed level ``[pos, crd]``, a coordinate
level ``[crd]``; values are 1-D; dense tensors are the row-major flattening.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import torch

_LEVELS = ("d", "s", "o")


class TensorFormat:
    """Per-level storage: 'd' dense, 's' compressed, 'o' coordinate (reference: format.py:7-27)."""

    def __init__(self, levels: Sequence[str]):
        levels = tuple(levels)
        for lv in levels:
            if lv not in _LEVELS:
                raise ValueError(f"unknown level format {lv!r}")
        self.levels = levels

    def is_dense(self) -> bool:
        return all(lv == "d" for lv in self.levels)

    def __str__(self) -> str:
        return ",".join(self.levels)

    def __repr__(self) -> str:
        return f"TensorFormat({str(self)!r})"

    def __eq__(self, other) -> bool:
        return str(self) == str(parse_format(other)) if other is not None else False

    def __hash__(self) -> int:
        return hash(self.levels)


def parse_format(fmt: Union[str, Sequence[str], TensorFormat]) -> TensorFormat:
    """Accepts "ds", "d,s", ["d","s"] or a TensorFormat (reference: utils.py parse_format)."""
    if isinstance(fmt, TensorFormat):
        return fmt
    if isinstance(fmt, str):
        fmt = [c for c in fmt.replace(",", "").strip()]
    return TensorFormat(list(fmt))


class TensorIndex:
    def __init__(self, mode_indices, tensor_format, mode_order: Optional[List[int]] = None):
        self.mode_indices = [[_as_int32(t) for t in lvl] for lvl in mode_indices]
        self.tensor_format = parse_format(tensor_format)
        self.mode_order = list(mode_order) if mode_order is not None else list(
            range(len(self.tensor_format.levels)))

    @property
    def format(self) -> TensorFormat:
        return self.tensor_format


def _as_int32(t: torch.Tensor) -> torch.Tensor:
    # the reference casts every index tensor to int32 (storage.py:46-51)
    return t if t.dtype == torch.int32 else t.to(torch.int32)


class TensorStorage:
    def __init__(self, index: TensorIndex, value: torch.Tensor):
        self.index = index
        self.value = value


class STensor:
    def __init__(self, shape: Sequence[int], storage: Optional[TensorStorage] = None,
                 index: Optional[TensorIndex] = None, value: Optional[torch.Tensor] = None,
                 name: Optional[str] = None):
        if storage is None:
            storage = TensorStorage(index, value)
        self.shape = tuple(int(s) for s in shape)
        self.storage = storage
        self.name = name or "tensor"

    # -- accessors (same names as the reference) --------------------------------------------------
    @property
    def index(self) -> TensorIndex:
        return self.storage.index

    @property
    def values(self) -> torch.Tensor:
        return self.storage.value

    @property
    def format(self) -> TensorFormat:
        return self.storage.index.tensor_format

    @property
    def dtype(self) -> torch.dtype:
        return self.storage.value.dtype

    @property
    def device(self) -> torch.device:
        return self.storage.value.device

    def dim(self) -> int:
        return len(self.shape)

    def nnz(self) -> int:
        return int(self.storage.value.numel())

    def copy(self) -> "STensor":
        idx = TensorIndex([[t.clone() for t in lvl] for lvl in self.index.mode_indices],
                          self.format, self.index.mode_order)
        return STensor(self.shape, TensorStorage(idx, self.values.clone()), name=self.name)

    def to(self, device) -> "STensor":
        """Move every array to ``device`` (the reference's ``to``/``cuda`` are unimplemented,
        stensor.py:147-154; here they are the way to keep operands resident on the GPU)."""
        idx = TensorIndex([[t.to(device) for t in lvl] for lvl in self.index.mode_indices],
                          self.format, self.index.mode_order)
        return STensor(self.shape, TensorStorage(idx, self.values.to(device)), name=self.name)

    def cuda(self) -> "STensor":
        return self.to(torch.device("cuda", torch.cuda.current_device()))

    def cpu(self) -> "STensor":
        return self.to("cpu")

    def change_mode_order(self, mode_order: List[int]) -> "STensor":
        """Re-lay-out a 2-D tensor so that its physical axes follow ``mode_order`` (reference:
        STensor.change_mode_order, stensor.py:740-896; ``mode_order[p]`` is the logical axis that
        physical axis ``p`` stores).  In place, returns self.  Dense tensors are permuted with
        torch; compressed (``d,s``) and coordinate (``o,o``) tensors go through the device
        transpose kernel (host tensors are moved to the GPU for it and back)."""
        dim = self.dim()
        if sorted(mode_order) != list(range(dim)):
            raise AssertionError("mode_order must be a permutation")
        old = list(self.index.mode_order)
        if old == list(mode_order):
            return self
        if dim != 2:
            raise NotImplementedError("mode-order changes are implemented for 2-D tensors")
        # the only other 2-D order is the transpose of the stored arrays
        rows, cols = self.shape
        f = str(self.format)
        if f == "d,d":
            values = self.values.reshape(rows, cols).t().contiguous().reshape(-1)
            mode_indices = [[], []]
        elif f in ("d,s", "o,o"):
            from . import kernels as K
            on_host = not self.values.is_cuda
            dev = torch.device("cuda", torch.cuda.current_device()) if on_host else self.values.device
            up = lambda t: t.to(dev)
            if f == "d,s":
                pos, crd = (up(t) for t in self.index.mode_indices[1])
            else:
                crd = up(self.index.mode_indices[1][0])
                pos = K.coo_rows_to_csr_pos(up(self.index.mode_indices[0][0]), rows)
            tpos, tcrd, tval = K.csr_transpose(pos, crd, up(self.values), cols)
            back = (lambda t: t.cpu()) if on_host else (lambda t: t)
            if f == "d,s":
                mode_indices = [[], [back(tpos), back(tcrd)]]
            else:
                mode_indices = [[back(K.csr_pos_to_coo_rows(tpos, tcrd.numel()))], [back(tcrd)]]
            values = back(tval)
        else:
            raise NotImplementedError(f"change_mode_order for format {f!r}")
        self.storage = TensorStorage(TensorIndex(mode_indices, self.format, list(mode_order)), values)
        self.shape = (cols, rows)
        return self

    # -- constructors -----------------------------------------------------------------------------
    @staticmethod
    def from_csr(csr_matrix: torch.Tensor, name: Optional[str] = None) -> "STensor":
        """Reference: STensor.from_csr, stensor.py:270-311."""
        if csr_matrix.layout != torch.sparse_csr:
            raise AssertionError("Input tensor must be a sparse CSR tensor.")
        if csr_matrix.dim() != 2:
            raise AssertionError("CSR format is only valid for 2D matrices.")
        idx = TensorIndex([[], [csr_matrix.crow_indices(), csr_matrix.col_indices()]], "d,s")
        return STensor(csr_matrix.shape, TensorStorage(idx, csr_matrix.values()), name=name)

    @staticmethod
    def from_csr_arrays(shape, pos, crd, values, name: Optional[str] = None) -> "STensor":
        idx = TensorIndex([[], [pos, crd]], "d,s")
        return STensor(shape, TensorStorage(idx, values), name=name)

    @staticmethod
    def from_coo(coo_matrix: Optional[torch.Tensor] = None, indices: Optional[torch.Tensor] = None,
                 values: Optional[torch.Tensor] = None, shape: Optional[Tuple[int, ...]] = None,
                 name: Optional[str] = None) -> "STensor":
        """Reference: STensor.from_coo, stensor.py:313-360."""
        if coo_matrix is not None:
            coo_matrix = coo_matrix.coalesce()
            indices, values, shape = coo_matrix.indices(), coo_matrix.values(), coo_matrix.shape
        idx = TensorIndex([[indices[i]] for i in range(len(shape))], ["o"] * len(shape))
        return STensor(tuple(shape), TensorStorage(idx, values), name=name)

    @staticmethod
    def from_torch(tensor: torch.Tensor, name: Optional[str] = None) -> "STensor":
        """Reference: STensor.from_torch, stensor.py:362-452."""
        if tensor.layout == torch.sparse_coo:
            return STensor.from_coo(tensor, name=name)
        if tensor.layout == torch.sparse_csr:
            return STensor.from_csr(tensor, name=name)
        idx = TensorIndex([[] for _ in tensor.shape], ["d"] * tensor.dim())
        return STensor(tuple(tensor.shape), TensorStorage(idx, tensor.flatten()), name=name)

    # -- conversions ------------------------------------------------------------------------------
    def to_torch(self, in_place: bool = True) -> torch.Tensor:
        """Dense STensor -> torch.Tensor (a reshape of the value blob, reference stensor.py:454-475);
        CSR / COO -> the matching torch sparse tensor."""
        f = str(self.format)
        if self.format.is_dense():
            return self.values.view(self.shape)
        if f == "d,s":
            pos, crd = self.index.mode_indices[1]
            return torch.sparse_csr_tensor(pos, crd, self.values, size=self.shape)
        if f == "o,o":
            ind = torch.stack([self.index.mode_indices[0][0], self.index.mode_indices[1][0]]).long()
            return torch.sparse_coo_tensor(ind, self.values, size=self.shape)
        raise NotImplementedError(f"to_torch for format {f!r}")

    def to_dense(self, in_place: bool = True) -> "STensor":
        t = self.to_torch()
        if t.layout != torch.strided:
            t = t.to_dense()
        return STensor.from_torch(t, name=self.name)

    def __add__(self, other: "STensor") -> "STensor":
        """Element-wise sum of two sparse matrices (reference: STensor.__add__)."""
        from . import ops
        return ops.elementwise("add", self, other)

    def __mul__(self, other: "STensor") -> "STensor":
        """Element-wise product of two sparse matrices."""
        from . import ops
        return ops.elementwise("mul", self, other)

    def __repr__(self) -> str:
        return f"STensor(shape={self.shape}, format='{self.format}', dtype={self.dtype}, nnz={self.nnz()})"
