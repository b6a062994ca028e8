"""Device-tensor front end of the C ABI: every function takes CUDA torch tensors (torch is used
for device memory and streams only) and launches the sm_100a kernels through ``_lib``.

No function here computes on the CPU; CPU tensors are rejected (the host-tensor convenience
path lives in ``scorch_ops``).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple, Union

import torch

from . import _lib
from ._lib import SB_F32, SB_F64, SB_I32, SB_I64, check

_DTYPE_CODE = {torch.float32: SB_F32, torch.float64: SB_F64, torch.int32: SB_I32, torch.int64: SB_I64}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor (no CPU path exists)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _wrote(t: torch.Tensor) -> torch.Tensor:
    """The library has written `t` through its raw pointer: bump the tensor's version counter, as
    a torch in-place op would, so that whatever is cached against the tensor's version (row
    plans, the all-ones verdict of a mask) is not reused for the new contents."""
    torch.autograd.graph.increment_version(t)
    return t


CSR_VIOLATIONS = {1: "pos[0] is not 0", 2: "pos[m] is not nnz", 3: "row pointer out of [0, nnz]",
                  4: "row pointers decrease", 5: "column index out of range", 6: "columns of a row not strictly ascending"}


def csr_validate(pos: torch.Tensor, crd: torch.Tensor, n: int, sorted_unique: bool = True):
    """Device-side check of a CSR structure against what the kernels assume (they trust their
    inputs, like the reference's loops).  Returns None when it is valid, else
    ``(message, row, entry, value)`` for the first violation (smallest row, then entry)."""
    pos, crd = _dev(pos, torch.int32, "pos"), _dev(crd, torch.int32, "crd")
    L = _lib.lib()
    ws = torch.empty(L.sb_csr_validate_workspace_bytes(), dtype=torch.uint8, device=pos.device)
    report = (C.c_int32 * 4)()
    with torch.cuda.device(pos.device):
        check(L.sb_csr_validate(pos.numel() - 1, int(n), crd.numel(), pos.data_ptr(), _ptr(crd),
                                1 if sorted_unique else 0, report, ws.data_ptr(), ws.numel(), _stream()))
    if report[0] == 0:
        return None
    return CSR_VIOLATIONS.get(report[0], f"code {report[0]}"), int(report[1]), int(report[2]), int(report[3])


def _validated(pos, crd, n: int, what: str, sorted_unique: bool = False) -> None:
    """With SCORCH_B200_VALIDATE=1 every CSR operand is checked before a kernel reads it (a
    synchronising pass over pos and crd: a debugging aid, off by default)."""
    if os.environ.get("SCORCH_B200_VALIDATE") != "1":
        return
    bad = csr_validate(pos, crd, n, sorted_unique)
    if bad is not None:
        raise ValueError(f"{what}: invalid CSR operand: {bad[0]} (row {bad[1]}, entry {bad[2]}, value {bad[3]})")


class CsrPlan:
    """Heavy-row plan of one CSR matrix (depends on ``pos`` only); see include/scorch_b200.h."""

    def __init__(self, pos: torch.Tensor, nnz: int):
        pos = _dev(pos, torch.int32, "pos")
        self.m = pos.numel() - 1
        self.nnz = int(nnz)
        L = _lib.lib()
        nbytes = L.sb_csr_plan_bytes(self.m, self.nnz)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=pos.device)
        with torch.cuda.device(pos.device):
            check(L.sb_csr_plan_build(self.m, self.nnz, pos.data_ptr(), self.buf.data_ptr(), nbytes,
                                      _stream()))
            h, s = C.c_int64(0), C.c_int64(0)
            check(L.sb_csr_plan_counts(self.buf.data_ptr(), C.byref(h), C.byref(s), _stream()))
        self.heavy_rows, self.segments = int(h.value), int(s.value)
        self._scratch: Optional[torch.Tensor] = None

    def scratch(self, nbytes: int) -> torch.Tensor:
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=self.buf.device)
        return self._scratch


def plan_for(pos: torch.Tensor, nnz: int) -> CsrPlan:
    """Plan cached on the ``pos`` tensor object (rebuilt if the tensor was written in place)."""
    cached = getattr(pos, "_sb_plan", None)
    if cached is not None and cached[0] == pos._version and cached[1].nnz == nnz:
        return cached[1]
    plan = CsrPlan(pos, nnz)
    try:
        pos._sb_plan = (pos._version, plan)
    except Exception:  # pragma: no cover - tensors always accept attributes
        pass
    return plan


class BlockPlan:
    """Dense 16x16 blocks + remainder entries of one CSR pattern (depends on ``pos``/``crd`` only);
    see include/scorch_b200.h.  ``dense_fraction`` tells whether the blocked kernels pay off."""

    def __init__(self, pos: torch.Tensor, crd: torch.Tensor, n: Optional[int] = None):
        pos, crd = _dev(pos, torch.int32, "pos"), _dev(crd, torch.int32, "crd")
        self.m, self.nnz = pos.numel() - 1, crd.numel()
        L = _lib.lib()
        nbytes = L.sb_block_plan_bytes(self.m, self.nnz)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=pos.device)
        b, r = C.c_int64(0), C.c_int64(0)
        with torch.cuda.device(pos.device):
            check(L.sb_block_plan_build(self.m, self.m if n is None else n, self.nnz, pos.data_ptr(),
                                        crd.data_ptr(), self.buf.data_ptr(), nbytes, C.byref(b),
                                        C.byref(r), _stream()))
        self.blocks, self.rem_nnz = int(b.value), int(r.value)

    @property
    def dense_fraction(self) -> float:
        return (self.blocks * 256) / self.nnz if self.nnz else 0.0


def block_plan_for(pos: torch.Tensor, crd: torch.Tensor) -> BlockPlan:
    """Block plan cached on the ``crd`` tensor object (rebuilt after in-place writes)."""
    cached = getattr(crd, "_sb_block_plan", None)
    if cached is not None and cached[0] == (pos._version, crd._version, pos.data_ptr()):
        return cached[1]
    plan = BlockPlan(pos, crd)
    crd._sb_block_plan = ((pos._version, crd._version, pos.data_ptr()), plan)
    return plan


class AttnPlan:
    """Blocks (aligned 16x16, at least 64 stored entries, with per-row column masks) + remaining
    entries of one CSR attention mask; see include/scorch_b200.h.  ``block_fraction`` is the share
    of the stored entries that lie in blocks."""

    def __init__(self, pos: torch.Tensor, crd: torch.Tensor, n: Optional[int] = None):
        pos, crd = _dev(pos, torch.int32, "pos"), _dev(crd, torch.int32, "crd")
        self.m, self.nnz = pos.numel() - 1, crd.numel()
        self.n = self.m if n is None else n
        L = _lib.lib()
        nbytes = L.sb_attn_plan_bytes(self.m, self.nnz)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=pos.device)
        b, r = C.c_int64(0), C.c_int64(0)
        with torch.cuda.device(pos.device):
            check(L.sb_attn_plan_build(self.m, self.n, self.nnz, pos.data_ptr(), crd.data_ptr(),
                                       self.buf.data_ptr(), nbytes, C.byref(b), C.byref(r), _stream()))
        self.blocks, self.rem_nnz = int(b.value), int(r.value)
        self._scratch: Optional[torch.Tensor] = None

    @property
    def block_fraction(self) -> float:
        return (self.nnz - self.rem_nnz) / self.nnz if self.nnz else 0.0

    def scratch(self, nbytes: int) -> torch.Tensor:
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.buf.device)
        return self._scratch


def attn_plan_for(pos: torch.Tensor, crd: torch.Tensor) -> AttnPlan:
    """Attention plan of a square mask, cached on the ``crd`` tensor object (rebuilt after
    in-place writes)."""
    cached = getattr(crd, "_sb_attn_plan", None)
    if cached is not None and cached[0] == (pos._version, crd._version, pos.data_ptr()):
        return cached[1]
    plan = AttnPlan(pos, crd)
    crd._sb_attn_plan = ((pos._version, crd._version, pos.data_ptr()), plan)
    return plan


class AttnBandPlan:
    """Band plan of one CSR attention mask for the tcgen05 path: per 128-row tile a window of 384
    columns around the diagonal, the stored columns inside it as bits per row, and a CSR list of
    the entries outside; see include/scorch_b200.h.  ``inside_fraction`` is the share of the
    stored entries that lie inside the windows."""

    ROWS, COLS = 128, 384

    def __init__(self, pos: torch.Tensor, crd: torch.Tensor, n: Optional[int] = None):
        pos, crd = _dev(pos, torch.int32, "pos"), _dev(crd, torch.int32, "crd")
        self.m, self.nnz = pos.numel() - 1, crd.numel()
        self.n = self.m if n is None else n
        L = _lib.lib()
        nbytes = L.sb_attn_band_plan_bytes(self.m, self.nnz)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=pos.device)
        a, r = C.c_int64(0), C.c_int64(0)
        with torch.cuda.device(pos.device):
            check(L.sb_attn_band_plan_build(self.m, self.n, self.nnz, pos.data_ptr(), crd.data_ptr(),
                                            self.buf.data_ptr(), nbytes, C.byref(a), C.byref(r), _stream()))
        self.inside, self.rem_nnz = int(a.value), int(r.value)
        self._scratch: Optional[torch.Tensor] = None

    @property
    def inside_fraction(self) -> float:
        return self.inside / self.nnz if self.nnz else 0.0

    @property
    def window_fill(self) -> float:
        """Stored entries inside the windows / window cells (rows x 384)."""
        return self.inside / (self.m * self.COLS) if self.m else 0.0

    def window_start(self, tile: int) -> int:
        return max(0, min(tile * self.ROWS - (self.COLS - self.ROWS) // 2, self.n - self.COLS))

    scratch = AttnPlan.scratch


def attn_band_plan_for(pos: torch.Tensor, crd: torch.Tensor) -> AttnBandPlan:
    """Band plan of a square mask, cached on the ``crd`` tensor object (rebuilt after in-place
    writes)."""
    cached = getattr(crd, "_sb_attn_band_plan", None)
    if cached is not None and cached[0] == (pos._version, crd._version, pos.data_ptr()):
        return cached[1]
    plan = AttnBandPlan(pos, crd)
    crd._sb_attn_band_plan = ((pos._version, crd._version, pos.data_ptr()), plan)
    return plan


def attn_band_status() -> int:
    """0 unless a tensor-core wait of the band kernel ran out since the library was loaded
    (synchronises the device)."""
    return int(_lib.lib().sb_attn_band_status())


def attn_band_probe(Q: torch.Tensor, Kmat: torch.Tensor, V: Optional[torch.Tensor] = None, tile: int = 0,
                    with_clocks: bool = False):
    """Self-test of the tcgen05 path on one tile, every window column counted as stored, scale 1.
    Returns (raw, image, clocks): raw = the 128 x 384 products of rows [128 tile, +128) of Q with the rows
    of Kmat in the tile's window (zeros outside the matrices); image = the tile's 128 x 512
    tensor-memory cells at the end (hi parts of P, unnormalised P V, lo parts of P's last 64
    columns); clocks (``with_clocks``; raw is then left zero) = 36 SM clock values at the kernel's phase
    boundaries."""
    Q, Kmat = _dev(Q, torch.float32, "Q").contiguous(), _dev(Kmat, torch.float32, "K").contiguous()
    V = Kmat if V is None else _dev(V, torch.float32, "V").contiguous()
    if Q.dim() != 2 or Kmat.dim() != 2 or Q.shape[1] != 64 or Kmat.shape[1] != 64 or V.shape != Kmat.shape:
        raise ValueError("Q must be (rows, 64), K and V (cols, 64)")
    raw = torch.zeros((AttnBandPlan.ROWS, AttnBandPlan.COLS), dtype=torch.float32, device=Q.device)
    image = torch.zeros((AttnBandPlan.ROWS, 512), dtype=torch.float32, device=Q.device)
    clocks = torch.zeros(36, dtype=torch.int64, device=Q.device) if with_clocks else None
    with torch.cuda.device(Q.device):
        check(_lib.lib().sb_attn_band_probe(Q.shape[0], Kmat.shape[0], 64, int(tile), Q.data_ptr(), 64,
                                            Kmat.data_ptr(), 64, V.data_ptr(), 64, raw.data_ptr(),
                                            image.data_ptr(), _ptr(clocks), _stream()))
    return _wrote(raw), _wrote(image), clocks


FUSED_ATTENTION_D = (32, 64)


def _mask_is_all_ones(mask_val: torch.Tensor) -> bool:
    """True when every mask value is exactly 1.0 (a pure pattern mask): multiplying by it is the
    identity, so the kernels need not read it.  Checked once per tensor (one synchronising
    reduction) and remembered on the tensor object until it is written in place."""
    cached = getattr(mask_val, "_sb_all_ones", None)
    if cached is not None and cached[0] == (mask_val._version, mask_val.data_ptr()):
        return cached[1]
    ones = bool((mask_val == 1.0).all().item())
    mask_val._sb_all_ones = ((mask_val._version, mask_val.data_ptr()), ones)
    return ones


def sparse_attention_csr(pos, crd, mask_val, Q, Kmat, V, scale: float = 1.0,
                         attn_plan: Optional[Union[AttnPlan, AttnBandPlan]] = None,
                         out: Optional[torch.Tensor] = None, stages: int = 3) -> torch.Tensor:
    """O = softmax_rows(scale * mask_val .* (Q Kmat^T) on the stored entries) V in one call, the
    scores never written out.  Q: (m, d) or (batch, m, d); Kmat, V: (n, d) or (batch, n, d); head
    dimension d in FUSED_ATTENTION_D.  Rows without stored entries give zero rows.
    ``attn_plan``: an ``AttnPlan`` (16x16 blocks, mma.sync) or an ``AttnBandPlan`` (128-row tiles of
    a band on tcgen05, d = 64); default: the block plan.
    ``stages``: 3 = the whole call; 1, 2 = its two kernels one by one (scattered entries, then
    blocks / tiles; same arguments and ``out``), for callers that time them."""
    pos = _dev(pos, torch.int32, "pos")
    crd = _dev(crd, torch.int32, "crd")
    m, nnz = pos.numel() - 1, crd.numel()
    Q, Kmat, V = (_dev(x, torch.float32, nm).contiguous() for x, nm in ((Q, "Q"), (Kmat, "K"), (V, "V")))
    batched = Q.dim() == 3
    batch = Q.shape[0] if batched else 1
    d, n = Q.shape[-1], Kmat.shape[-2]
    if d not in FUSED_ATTENTION_D:
        raise ValueError(f"head dimension must be one of {FUSED_ATTENTION_D}")
    if Q.shape[-2] != m or Kmat.shape != V.shape or Kmat.shape[-1] != d or Kmat.dim() != Q.dim() \
            or (batched and Kmat.shape[0] != batch):
        raise ValueError("Q must be (.., m, d) and K, V (.., n, d) with the same batch")
    if mask_val is not None:
        mask_val = _dev(mask_val, torch.float32, "mask_val")
        if mask_val.numel() != nnz:
            raise ValueError("mask_val and crd differ in length")
        if _mask_is_all_ones(mask_val):
            mask_val = None
    if attn_plan is None:
        attn_plan = AttnPlan(pos, crd, n=n) if n != m else attn_plan_for(pos, crd)
    if attn_plan.m != m or attn_plan.nnz != nnz or attn_plan.n != n:
        raise ValueError("attention plan was built for another mask")
    shape = (batch, m, d) if batched else (m, d)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=Q.device)
    elif not (out.is_cuda and out.dtype == torch.float32 and tuple(out.shape) == shape and out.is_contiguous()):
        raise ValueError(f"out must be a contiguous float32 CUDA tensor of shape {shape}")
    L = _lib.lib()
    sbytes = L.sb_sparse_attention_scratch_bytes(m, attn_plan.rem_nnz, batch)
    scratch = attn_plan.scratch(sbytes) if sbytes else None
    if isinstance(attn_plan, AttnBandPlan):
        if d != 64:
            raise ValueError("the band path needs head dimension 64")
        with torch.cuda.device(Q.device):
            check(L.sb_sparse_attention_band_f32(m, n, d, nnz, pos.data_ptr(), crd.data_ptr(), _ptr(mask_val),
                                                 Q.data_ptr(), d, Kmat.data_ptr(), d, V.data_ptr(), d,
                                                 float(scale), out.data_ptr(), d, batch, m * d, n * d, n * d,
                                                 m * d, attn_plan.buf.data_ptr(), attn_plan.rem_nnz,
                                                 _ptr(scratch), sbytes, int(stages), _stream()))
        return _wrote(out)
    with torch.cuda.device(Q.device):
        check(L.sb_sparse_attention_csr_f32(m, n, d, nnz, pos.data_ptr(), crd.data_ptr(), _ptr(mask_val),
                                            Q.data_ptr(), d, Kmat.data_ptr(), d, V.data_ptr(), d,
                                            float(scale), out.data_ptr(), d, batch, m * d, n * d, n * d,
                                            m * d, attn_plan.buf.data_ptr(), attn_plan.blocks,
                                            attn_plan.rem_nnz, _ptr(scratch), sbytes, int(stages), _stream()))
    return _wrote(out)


BLOCKED_MIN_DENSE_FRACTION = 0.5   # below this the gather kernels alone are used
_BLOCKED_SDDMM_D = (16, 32, 64, 128)
_BLOCKED_SPMM_K = (32, 64, 128)


def _row_major_2d(t: torch.Tensor, name: str) -> torch.Tensor:
    """2-D operand whose rows are contiguous; the row pitch (leading dimension) may exceed the width."""
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1]:
        return t
    return t.contiguous()


def spmm_csr(pos, crd, val, B, bias=None, relu: bool = False, plan: Optional[CsrPlan] = None,
             out: Optional[torch.Tensor] = None, n: Optional[int] = None,
             block_plan: Optional[BlockPlan] = None, accumulate: bool = False) -> torch.Tensor:
    """C = act(bias + A @ B) for CSR A.  ``B`` is (n, k) or (batch, n, k); ``val`` is (nnz,) —
    shared by all batch items — or (batch, nnz).  Returns (m, k) or (batch, m, k).
    2-D ``B`` / ``out`` may be column slices of wider row-major buffers (row pitch > k).
    ``accumulate``: act(bias + out + A @ B), ``out`` required."""
    pos = _dev(pos, torch.int32, "pos")
    crd = _dev(crd, torch.int32, "crd")
    m, nnz = pos.numel() - 1, crd.numel()
    if val.dtype != torch.float32:
        return _spmm_typed(pos, crd, val, B, n)
    val = _dev(val, torch.float32, "val")
    if not (isinstance(B, torch.Tensor) and B.is_cuda and B.dtype == torch.float32):
        B = _dev(B, torch.float32, "B")
    batched = B.dim() == 3
    B = B.contiguous() if batched else _row_major_2d(B, "B")
    batch = B.shape[0] if batched else 1
    nb, k = B.shape[-2], B.shape[-1]
    _validated(pos, crd, nb, "spmm_csr")
    ldb = k if batched else B.stride(0)
    if val.dim() == 2:
        if val.shape[0] != batch or val.shape[1] != nnz:
            raise ValueError("val must be (nnz,) or (batch, nnz)")
        stride_val = nnz
    else:
        if val.numel() != nnz:
            raise ValueError("val and crd differ in length")
        stride_val = 0
    if bias is not None:
        bias = _dev(bias, torch.float32, "bias")
        if bias.numel() != k:
            raise ValueError("bias must have k elements")
    shape = (batch, m, k) if batched else (m, k)
    if accumulate and out is None:
        raise ValueError("accumulate needs the tensor to add to (out=)")
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=B.device)
        ldc = k
    else:
        if not (out.is_cuda and out.dtype == torch.float32 and tuple(out.shape) == shape):
            raise ValueError(f"out must be a float32 CUDA tensor of shape {shape}")
        if batched:
            if not out.is_contiguous():
                raise ValueError("batched out must be contiguous")
            ldc = k
        else:
            if out.stride(1) != 1 or out.stride(0) < k:
                raise ValueError("out rows must be contiguous")
            ldc = out.stride(0)
    if plan is None:
        plan = plan_for(pos, nnz)
    L = _lib.lib()
    if (block_plan is not None and not accumulate and block_plan.blocks > 0 and plan.segments == 0
            and k in _BLOCKED_SPMM_K and ldb % 4 == 0 and ldc % 4 == 0):
        with torch.cuda.device(B.device):
            check(L.sb_spmm_csr_blocked_f32(m, nb if n is None else n, k, nnz, pos.data_ptr(),
                                            crd.data_ptr(), val.data_ptr(), B.data_ptr(), ldb,
                                            _ptr(bias), int(bool(relu)), out.data_ptr(), ldc, batch,
                                            stride_val, nb * k, m * k, block_plan.buf.data_ptr(),
                                            block_plan.blocks, block_plan.rem_nnz, _stream()))
        return _wrote(out)
    sbytes = L.sb_spmm_csr_scratch_bytes(plan.segments, k, batch)
    scratch = plan.scratch(sbytes) if sbytes else None
    with torch.cuda.device(B.device):
        fn = L.sb_spmm_csr_acc_f32 if accumulate else L.sb_spmm_csr_f32
        check(fn(m, nb if n is None else n, k, nnz, pos.data_ptr(), crd.data_ptr(),
                 val.data_ptr(), B.data_ptr(), ldb, _ptr(bias), int(bool(relu)),
                 out.data_ptr(), ldc, batch, stride_val, nb * k, m * k,
                 plan.buf.data_ptr(), plan.segments, _ptr(scratch), sbytes, _stream()))
    return _wrote(out)


def _spmm_typed(pos, crd, val, B, n):
    code = _DTYPE_CODE.get(val.dtype)
    if code is None:
        raise TypeError(f"unsupported value dtype {val.dtype}")
    val = _dev(val, val.dtype, "val")
    B = _dev(B, val.dtype, "B")
    if B.dim() != 2:
        raise ValueError("typed SpMM takes a 2-D dense operand")
    m, nnz, k = pos.numel() - 1, crd.numel(), B.shape[1]
    out = torch.empty((m, k), dtype=val.dtype, device=B.device)
    with torch.cuda.device(B.device):
        check(_lib.lib().sb_spmm_csr_typed(code, m, B.shape[0] if n is None else n, k, nnz,
                                           pos.data_ptr(), crd.data_ptr(), val.data_ptr(),
                                           B.data_ptr(), k, out.data_ptr(), k, _stream()))
    return out


def spmv_csr(pos, crd, val, x, plan: Optional[CsrPlan] = None) -> torch.Tensor:
    """y = A @ x for CSR A (``plan`` is accepted for symmetry with ``spmm_csr`` and not needed:
    the fp32 kernel is balanced by entries, not rows)."""
    pos = _dev(pos, torch.int32, "pos")
    crd = _dev(crd, torch.int32, "crd")
    m, nnz = pos.numel() - 1, crd.numel()
    code = _DTYPE_CODE.get(val.dtype)
    if code is None:
        raise TypeError(f"unsupported value dtype {val.dtype}")
    val = _dev(val, val.dtype, "val")
    x = _dev(x, val.dtype, "x")
    _validated(pos, crd, x.numel(), "spmv_csr")
    y = torch.empty(m, dtype=val.dtype, device=x.device)
    L = _lib.lib()
    with torch.cuda.device(x.device):
        if code != SB_F32:
            check(L.sb_spmv_csr_typed(code, m, x.numel(), nnz, pos.data_ptr(), crd.data_ptr(),
                                      val.data_ptr(), x.data_ptr(), y.data_ptr(), _stream()))
            return y
        sbytes = L.sb_spmv_csr_scratch_bytes(nnz)
        scratch = torch.empty(max(sbytes, 16), dtype=torch.uint8, device=x.device)
        check(L.sb_spmv_csr_f32(m, x.numel(), nnz, pos.data_ptr(), crd.data_ptr(), val.data_ptr(),
                                x.data_ptr(), y.data_ptr(), scratch.data_ptr(), sbytes, _stream()))
    return y


def _qk(Q, K):
    Q = _dev(Q, torch.float32, "Q")
    K = _dev(K, torch.float32, "K")
    if Q.dim() != K.dim() or Q.dim() not in (2, 3) or Q.shape[-1] != K.shape[-1]:
        raise ValueError("Q and K must be (rows, d) or (batch, rows, d) with equal d")
    batch = Q.shape[0] if Q.dim() == 3 else 1
    if K.dim() == 3 and K.shape[0] != batch:
        raise ValueError("Q and K differ in batch size")
    return Q, K, batch


def sddmm_csr(pos, crd, mask_val, Q, K, want_coords: bool = False,
              out: Optional[torch.Tensor] = None, block_plan: Optional[BlockPlan] = None):
    """out[p] = mask_val[p] * <Q[i_p], K[j_p]> over the entries of a CSR mask, entry order kept.
    Returns values (nnz,) or (batch, nnz); with ``want_coords`` also fresh int32 (row, col)."""
    pos = _dev(pos, torch.int32, "pos")
    crd = _dev(crd, torch.int32, "crd")
    Q, K, batch = _qk(Q, K)
    m, nnz, d = pos.numel() - 1, crd.numel(), Q.shape[-1]
    _validated(pos, crd, K.shape[-2], "sddmm_csr")
    if mask_val is not None:
        mask_val = _dev(mask_val, torch.float32, "mask_val")
    shape = (batch, nnz) if Q.dim() == 3 else (nnz,)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=Q.device)
    elif not (out.is_cuda and out.dtype == torch.float32 and out.is_contiguous()
              and tuple(out.shape) == shape):
        raise ValueError(f"out must be a contiguous float32 CUDA tensor of shape {shape}")
    if block_plan is not None and block_plan.blocks > 0 and not want_coords and d in _BLOCKED_SDDMM_D:
        with torch.cuda.device(Q.device):
            check(_lib.lib().sb_sddmm_csr_blocked_f32(
                m, K.shape[-2], d, nnz, pos.data_ptr(), crd.data_ptr(), _ptr(mask_val), Q.data_ptr(), d,
                K.data_ptr(), d, out.data_ptr(), batch, Q.shape[-2] * d, K.shape[-2] * d, nnz,
                block_plan.buf.data_ptr(), block_plan.blocks, block_plan.rem_nnz, _stream()))
        return _wrote(out)
    row = col = None
    if want_coords:
        row = torch.empty(nnz, dtype=torch.int32, device=Q.device)
        col = torch.empty(nnz, dtype=torch.int32, device=Q.device)
    with torch.cuda.device(Q.device):
        check(_lib.lib().sb_sddmm_csr_f32(m, K.shape[-2], d, nnz, pos.data_ptr(), crd.data_ptr(),
                                          _ptr(mask_val), Q.data_ptr(), d, K.data_ptr(), d,
                                          out.data_ptr(), _ptr(row), _ptr(col), batch,
                                          Q.shape[-2] * d, K.shape[-2] * d, nnz, _stream()))
    _wrote(out)
    return (out, row, col) if want_coords else out


def sddmm_coo(row, col, mask_val, Q, K):
    row = _dev(row, torch.int32, "row")
    col = _dev(col, torch.int32, "col")
    Q, K, batch = _qk(Q, K)
    nnz, d = col.numel(), Q.shape[-1]
    if mask_val is not None:
        mask_val = _dev(mask_val, torch.float32, "mask_val")
    out = torch.empty((batch, nnz) if Q.dim() == 3 else (nnz,), dtype=torch.float32, device=Q.device)
    with torch.cuda.device(Q.device):
        check(_lib.lib().sb_sddmm_coo_f32(Q.shape[-2], K.shape[-2], d, nnz, row.data_ptr(),
                                          col.data_ptr(), _ptr(mask_val), Q.data_ptr(), d,
                                          K.data_ptr(), d, out.data_ptr(), batch, Q.shape[-2] * d,
                                          K.shape[-2] * d, nnz, _stream()))
    return out


def csr_row_softmax(pos, val, scale: float = 1.0, out: Optional[torch.Tensor] = None):
    pos = _dev(pos, torch.int32, "pos")
    val = _dev(val, torch.float32, "val")
    m = pos.numel() - 1
    nnz = val.shape[-1]
    batch = val.shape[0] if val.dim() == 2 else 1
    if out is None:
        out = torch.empty_like(val)
    with torch.cuda.device(val.device):
        check(_lib.lib().sb_csr_row_softmax_f32(m, nnz, pos.data_ptr(), val.data_ptr(),
                                                out.data_ptr(), float(scale), batch, nnz, _stream()))
    return _wrote(out)


def spgemm_csr(Apos, Acrd, Aval, Bpos, Bcrd, Bval, n: int, timings: Optional[dict] = None
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """C = A @ B for CSR operands.  Returns (Cpos int32, Ccrd int32 ascending per row, Cval)."""
    Apos, Acrd = _dev(Apos, torch.int32, "Apos"), _dev(Acrd, torch.int32, "Acrd")
    Bpos, Bcrd = _dev(Bpos, torch.int32, "Bpos"), _dev(Bcrd, torch.int32, "Bcrd")
    code = _DTYPE_CODE.get(Aval.dtype)
    if code is None or Bval.dtype != Aval.dtype:
        raise TypeError("SpGEMM operands must share one of f32/f64/i32/i64")
    Aval, Bval = _dev(Aval, Aval.dtype, "Aval"), _dev(Bval, Aval.dtype, "Bval")
    m, kb = Apos.numel() - 1, Bpos.numel() - 1
    _validated(Apos, Acrd, kb, "spgemm_csr (A)", sorted_unique=True)
    _validated(Bpos, Bcrd, n, "spgemm_csr (B)", sorted_unique=True)
    L = _lib.lib()
    dev = Aval.device
    with torch.cuda.device(dev):
        wbytes = L.sb_spgemm_workspace_bytes(m, n, code)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        Cpos = torch.empty(m + 1, dtype=torch.int32, device=dev)
        total = C.c_int64(0)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if timings is not None else None
        if ev:
            ev[0].record()
        check(L.sb_spgemm_symbolic(m, kb, n, Apos.data_ptr(), Acrd.data_ptr(), Bpos.data_ptr(),
                                   Bcrd.data_ptr(), Cpos.data_ptr(), C.byref(total),
                                   ws.data_ptr(), wbytes, _stream()))
        if ev:
            ev[1].record()
        Ccrd = torch.empty(total.value, dtype=torch.int32, device=dev)
        Cval = torch.empty(total.value, dtype=Aval.dtype, device=dev)
        check(L.sb_spgemm_numeric(code, m, kb, n, Apos.data_ptr(), Acrd.data_ptr(), Aval.data_ptr(),
                                  Bpos.data_ptr(), Bcrd.data_ptr(), Bval.data_ptr(),
                                  Cpos.data_ptr(), Ccrd.data_ptr(), Cval.data_ptr(), ws.data_ptr(),
                                  wbytes, _stream()))
        if ev:
            ev[2].record()
            ev[2].synchronize()
            timings["symbolic_ms"] = ev[0].elapsed_time(ev[1])
            timings["numeric_ms"] = ev[1].elapsed_time(ev[2])
    return Cpos, Ccrd, Cval


def partition_rows_by_nnz(pos: torch.Tensor, parts: int) -> list:
    """Row bounds [r_0=0, r_1, ..., r_parts=m] of nnz-balanced contiguous row blocks."""
    pos = _dev(pos, torch.int32, "pos")
    out = torch.empty(parts + 1, dtype=torch.int64, device=pos.device)
    with torch.cuda.device(pos.device):
        check(_lib.lib().sb_partition_rows_by_nnz(pos.numel() - 1, pos.data_ptr(), parts,
                                                  out.data_ptr(), _stream()))
    return out.cpu().tolist()


def coo_rows_to_csr_pos(row_sorted: torch.Tensor, m: int) -> torch.Tensor:
    row_sorted = _dev(row_sorted, torch.int32, "row")
    pos = torch.empty(m + 1, dtype=torch.int32, device=row_sorted.device)
    with torch.cuda.device(row_sorted.device):
        check(_lib.lib().sb_coo_rows_to_csr_pos(m, row_sorted.numel(), row_sorted.data_ptr(),
                                                pos.data_ptr(), _stream()))
    return pos


def csr_pos_to_coo_rows(pos: torch.Tensor, nnz: int) -> torch.Tensor:
    pos = _dev(pos, torch.int32, "pos")
    row = torch.empty(nnz, dtype=torch.int32, device=pos.device)
    with torch.cuda.device(pos.device):
        check(_lib.lib().sb_csr_pos_to_coo_rows(pos.numel() - 1, nnz, pos.data_ptr(),
                                                row.data_ptr(), _stream()))
    return row


def dense_to_csr(A: torch.Tensor):
    """(pos, crd, val) of the non-zero entries of a 2-D float32 CUDA matrix, rows and columns
    ascending — torch's ``to_sparse_csr()`` on the device through the library (the reference's
    callers convert pruned weight matrices this way, bench/bench_sparse_autoencoder.py:233,261)."""
    A = _row_major_2d(_dev(A, torch.float32, "A"), "A")
    if A.dim() != 2:
        raise ValueError("A must be 2-D")
    m, n = A.shape
    L = _lib.lib()
    pos = torch.empty(m + 1, dtype=torch.int32, device=A.device)
    wbytes = L.sb_dense_to_csr_workspace_bytes(m)
    ws = torch.empty(wbytes, dtype=torch.uint8, device=A.device)
    nnz = C.c_int64(0)
    with torch.cuda.device(A.device):
        check(L.sb_dense_to_csr_count(m, n, A.data_ptr(), A.stride(0), pos.data_ptr(), C.byref(nnz),
                                      ws.data_ptr(), wbytes, _stream()))
        crd = torch.empty(nnz.value, dtype=torch.int32, device=A.device)
        val = torch.empty(nnz.value, dtype=torch.float32, device=A.device)
        check(L.sb_dense_to_csr_fill(m, n, A.data_ptr(), A.stride(0), pos.data_ptr(), crd.data_ptr(),
                                     val.data_ptr(), _stream()))
    return pos, crd, val


def csr_sym_normalize(pos: torch.Tensor, crd: torch.Tensor) -> torch.Tensor:
    """Values d_i^-1/2 d_j^-1/2 of the symmetric normalisation D^-1/2 (A + I) D^-1/2 for a square
    CSR pattern that already holds the self-loops; d = stored entries per row
    (reference: compute_normalized_adj, bench/bench_gcn.py:233-267)."""
    pos = _dev(pos, torch.int32, "pos")
    crd = _dev(crd, torch.int32, "crd")
    val = torch.empty(crd.numel(), dtype=torch.float32, device=crd.device)
    with torch.cuda.device(crd.device):
        check(_lib.lib().sb_csr_sym_normalize_f32(pos.numel() - 1, crd.numel(), pos.data_ptr(),
                                                  crd.data_ptr(), val.data_ptr(), _stream()))
    return val


def csr_transpose(pos: torch.Tensor, crd: torch.Tensor, val: Optional[torch.Tensor], n: int):
    """(tpos, tcrd, tval) of the transpose of the (m x n) CSR matrix (pos, crd, val): its CSC form,
    output rows in ascending source-row order.  ``val`` may be None (pattern only).  What the
    reference's front end does with torch ops for an operand stored in the other mode order
    (src/scorch/stensor.py:785-896)."""
    pos = _dev(pos, torch.int32, "pos")
    crd = _dev(crd, torch.int32, "crd")
    m, nnz = pos.numel() - 1, crd.numel()
    code = SB_F32
    if val is not None:
        code = _DTYPE_CODE.get(val.dtype)
        if code is None:
            raise TypeError(f"unsupported value dtype {val.dtype}")
        val = _dev(val, val.dtype, "val")
        if val.numel() != nnz:
            raise ValueError("val and crd differ in length")
    L = _lib.lib()
    dev = crd.device
    tpos = torch.empty(n + 1, dtype=torch.int32, device=dev)
    tcrd = torch.empty(nnz, dtype=torch.int32, device=dev)
    tval = None if val is None else torch.empty_like(val)
    wbytes = L.sb_csr_transpose_workspace_bytes(n, nnz)
    ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check(L.sb_csr_transpose(code, m, n, nnz, pos.data_ptr(), crd.data_ptr(), _ptr(val),
                                 tpos.data_ptr(), tcrd.data_ptr(), _ptr(tval), ws.data_ptr(), wbytes,
                                 _stream()))
    return tpos, tcrd, tval


def topk_rows_to_csr(X: torch.Tensor, k: int, relu: bool = False):
    """(pos, crd, val) with exactly k entries per row: the k largest values of each row of the
    dense float32 matrix ``X``, columns ascending (ties go to the lower column), values clamped at
    zero with ``relu`` — the activations of a top-k sparse autoencoder, ready for ``spmm_csr``."""
    X = _row_major_2d(_dev(X, torch.float32, "X"), "X")
    if X.dim() != 2:
        raise ValueError("X must be 2-D")
    m, n = X.shape
    if not 0 <= k <= n:
        raise ValueError("k must be in [0, columns]")
    pos = torch.empty(m + 1, dtype=torch.int32, device=X.device)
    crd = torch.empty(m * k, dtype=torch.int32, device=X.device)
    val = torch.empty(m * k, dtype=torch.float32, device=X.device)
    with torch.cuda.device(X.device):
        check(_lib.lib().sb_topk_rows_to_csr_f32(m, n, k, X.data_ptr(), X.stride(0), int(bool(relu)),
                                                 pos.data_ptr(), crd.data_ptr(), val.data_ptr(), _stream()))
    return pos, crd, val


def csr_ewise(op: str, Apos, Acrd, Aval, Bpos, Bcrd, Bval):
    """Element-wise ``"mul"`` (stored where both operands store an entry) or ``"add"`` (where
    either does) of two CSR matrices of the same shape: (Cpos, Ccrd, Cval), columns ascending,
    symbolic structure kept.  The loops the reference's compiler emits for
    ``einsum("ij,ij->ij", A, B)`` and ``A + B`` over compressed operands."""
    code_op = {"mul": 0, "add": 1}[op]
    Apos, Acrd = _dev(Apos, torch.int32, "Apos"), _dev(Acrd, torch.int32, "Acrd")
    Bpos, Bcrd = _dev(Bpos, torch.int32, "Bpos"), _dev(Bcrd, torch.int32, "Bcrd")
    code = _DTYPE_CODE.get(Aval.dtype)
    if code is None or Bval.dtype != Aval.dtype:
        raise TypeError("element-wise operands must share one of f32/f64/i32/i64")
    Aval, Bval = _dev(Aval, Aval.dtype, "Aval"), _dev(Bval, Aval.dtype, "Bval")
    m = Apos.numel() - 1
    if Bpos.numel() - 1 != m:
        raise ValueError("operands differ in row count")
    L = _lib.lib()
    dev = Aval.device
    with torch.cuda.device(dev):
        wbytes = L.sb_csr_ewise_workspace_bytes(m)
        ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        Cpos = torch.empty(m + 1, dtype=torch.int32, device=dev)
        total = C.c_int64(0)
        check(L.sb_csr_ewise_symbolic(code_op, m, Apos.data_ptr(), Acrd.data_ptr(), Bpos.data_ptr(),
                                      Bcrd.data_ptr(), Cpos.data_ptr(), C.byref(total), ws.data_ptr(), wbytes,
                                      _stream()))
        Ccrd = torch.empty(total.value, dtype=torch.int32, device=dev)
        Cval = torch.empty(total.value, dtype=Aval.dtype, device=dev)
        check(L.sb_csr_ewise_numeric(code_op, code, m, Apos.data_ptr(), Acrd.data_ptr(), Aval.data_ptr(),
                                     Bpos.data_ptr(), Bcrd.data_ptr(), Bval.data_ptr(), Cpos.data_ptr(),
                                     Ccrd.data_ptr(), Cval.data_ptr(), _stream()))
    return Cpos, Ccrd, Cval
