"""Float8 (e4m3, per-tensor scales) form of the FST layer: forward, input gradient and weight gradient as 2:4 sparse
GEMMs on 8-bit operands.

The reference cannot run its backward pass in float8: its 8-bit GEMMs take a row-major sparse operand only
(sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:735-738, :778-781 of the reference), while its conversion of a
transposed view (``W.T``, ``grad_output.t()``) writes column-major packed values, and its MVUE branch for 8-bit
outputs is incomplete (sparse/_semi_structured_conversions.py:822-839).  Here the conversion kernel writes the
K-major (row-major) packed operand straight from the transposed view (``sp24_prune_compress_q8``), so all three GEMMs
of ``sparse_linear_transpose`` (README.md:169-200 of the reference) run on the float8 tensor-core path:

    Y  = (Xq  Wq_s^T)            * (sx * sw)        Xq  = X / sx,  Wq = W / sw   (e4m3)
    dX = (dYq Wq_s)              * (sg * sw)        dYq = dY / sg
    dW = (MVUE24(dY^T)/sg  Xq)   * (sg * sx)        MVUE drawn on the 16-bit gradient, quantised on store

The dequantisation scales are applied in the GEMM epilogue (``sp24_spmm_scaled``).  Scales are per tensor, ``amax / 448``, read back to the host (one synchronisation per quantised tensor): the layer is
a functional reference of the float8 recipe, not a tuned training loop.
"""
import random
from typing import Optional

import torch
from torch import autograd

from . import _ext
from .spmm import sparse_linear as _spmm

E4M3 = torch.float8_e4m3fn
E4M3_MAX = 448.0


def scale_of(t: torch.Tensor) -> float:
    """Per-tensor dequantisation scale: amax / 448 (1 for an all-zero tensor)."""
    a = float(t.detach().abs().amax())
    return a / E4M3_MAX if a > 0 else 1.0


def quantize(t: torch.Tensor, scale: Optional[float] = None):
    """(t / scale) rounded to e4m3, and the scale."""
    s = scale_of(t) if scale is None else float(scale)
    return (t.float() / s).to(E4M3), s


def compress_q8(dense: torch.Tensor, *, mode: int, mask: Optional[torch.Tensor] = None, scale: float = 1.0,
                seed: int = 0, offset: int = 0, dtype: torch.dtype = E4M3):
    """2:4 compression of the logical (m, k) matrix ``dense`` (row-major, or a transposed view of a row-major
    tensor) to float8: returns (packed (m, k/2) ROW-major, metadata (m, k/32) int32).  Stored values are
    ``value / scale``.  ``mode``: ``_ext.PRUNE_MSE`` / ``PRUNE_MASK`` (with ``mask``, same shape) /
    ``PRUNE_MVUE`` / ``PRUNE_MVUE_FAST`` (seeded by ``seed``, ``offset``)."""
    _ext.require_cuda(dense, mask)
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    if dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise RuntimeError(f"compress_q8: float8 output types only, got {dtype}")
    m, k = dense.shape
    if m % 32 or k % 128:
        raise RuntimeError(f"compress_q8: shape {(m, k)}: rows % 32 == 0 and columns % 128 == 0 required")
    lay = _ext.layout_of(dense)
    if lay is None or dense.data_ptr() % 16 or (lay[1] * dense.element_size()) % 16:
        dense = dense.contiguous()
        lay = (0, k)
    col_major, ld_d = lay
    ld_m = 0
    if mask is not None:
        if mask.dtype not in (torch.bool, torch.uint8):
            mask = mask != 0
        mask = _ext.as_layout(mask, col_major)
        ld_m = _ext.layout_of(mask)[1]
    packed = torch.empty((m, k // 2), dtype=dtype, device=dense.device)
    meta = torch.empty((m, k // 32), dtype=torch.int32, device=dense.device)
    rc = _ext.lib().sp24_prune_compress_q8(dense.data_ptr(), _ext.dt(dense.dtype), m, k, ld_d, col_major, packed.data_ptr(),
                                           _ext.dt(dtype), k // 2, meta.data_ptr(), mode, _ext.ptr(mask), ld_m,
                                           1.0 / float(scale), seed & (2 ** 64 - 1), offset & (2 ** 64 - 1), _ext.stream())
    _ext.check(rc, "sp24_prune_compress_q8")
    return packed, meta


class Fp8SparseWeight:
    """W (out_features, in_features) under a transposable 2:4 mask, compressed twice in e4m3 with one scale:
    ``pw, mw`` = W for the forward GEMM, ``pt, mt`` = W^T (K-major, from the transposed view) for the input
    gradient."""

    def __init__(self, weight: torch.Tensor, mask: torch.Tensor):
        w = weight.detach()
        self.scale = scale_of(torch.where(mask, w, torch.zeros((), dtype=w.dtype, device=w.device)))
        self.pw, self.mw = compress_q8(w, mode=_ext.PRUNE_MASK, mask=mask, scale=self.scale)
        self.pt, self.mt = compress_q8(w.t(), mode=_ext.PRUNE_MASK, mask=mask.t(), scale=self.scale)
        self.shape = tuple(w.shape)


def fst_fp8_forward(xq: torch.Tensor, sx: float, w8: Fp8SparseWeight, bias: Optional[torch.Tensor] = None):
    """Y (tokens, out_features) fp32 = dequantised Xq W_s^T (+ bias)."""
    return _spmm(xq, w8.pw, w8.mw, bias=None if bias is None else bias.float().contiguous(), alpha=sx * w8.scale)


def fst_fp8_input_grad(gq: torch.Tensor, sg: float, w8: Fp8SparseWeight):
    """dX (tokens, in_features) fp32 = dequantised dYq W_s, through the K-major compressed W^T."""
    return _spmm(gq, w8.pt, w8.mt, alpha=sg * w8.scale)


def fst_fp8_weight_grad(g: torch.Tensor, sg: float, xq_t: torch.Tensor, sx: float, seed: Optional[int] = None,
                        fast: bool = True):
    """dW (out_features, in_features) fp32 = MVUE24(dY^T) X.  ``g``: the 16-bit / fp32 gradient (tokens,
    out_features); the MVUE draw runs on it and the kept values are stored as e4m3 of ``value / sg``.
    ``xq_t``: Xq^T (in_features, tokens) contiguous e4m3 (the dense operand must be K-major for 8-bit types)."""
    if seed is None:
        seed = random.randint(0, 2 ** 31 - 1)
    mode = _ext.PRUNE_MVUE_FAST if fast else _ext.PRUNE_MVUE
    pg, mg = compress_q8(g.t(), mode=mode, scale=sg, seed=seed)                   # (out_features, tokens / 2)
    return _spmm(xq_t, pg, mg, alpha=sg * sx).t()


class sparse_linear_transpose_fp8(autograd.Function):
    """``sparse_linear_transpose`` (README.md:169-200 of the reference) with every GEMM in e4m3.  ``weight`` only
    routes the gradient; ``w8`` is its compressed form (``Fp8SparseWeight``)."""

    @staticmethod
    def forward(ctx, input, weight, w8, bias):
        x = input.reshape(-1, input.shape[-1])
        xq, sx = quantize(x)
        ctx.save_for_backward(xq.t().contiguous())
        ctx.sx, ctx.w8, ctx.shape, ctx.has_bias, ctx.dtype = sx, w8, input.shape, bias is not None, input.dtype
        y = fst_fp8_forward(xq, sx, w8, bias)
        return y.to(input.dtype).view(*input.shape[:-1], -1)

    @staticmethod
    def backward(ctx, grad_output):
        (xq_t,) = ctx.saved_tensors
        g = grad_output.reshape(-1, grad_output.shape[-1])
        if g.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            g = g.float()
        g = g.contiguous()
        sg = scale_of(g)
        grad_input = grad_weight = grad_bias = None
        if ctx.needs_input_grad[0]:
            gq, _ = quantize(g, sg)
            grad_input = fst_fp8_input_grad(gq, sg, ctx.w8).to(ctx.dtype).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            grad_weight = fst_fp8_weight_grad(g, sg, xq_t, ctx.sx)
        if ctx.has_bias and ctx.needs_input_grad[3]:
            grad_bias = g.sum(0)
        return grad_input, grad_weight, None, grad_bias
