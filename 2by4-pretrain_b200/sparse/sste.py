"""S-STE training layer: continuous 2:4 pruning by soft thresholding with a frozen per-tensor scale.

The reference lists these classes only in its README (README.md:233-267 of the reference); here they are
real.  ``SoftThreshold`` prunes with ``soft_threshold24_triton`` and passes the gradient straight
through; ``SoftThresholdLinear`` is the ``nn.Linear`` replacement (the README calls it ``SparseLinear``,
a name the package already uses for the MVUE layer of sparse/sparse_ops.py:86-87).  The scale is folded
into the pruning kernel's store, and with ``spmm=True`` the forward GEMM runs on the 2:4 sparse tensor
cores from a compressed copy of the pruned weight.
"""
import torch
import torch.nn.functional as F
from torch import autograd, nn

from .triton_ops import soft_threshold24_triton


class SoftThreshold(autograd.Function):
    """weight -> soft_threshold24(weight) * scale; d/dweight = identity (straight-through)."""

    @staticmethod
    def forward(ctx, weight, scale):
        s = float(scale) if not isinstance(scale, float) else scale
        sparse, _ = soft_threshold24_triton(weight.detach(), scale=s)
        return sparse

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


def soft_threshold24_compress(weight: torch.Tensor, scale=None, dtype: torch.dtype = torch.float16):
    """One pass over ``weight``: S-STE soft threshold (times ``scale`` if given) and 2:4 compression to ``dtype``.
    Returns (packed (m, k/2), reordered metadata (m, k/16) int16), the operands of ``sparse_linear``; the
    tensor-core order of the metadata is written by the same kernel when m is a multiple of 128.  Bit-identical to
    ``soft_threshold24_triton(weight, scale=scale)``, a cast and ``to_sparse_semi_structured(..., mask=mask)``."""
    from . import _ext, spmm as _spmm
    _ext.require_cuda(weight)
    if weight.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {weight.dim()}-dimensional tensor")
    if dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"soft_threshold24_compress: packed dtype must be float16 or bfloat16, got {dtype}")
    m, k = weight.shape
    if m % 32 or k % 64:
        raise RuntimeError(f"soft_threshold24_compress: shape {(m, k)}: rows % 32 == 0 and columns % 64 == 0 required")
    w = _ext.as_layout(weight.detach(), 0)
    buf = torch.empty(m * k * 9 // 16, dtype=dtype, device=w.device)
    packed = buf[: m * k // 2].view(m, k // 2)
    meta = buf[m * k // 2:].view(torch.int16).view(m, k // 16)
    e_tc = torch.empty(_spmm.tc_bytes(m, k), dtype=torch.uint8, device=w.device) if m % 128 == 0 else None
    rc = _ext.lib().sp24_soft_threshold24_compress(w.data_ptr(), _ext.dt(w.dtype), m, k, _ext.layout_of(w)[1], 0,
                                                   packed.data_ptr(), _ext.dt(dtype), k // 2, meta.data_ptr(),
                                                   0 if scale is None else 1, 0.0 if scale is None else float(scale),
                                                   _ext.ptr(e_tc), _ext.stream())
    _ext.check(rc, "sp24_soft_threshold24_compress")
    if e_tc is not None:
        _spmm.register_tc_metadata(meta, e_tc)
    return packed, meta


class _soft_threshold_spmm_linear(autograd.Function):
    """Forward on the sparse tensor cores from a copy of the weight that one kernel soft-thresholds, scales and
    compresses.  Both gradients are dense GEMMs by construction: the soft-threshold mask is 2:4 along the rows of W
    only, so W_s^T has no 2:4 structure along its rows and the input gradient dY W_s has no sparse-tensor-core form;
    the weight gradient is the straight-through dense dY^T X of the recipe (README.md:233-267 of the reference)."""

    @staticmethod
    def forward(ctx, x, weight, bias, scale, dtype):
        from .spmm import sparse_linear
        packed, meta = soft_threshold24_compress(weight, scale=scale, dtype=dtype)
        x2 = x.reshape(-1, x.shape[-1]).to(dtype)
        b = None if bias is None else bias.to(dtype)
        y = sparse_linear(x2, packed, meta, bias=b)
        ctx.save_for_backward(x2, packed, meta)
        ctx.shape = x.shape
        ctx.has_bias = bias is not None
        return y.view(*x.shape[:-1], -1)

    @staticmethod
    def backward(ctx, grad_output):
        from ._semi_structured_conversions import sparse_semi_structured_to_dense
        x2, packed, meta = ctx.saved_tensors
        g = grad_output.reshape(-1, grad_output.shape[-1]).to(packed.dtype)
        grad_x = grad_w = grad_b = None
        if ctx.needs_input_grad[0]:
            grad_x = torch.mm(g, sparse_semi_structured_to_dense(packed, meta)).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            grad_w = torch.mm(g.t(), x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = g.sum(0)
        return grad_x, grad_w, grad_b, None, None


class SoftThresholdLinear(nn.Linear):
    """``nn.Linear`` whose weight passes through the S-STE pruning function on every forward.

    ``init_scale()`` freezes ``scale = <w, S(w)> / <S(w), S(w)>`` (S = soft threshold) once, before
    training, as in the README listing; the value is kept as a buffer (checkpointed) and as a Python
    float so that the forward pass needs no device-to-host read.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 spmm: bool = False, spmm_dtype: torch.dtype = torch.float16):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.register_buffer('scale', torch.tensor(0.))
        self._scale_value = None
        self.spmm = spmm
        self.spmm_dtype = spmm_dtype

    def _scale(self) -> float:
        if self._scale_value is None:      # e.g. after load_state_dict
            self._scale_value = float(self.scale)
        return self._scale_value

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self._scale_value = None

    def get_sparse_weights(self):
        return SoftThreshold.apply(self.weight, self._scale())

    @torch.no_grad()
    def init_scale(self):
        weight = self.weight.detach()
        weight_sparse, _ = soft_threshold24_triton(weight)
        w, ws = weight.flatten().float(), weight_sparse.flatten().float()
        value = torch.dot(w, ws) / torch.dot(ws, ws)
        self.scale.copy_(value)
        self._scale_value = float(value)
        self.weight.scale = self.scale

    def forward(self, x):
        if self.spmm:
            return _soft_threshold_spmm_linear.apply(x, self.weight, self.bias, self._scale(), self.spmm_dtype)
        return F.linear(x, self.get_sparse_weights(), self.bias)
