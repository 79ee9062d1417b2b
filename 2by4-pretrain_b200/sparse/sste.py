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


class _soft_threshold_spmm_linear(autograd.Function):
    """Forward on the sparse tensor cores; both gradients are dense GEMMs (the soft-threshold mask is
    not transposable, so W_s^T has no 2:4 structure along its rows)."""

    @staticmethod
    def forward(ctx, x, weight, bias, scale, dtype):
        from .semi_structured import to_sparse_semi_structured
        from .spmm import sparse_linear
        w_s, mask = soft_threshold24_triton(weight.detach(), scale=scale)
        w_s = w_s.to(dtype)
        comp = to_sparse_semi_structured(w_s, mask=mask != 0, dtype=dtype)
        x2 = x.reshape(-1, x.shape[-1]).to(dtype)
        b = None if bias is None else bias.to(dtype)
        y = sparse_linear(x2, comp.sparse_tensor_cutlass, comp.meta_tensor_cutlass, bias=b)
        ctx.save_for_backward(x2, w_s)
        ctx.shape = x.shape
        ctx.has_bias = bias is not None
        return y.view(*x.shape[:-1], -1)

    @staticmethod
    def backward(ctx, grad_output):
        x2, w_s = ctx.saved_tensors
        g = grad_output.reshape(-1, grad_output.shape[-1]).to(w_s.dtype)
        grad_x = grad_w = grad_b = None
        if ctx.needs_input_grad[0]:
            grad_x = torch.mm(g, w_s).view(ctx.shape)
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
