"""Layer normalisation and cross entropy of the trainer as streaming CUDA kernels (``sp24_layernorm_fwd / _bwd``,
``sp24_cross_entropy_fwd / _bwd``).  Neither op is part of the reference package (its model and training scripts live
in another repository); they stand where the framework's generic kernels dominated a step of the GPT-2 configuration:
the float32 layer norm followed by a cast to the GEMM's 16-bit operand type, its gamma / beta gradient kernel, and the
float32 copies of the (tokens x vocabulary) logits around log-softmax."""
import torch
from torch import autograd, nn

from . import _ext


class _layer_norm(autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if x2.dtype != torch.float32:
            x2 = x2.float()
        x2 = x2.contiguous()
        rows = x2.shape[0]
        out = torch.empty((rows, d), dtype=out_dtype, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _ext.lib().sp24_layernorm_fwd(x2.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(), _ext.dt(out_dtype),
                                           mean.data_ptr(), rstd.data_ptr(), rows, d, float(eps), _ext.stream())
        _ext.check(rc, "sp24_layernorm_fwd")
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape, ctx.x_dtype = x.shape, x.dtype
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, grad_output):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy = grad_output.reshape(rows, d)
        if dy.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            dy = dy.float()
        dy = dy.contiguous()
        dx = torch.empty_like(x2)
        dgb = torch.zeros((2, d), dtype=torch.float32, device=x2.device)
        rc = _ext.lib().sp24_layernorm_bwd(dy.data_ptr(), _ext.dt(dy.dtype), x2.data_ptr(), weight.data_ptr(), mean.data_ptr(),
                                           rstd.data_ptr(), dx.data_ptr(), dgb[0].data_ptr(), dgb[1].data_ptr(), rows, d,
                                           _ext.stream())
        _ext.check(rc, "sp24_layernorm_bwd")
        return dx.view(ctx.shape).to(ctx.x_dtype), dgb[0], dgb[1], None, None


class LayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` over the last dimension (float32 parameters and input, d % 128 == 0, d <= 1024) on the library's
    kernels.  Under CUDA autocast the output is written in the autocast dtype, i.e. as the operand of the linear
    layer that follows, instead of float32 plus a cast; otherwise float32.  Other inputs fall back to the parent."""

    def forward(self, x):
        d = x.shape[-1]
        ok = (x.is_cuda and self.elementwise_affine and self.bias is not None and len(self.normalized_shape) == 1
              and d % 128 == 0 and d <= 1024 and self.weight.dtype == torch.float32)
        if not ok:
            return super().forward(x)
        _ext.require_cuda(x, self.weight, self.bias)
        out_dtype = torch.get_autocast_dtype('cuda') if torch.is_autocast_enabled('cuda') else torch.float32
        if out_dtype not in (torch.float16, torch.bfloat16, torch.float32):
            out_dtype = torch.float32
        return _layer_norm.apply(x, self.weight, self.bias, self.eps, out_dtype)


class _cross_entropy(autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        rows, v = logits.shape
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        rc = _ext.lib().sp24_cross_entropy_fwd(logits.data_ptr(), _ext.dt(logits.dtype), targets.data_ptr(), lse.data_ptr(),
                                               loss.data_ptr(), rows, v, logits.stride(0), _ext.stream())
        _ext.check(rc, "sp24_cross_entropy_fwd")
        ctx.save_for_backward(logits, targets, lse)
        return loss.mean()

    @staticmethod
    def backward(ctx, grad_output):
        logits, targets, lse = ctx.saved_tensors
        rows, v = logits.shape
        up = grad_output.reshape(1).float().contiguous()
        dlogits = torch.empty((rows, v), dtype=logits.dtype, device=logits.device)
        rc = _ext.lib().sp24_cross_entropy_bwd(logits.data_ptr(), _ext.dt(logits.dtype), targets.data_ptr(), lse.data_ptr(),
                                               up.data_ptr(), 1.0 / rows, dlogits.data_ptr(), rows, v, logits.stride(0), v,
                                               _ext.stream())
        _ext.check(rc, "sp24_cross_entropy_bwd")
        return dlogits, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross entropy of 16-bit ``logits`` (rows, classes) against int64 class ``targets`` (rows), computed in
    float32 from one read of the logits; the gradient comes back in the logits' dtype.  Same value as
    ``F.cross_entropy(logits.float(), targets)`` up to float32 summation order, without the float32 copy of the logits.
    No ``ignore_index``, no label smoothing, no class weights."""
    _ext.require_cuda(logits, targets)
    if logits.dim() != 2 or logits.dtype not in (torch.float16, torch.bfloat16) or logits.shape[1] % 8 or logits.stride(1) != 1 \
            or logits.stride(0) % 8 or logits.data_ptr() % 16:
        raise RuntimeError("cross_entropy: expected 16-bit logits (rows, classes), classes % 8 == 0, unit inner stride")
    if targets.dtype != torch.int64 or targets.numel() != logits.shape[0]:
        raise RuntimeError("cross_entropy: expected one int64 target per row")
    return _cross_entropy.apply(logits, targets.reshape(-1).contiguous())
