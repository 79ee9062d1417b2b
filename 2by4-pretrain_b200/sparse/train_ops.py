"""Layer normalisation (alone, or with the residual add in front of it), cross entropy and the token + position
embedding of the trainer as streaming CUDA kernels (``sp24_layernorm_*``, ``sp24_add_layernorm_*``,
``sp24_cross_entropy_*``, ``sp24_embedding_*``).  None of them is part of the reference package (its model and training
scripts live in another repository); they stand where the framework's generic kernels dominated a step of the GPT-2
configuration: the float32 layer norm followed by a cast to the GEMM's 16-bit operand type, its gamma / beta gradient
kernel, the residual adds and gradient accumulations around it, the float32 copies of the (tokens x vocabulary) logits
around log-softmax, and the sort-based embedding gradient."""
import torch
from torch import autograd, nn

from . import _ext


def _affine_grad_targets(weight, bias, into_grad, d, device):
    """Where the backward kernel adds the gamma / beta gradients: straight into ``weight.grad`` / ``bias.grad`` when
    asked to and both exist as contiguous float32 buffers (autograd then receives None for them: no temporaries, no
    accumulation launches), else into a zeroed temporary that is returned through autograd."""
    if into_grad:
        gw, gb = weight.grad, bias.grad
        if gw is not None and gb is not None and gw.dtype == gb.dtype == torch.float32 and gw.is_contiguous() \
                and gb.is_contiguous():
            return gw, gb, None, None
    dgb = torch.zeros((2, d), dtype=torch.float32, device=device)
    return dgb[0], dgb[1], dgb[0], dgb[1]


class _layer_norm(autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype, into_grad=False):
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
        ctx.save_for_backward(x2, mean, rstd)
        ctx.shape, ctx.x_dtype = x.shape, x.dtype
        ctx.weight, ctx.bias, ctx.into_grad = weight, bias, into_grad
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, grad_output):
        x2, mean, rstd = ctx.saved_tensors
        weight = ctx.weight
        rows, d = x2.shape
        dy = grad_output.reshape(rows, d)
        if dy.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            dy = dy.float()
        dy = dy.contiguous()
        dx = torch.empty_like(x2)
        tg, tb, rg, rb = _affine_grad_targets(weight, ctx.bias, ctx.into_grad, d, x2.device)
        rc = _ext.lib().sp24_layernorm_bwd(dy.data_ptr(), _ext.dt(dy.dtype), x2.data_ptr(), weight.data_ptr(), mean.data_ptr(),
                                           rstd.data_ptr(), dx.data_ptr(), tg.data_ptr(), tb.data_ptr(), rows, d, _ext.stream())
        _ext.check(rc, "sp24_layernorm_bwd")
        return dx.view(ctx.shape).to(ctx.x_dtype), rg, rb, None, None, None


class _add_layer_norm(autograd.Function):
    """(x + delta, layer_norm(x + delta)) in one pass; the backward pass adds the gradient arriving along the residual
    stream to the norm's input gradient and hands the sum to both inputs (float32 for x, delta's dtype for delta)."""

    @staticmethod
    def forward(ctx, x, delta, weight, bias, eps, into_grad=False):
        d = x.shape[-1]
        x2, dl = x.reshape(-1, d), delta.reshape(-1, d)
        rows = x2.shape[0]
        res = torch.empty((rows, d), dtype=torch.float32, device=x.device)
        out = torch.empty((rows, d), dtype=delta.dtype, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _ext.lib().sp24_add_layernorm_fwd(x2.data_ptr(), dl.data_ptr(), res.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                               out.data_ptr(), _ext.dt(out.dtype), mean.data_ptr(), rstd.data_ptr(), rows, d,
                                               float(eps), _ext.stream())
        _ext.check(rc, "sp24_add_layernorm_fwd")
        ctx.save_for_backward(res, mean, rstd)
        ctx.shape, ctx.delta_dtype = x.shape, delta.dtype
        ctx.weight, ctx.bias, ctx.into_grad = weight, bias, into_grad
        return res.view(x.shape), out.view(x.shape)

    @staticmethod
    def backward(ctx, grad_res, grad_out):
        res, mean, rstd = ctx.saved_tensors
        weight = ctx.weight
        rows, d = res.shape
        if grad_out is None:                          # the normalised output was not used: only the residual path
            return grad_res, grad_res.to(ctx.delta_dtype), None, None, None, None
        dy = grad_out.reshape(rows, d).contiguous()
        dres = None
        if grad_res is not None:
            dres = grad_res.reshape(rows, d)
            if dres.dtype != torch.float32 or not dres.is_contiguous():
                dres = dres.float().contiguous()
        dx = torch.empty_like(res)
        ddelta = torch.empty((rows, d), dtype=dy.dtype, device=res.device)
        tg, tb, rg, rb = _affine_grad_targets(weight, ctx.bias, ctx.into_grad, d, res.device)
        rc = _ext.lib().sp24_add_layernorm_bwd(dy.data_ptr(), _ext.dt(dy.dtype), _ext.ptr(dres), res.data_ptr(), weight.data_ptr(),
                                               mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), ddelta.data_ptr(),
                                               tg.data_ptr(), tb.data_ptr(), rows, d, _ext.stream())
        _ext.check(rc, "sp24_add_layernorm_bwd")
        return dx.view(ctx.shape), ddelta.view(ctx.shape), rg, rb, None, None


def add_layer_norm(x: torch.Tensor, delta: torch.Tensor, norm: nn.LayerNorm):
    """The residual connection in front of a pre-norm block and the block's norm as one kernel each way:
    returns ``(x + delta, norm(x + delta))``.  ``x``: the float32 residual stream; ``delta``: the branch output that
    joins it (the attention or MLP output), in the dtype the next linear layer consumes; the normalised output comes
    back in that dtype.  Anything the kernel does not cover (other dtypes, d % 128 != 0, d > 1024, no affine
    parameters) runs as the two separate ops."""
    d = x.shape[-1]
    ok = (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous() and delta.shape == x.shape
          and delta.dtype in (torch.float16, torch.bfloat16, torch.float32)
          and isinstance(norm, nn.LayerNorm) and norm.elementwise_affine and norm.bias is not None
          and len(norm.normalized_shape) == 1 and d % 128 == 0 and d <= 1024 and norm.weight.dtype == torch.float32)
    if ok:
        want = torch.get_autocast_dtype('cuda') if torch.is_autocast_enabled('cuda') else torch.float32
        ok = delta.dtype == want
    if not ok:
        res = x + delta
        return res, norm(res)
    _ext.require_cuda(x, delta, norm.weight, norm.bias)
    return _add_layer_norm.apply(x, delta, norm.weight, norm.bias, norm.eps, bool(getattr(norm, "accumulate_into_grad", False)))


class LayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` over the last dimension (float32 parameters and input, d % 128 == 0, d <= 1024) on the library's
    kernels.  Under CUDA autocast the output is written in the autocast dtype, i.e. as the operand of the linear
    layer that follows, instead of float32 plus a cast; otherwise float32.  Other inputs fall back to the parent.
    ``accumulate_into_grad``: the backward kernel adds the gamma / beta gradients straight into existing float32
    ``weight.grad`` / ``bias.grad`` buffers (trainers that keep gradients in one flat buffer), autograd gets None."""

    accumulate_into_grad = False

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
        return _layer_norm.apply(x, self.weight, self.bias, self.eps, out_dtype, self.accumulate_into_grad)


class _cross_entropy(autograd.Function):
    """Two launches (forward, backward), each reading the logits once."""

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


class _cross_entropy_fused(autograd.Function):
    """One launch: the forward pass also writes the gradient for an upstream gradient of 1 (what ``loss.backward()``
    supplies), from the same read of each row; the backward pass multiplies it by the upstream gradient on the device
    only when that is not 1."""

    @staticmethod
    def forward(ctx, logits, targets):
        rows, v = logits.shape
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        dlogits = torch.empty((rows, v), dtype=logits.dtype, device=logits.device)
        rc = _ext.lib().sp24_cross_entropy_fused(logits.data_ptr(), _ext.dt(logits.dtype), targets.data_ptr(), lse.data_ptr(),
                                                 loss.data_ptr(), 1.0 / rows, dlogits.data_ptr(), rows, v, logits.stride(0), v,
                                                 _ext.stream())
        _ext.check(rc, "sp24_cross_entropy_fused")
        ctx.save_for_backward(dlogits)
        return loss.mean()

    @staticmethod
    def backward(ctx, grad_output):
        (dlogits,) = ctx.saved_tensors
        if getattr(ctx, "consumed", False):
            raise RuntimeError("cross_entropy: the fused gradient buffer was already handed out by an earlier backward pass")
        ctx.consumed = True
        up = grad_output.reshape(1).float().contiguous()
        rc = _ext.lib().sp24_scale_unless_one(dlogits.data_ptr(), _ext.dt(dlogits.dtype), up.data_ptr(), dlogits.numel(),
                                              _ext.stream())
        _ext.check(rc, "sp24_scale_unless_one")
        return dlogits, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, fused: bool = True) -> torch.Tensor:
    """Mean cross entropy of 16-bit ``logits`` (rows, classes) against int64 class ``targets`` (rows), computed in
    float32 from one read of the logits; the gradient comes back in the logits' dtype.  Same value as
    ``F.cross_entropy(logits.float(), targets)`` up to float32 summation order, without the float32 copy of the logits.
    No ``ignore_index``, no label smoothing, no class weights.  ``fused`` (when a gradient is wanted): the forward launch
    also writes the gradient for an upstream gradient of 1, from the same read of each row; the backward pass rescales it
    on the device only if the upstream gradient is not 1.  ``fused=False``: one launch per direction."""
    _ext.require_cuda(logits, targets)
    if logits.dim() != 2 or logits.dtype not in (torch.float16, torch.bfloat16) or logits.shape[1] % 8 or logits.stride(1) != 1 \
            or logits.stride(0) % 8 or logits.data_ptr() % 16:
        raise RuntimeError("cross_entropy: expected 16-bit logits (rows, classes), classes % 8 == 0, unit inner stride")
    if targets.dtype != torch.int64 or targets.numel() != logits.shape[0]:
        raise RuntimeError("cross_entropy: expected one int64 target per row")
    targets = targets.reshape(-1).contiguous()
    if fused and logits.requires_grad and torch.is_grad_enabled():
        return _cross_entropy_fused.apply(logits, targets)
    return _cross_entropy.apply(logits, targets)


class _embed_tokens(autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, wpe, into_grad):
        b, t = ids.shape
        vocab, d = wte.shape
        ids = ids.contiguous()
        out = torch.empty((b, t, d), dtype=torch.float32, device=wte.device)
        rc = _ext.lib().sp24_embedding_fwd(ids.data_ptr(), wte.data_ptr(), wpe.data_ptr(), out.data_ptr(), b * t, t, d, vocab,
                                           _ext.stream())
        _ext.check(rc, "sp24_embedding_fwd")
        ctx.save_for_backward(ids)
        ctx.wte, ctx.wpe, ctx.into_grad = wte, wpe, into_grad
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (ids,) = ctx.saved_tensors
        wte, wpe = ctx.wte, ctx.wpe
        b, t = ids.shape
        vocab, d = wte.shape
        dx = grad_output
        if dx.dtype != torch.float32 or not dx.is_contiguous():
            dx = dx.float().contiguous()
        gw, gp = wte.grad, wpe.grad
        into = ctx.into_grad and gw is not None and gp is not None and gw.dtype == gp.dtype == torch.float32 \
            and gw.is_contiguous() and gp.is_contiguous()
        if not into:
            gw, gp = torch.zeros_like(wte, dtype=torch.float32), torch.zeros_like(wpe, dtype=torch.float32)
        rc = _ext.lib().sp24_embedding_bwd(dx.data_ptr(), ids.data_ptr(), gw.data_ptr(), gp.data_ptr(), b * t, t, d, vocab,
                                           _ext.stream())
        _ext.check(rc, "sp24_embedding_bwd")
        if into:
            return None, None, None, None
        return None, gw, gp, None


def embed_tokens(ids: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor, into_grad: bool = False) -> torch.Tensor:
    """``wte[ids] + wpe[arange(t)]`` for int64 ``ids`` (batch, t): the token and learned position embeddings of a
    decoder as one gather kernel, float32 (batch, t, d).  The backward pass adds each token's gradient row to its two
    table rows with float32 vector reductions (one launch instead of the sort-based embedding gradient); with
    ``into_grad`` and float32 ``.grad`` buffers in place it adds straight into them and autograd receives None.
    The summation order over tokens that share a row is not fixed (last-bit differences between runs)."""
    _ext.require_cuda(ids, wte, wpe)
    if ids.dim() != 2 or ids.dtype != torch.int64:
        raise RuntimeError("embed_tokens: expected int64 ids of shape (batch, t)")
    if wte.dim() != 2 or wpe.dim() != 2 or wte.shape[1] != wpe.shape[1] or wte.shape[1] % 4 or wte.dtype != torch.float32 \
            or wpe.dtype != torch.float32 or not wte.is_contiguous() or not wpe.is_contiguous():
        raise RuntimeError("embed_tokens: expected contiguous float32 tables of equal width, width % 4 == 0")
    if ids.shape[1] > wpe.shape[0]:
        raise RuntimeError(f"embed_tokens: {ids.shape[1]} positions, the position table holds {wpe.shape[0]}")
    return _embed_tokens.apply(ids, wte, wpe, into_grad)


class _gelu(autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        out = torch.empty_like(x)
        rc = _ext.lib().sp24_gelu(x.data_ptr(), None, out.data_ptr(), _ext.dt(x.dtype), x.numel(), _ext.stream())
        _ext.check(rc, "sp24_gelu")
        ctx.save_for_backward(x)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (x,) = ctx.saved_tensors
        dy = grad_output.contiguous()
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        out = torch.empty_like(x)
        rc = _ext.lib().sp24_gelu(x.data_ptr(), dy.data_ptr(), out.data_ptr(), _ext.dt(x.dtype), x.numel(), _ext.stream())
        _ext.check(rc, "sp24_gelu")
        return out


def gelu(x: torch.Tensor) -> torch.Tensor:
    """``F.gelu(x, approximate="tanh")`` for 16-bit CUDA tensors with a multiple of 8 elements on the library's streaming
    kernel (float32 arithmetic, ``tanh.approx``: the formula of the GEMM epilogues); anything else goes to torch."""
    if not (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and x.numel() % 8 == 0 and x.numel() > 0):
        return torch.nn.functional.gelu(x, approximate="tanh")
    _ext.require_cuda(x)
    return _gelu.apply(x)
