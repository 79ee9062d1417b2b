"""Autograd linear layers of the 2:4 training recipes.

``SparseLinearTranspose`` / ``sparse_linear_transpose`` are the FST layer the reference only lists in
its README (README.md:125-200 of the reference): forward Y = X W_s^T with the weight compressed under
a transposable 2:4 mask, backward dX = dY W_s through the separately compressed W^T, and
dW = MVUE24(dY^T) X with the gradient compressed on the fly.  ``MyLinear`` / ``SparseLinear`` are the
older dense-GEMM variants of sparse/sparse_ops.py:8-87 of the reference.
"""
import random

import torch
import torch.nn.functional as F
from torch import autograd, nn
from torch.amp import custom_fwd, custom_bwd

from . import _ext
from ._semi_structured_conversions import prune_compress
from .semi_structured import SparseSemiStructuredTensor, to_sparse_semi_structured
from .transposable_semi_structured import TransposableSparse, select_and_compress
from .triton_ops import MVUE24_approx_triton
from .spmm import sparse_linear as _spmm, sparse_mm_accumulate_ as _spmm_acc, sparse_linear_mlp as _spmm_mlp, mlp_fusable


def _dense_linear(name, dx_weight, doc):
    """Builds the autograd function of a dense linear layer, y = x W^T (+ b), whose input gradient is
    dY @ ``dx_weight(W)``.  The two dense layers of the reference differ only in that factor
    (sparse/sparse_ops.py:8-87 of the reference): W itself, or a fresh MVUE 2:4 estimate of it."""

    def forward(ctx, input, weight, bias):
        ctx.save_for_backward(input, weight)
        ctx.lead = input.shape[:-1]
        y = input.reshape(-1, input.shape[-1]).mm(weight.t()).view(*ctx.lead, weight.shape[0])
        return y if bias is None else y + bias

    def backward(ctx, grad_output):
        input, weight = ctx.saved_tensors
        want_x, want_w, want_b = ctx.needs_input_grad
        g = grad_output.reshape(-1, weight.shape[0])
        gx = g.mm(dx_weight(weight)).view(*ctx.lead, weight.shape[1]) if want_x else None
        gw = g.t().mm(input.reshape(-1, weight.shape[1])) if want_w else None
        gb = g.sum(0) if want_b else None
        return gx, gw, gb

    return type(name, (autograd.Function,), {
        "__doc__": doc,
        "forward": staticmethod(custom_fwd(device_type='cuda')(forward)),
        "backward": staticmethod(custom_bwd(device_type='cuda')(backward)),
    })


my_linear = _dense_linear("my_linear", lambda w: w, "Plain dense linear layer as a custom autograd function.")
sparse_linear = _dense_linear(
    "sparse_linear", lambda w: MVUE24_approx_triton(w.t()).t(),
    "Dense GEMMs; the input gradient multiplies dY with an MVUE 2:4 estimate of the weight, drawn along its "
    "output-feature axis on every backward pass.")


class MyLinear(nn.Linear):
    def forward(self, x):
        return my_linear.apply(x, self.weight, self.bias)


class SparseLinear(nn.Linear):
    def forward(self, x):
        return sparse_linear.apply(x, self.weight, self.bias)


class sparse_linear_transpose(autograd.Function):
    """README.md:169-200 of the reference.  Three sparse GEMMs per layer and micro-step."""

    @staticmethod
    @custom_fwd(device_type='cuda', cast_inputs=torch.float16)
    def forward(ctx, input, weight, weight_sparse, weight_sparse_T, bias):
        ctx.save_for_backward(input, weight_sparse_T, bias)
        ctx.shape = input.shape
        input = input.reshape(-1, input.shape[-1])
        # same product as torch.mm(input, weight_sparse.t()); calling the GEMM wrapper directly skips the
        # Python-level tensor-subclass dispatch; the bias is added in the GEMM epilogue (one rounding instead of
        # the listing's two)
        b = None if bias is None else bias.to(input.dtype)
        output = _spmm(input, weight_sparse.sparse_tensor_cutlass, weight_sparse.meta_tensor_cutlass, bias=b)
        return output.view(*ctx.shape[:-1], -1)

    @staticmethod
    @custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        input, weight_T, bias = ctx.saved_tensors
        grad_input = grad_weight = grad_bias = None
        if grad_output.dim() == 3 and grad_output.stride() == (0, 0, 0):
            grad_output = torch.ones_like(grad_output, device=grad_output.device, dtype=grad_output.dtype)
        grad_output = grad_output.reshape(-1, grad_output.shape[-1])
        if ctx.needs_input_grad[0]:
            # torch.mm(grad_output, weight_T.t())
            grad_input = _spmm(grad_output, weight_T.sparse_tensor_cutlass, weight_T.meta_tensor_cutlass).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            input = input.reshape(-1, input.shape[-1])
            # torch.mm(to_sparse_semi_structured(grad_output.t(), MVUE24=True), input)
            gs = to_sparse_semi_structured(grad_output.t(), MVUE24=True, dtype=grad_output.dtype)
            grad_weight = _spmm(input.t(), gs.sparse_tensor_cutlass, gs.meta_tensor_cutlass).t()
        if ctx.needs_input_grad[4]:
            grad_bias = grad_output.sum(0)
        return grad_input, grad_weight, None, None, grad_bias


def _mvue_compress_t(g, row_sums):
    """MVUE 2:4 compression of ``g.t()`` (features x tokens, column-major) into buffers carved like
    ``SparseSemiStructuredTensor`` carves them, with the per-feature sums of ``g`` added to ``row_sums``
    by the same pass.  Returns (packed values, reordered metadata)."""
    tokens, features = g.shape
    if features % 32 or tokens % 64:
        raise RuntimeError(f"gradient of shape {tuple(g.shape)}: features % 32 == 0 and tokens % 64 == 0 required")
    g = g.contiguous()
    buf = torch.empty((features * tokens * 9 // 16,), dtype=g.dtype, device=g.device)
    packed = buf[: features * tokens // 2].view(-1, features).t()
    meta = buf[features * tokens // 2:].view(torch.int16).view(features, -1)
    prune_compress(g.t(), packed, meta, mode=_ext.PRUNE_MVUE_FAST, seed=random.randint(0, 2 ** 31 - 1), row_sums=row_sums)
    return packed, meta


def _mm_f32(a, b, acc=None):
    """a @ b (16-bit operands) with a float32 result; added into ``acc`` in the GEMM's epilogue when given."""
    try:
        if acc is not None:
            return torch.addmm(acc, a, b, out_dtype=torch.float32, out=acc)
        return torch.mm(a, b, out_dtype=torch.float32)
    except (TypeError, RuntimeError):             # a torch without the out_dtype argument on this overload
        r = torch.mm(a, b).float()
        return r if acc is None else acc.add_(r)


def _dense_weight_grads(g, x, weight, bias, into_grad, need_w, need_b):
    """The exact dW = g^T x as a dense GEMM with float32 output (the option ``weight_grad = "dense"`` of the layer).
    Same contract as ``_fst_weight_grads``."""
    grad_weight = grad_bias = None
    into = into_grad and weight.grad is not None and weight.grad.dtype == torch.float32 and weight.grad.is_contiguous()
    if need_w:
        if into:
            _mm_f32(g.t(), x, weight.grad)
        else:
            gw = _mm_f32(g.t(), x)
            grad_weight = gw if weight.dtype == torch.float32 else gw.to(weight.dtype)
    if bias is not None and need_b:
        if into and need_w and bias.grad is not None and bias.grad.dtype == torch.float32:
            bias.grad.add_(g.sum(0, dtype=torch.float32))
        else:
            grad_bias = g.sum(0)
    return grad_weight, grad_bias


def _fst_weight_grads(g, x, weight, bias, into_grad, need_w, need_b):
    """dW = MVUE24(g^T) x and db = g.sum(0) of one FST layer; ``g`` (tokens, out_features) and ``x`` (tokens,
    in_features) are 16-bit.  With ``into_grad`` (and an fp32 ``weight.grad`` already allocated) the GEMM adds dW
    straight into ``weight.grad`` and the compression pass adds the column sums of ``g`` into ``bias.grad``; autograd
    then receives None for both.  Returns (grad_weight, grad_bias)."""
    if getattr(weight, 'weight_grad', 'mvue') == 'dense':
        return _dense_weight_grads(g, x, weight, bias, into_grad, need_w, need_b)
    grad_weight = grad_bias = None
    bias_done = False
    if need_w:
        fp32_grad = weight.dtype == torch.float32 and x.shape[1] % 8 == 0
        target = weight if (into_grad and fp32_grad) else None
        into = target is not None and target.grad is not None and target.grad.dtype == torch.float32 \
            and target.grad.is_contiguous()
        bias_grad = None
        if into and bias is not None and need_b and g.dtype in (torch.float16, torch.bfloat16):
            bg = bias.grad
            if bg is not None and bg.dtype == torch.float32 and bg.is_contiguous():
                bias_grad = bg
        if bias_grad is not None:
            # the pass that compresses dY^T also adds its row sums (= grad_output.sum(0)) to bias.grad
            gp, gm = _mvue_compress_t(g, bias_grad)
            bias_done = True
        else:
            gs = to_sparse_semi_structured(g.t(), MVUE24=True, dtype=g.dtype)
            gp, gm = gs.sparse_tensor_cutlass, gs.meta_tensor_cutlass
        if into:
            _spmm_acc(target.grad, gp, gm, x)
        elif fp32_grad:
            # split-K GEMM with fp32 accumulation: the gradient arrives in the dtype of the master weight
            grad_weight = torch.zeros((g.shape[1], x.shape[1]), dtype=torch.float32, device=g.device)
            _spmm_acc(grad_weight, gp, gm, x)
        else:
            grad_weight = _spmm(x.t(), gp, gm).t()
    if bias is not None and need_b and not bias_done:
        grad_bias = g.sum(0)
    return grad_weight, grad_bias


class _fst_linear(autograd.Function):
    """What ``sparse_linear_transpose`` computes, on the raw compressed buffers: no tensor-subclass objects,
    no cast of the (unused) fp32 weight.  ``weight`` only routes the gradient.  With ``into_grad`` the weight
    gradient is accumulated by the GEMM itself into the existing fp32 ``weight.grad`` (D += A B) and autograd
    receives no gradient for the weight: no zero-filled temporary, no separate add."""

    @staticmethod
    def forward(ctx, input, weight, pw, mw, pt, mt, bias, into_grad=False):
        x = input.reshape(-1, input.shape[-1])
        if x.dtype != pw.dtype:
            x = x.to(pw.dtype)
        ctx.save_for_backward(x, pt, mt)
        ctx.shape = input.shape
        ctx.weight, ctx.bias, ctx.into_grad = weight, bias, into_grad
        if bias is not None and bias.dtype == torch.float32 and mlp_fusable(pw, x):
            output = _spmm_mlp(x, pw, mw, bias=bias)      # float32 bias read by the epilogue: no cast launch
        else:
            b = None if bias is None else (bias if bias.dtype == pw.dtype else bias.to(pw.dtype))
            output = _spmm(x, pw, mw, bias=b)             # bias added in the GEMM epilogue
        return output.view(*input.shape[:-1], -1)

    @staticmethod
    def backward(ctx, grad_output):
        x, pt, mt = ctx.saved_tensors
        grad_input = None
        if grad_output.dim() == 3 and grad_output.stride() == (0, 0, 0):
            grad_output = torch.ones_like(grad_output)
        g = grad_output.reshape(-1, grad_output.shape[-1])
        if g.dtype != pt.dtype:
            g = g.to(pt.dtype)
        if ctx.needs_input_grad[0]:
            grad_input = _spmm(g, pt, mt).view(ctx.shape)
        grad_weight, grad_bias = _fst_weight_grads(g, x, ctx.weight, ctx.bias, ctx.into_grad, ctx.needs_input_grad[1],
                                                   ctx.needs_input_grad[6])
        return grad_input, grad_weight, None, None, None, None, grad_bias, None


class _fst_mlp(autograd.Function):
    """Transformer MLP, proj(gelu(fc(x))), on two FST layers with the element-wise work folded into the GEMM epilogues:
    the up-projection writes both the pre-activation h and gelu(h); in the backward pass the down-projection's input
    gradient is multiplied by gelu'(h) in its epilogue, so the gradient of h is written directly.  Saves four passes
    over the (tokens, 4 d) activations per layer and step (GELU forward, its backward, and the tensors between them).
    ``fc`` / ``proj`` are (weight, bias, (pw, mw, pt, mt), into_grad)."""

    @staticmethod
    def forward(ctx, input, w_fc, b_fc, w_proj, b_proj, comp_fc, comp_proj, into_grad):
        pw1, mw1, pt1, mt1 = comp_fc
        pw2, mw2, pt2, mt2 = comp_proj
        x = input.reshape(-1, input.shape[-1])
        if x.dtype != pw1.dtype:
            x = x.to(pw1.dtype)
        act, pre = _spmm_mlp(x, pw1, mw1, bias=b_fc, epilogue="gelu")
        out = _spmm_mlp(act, pw2, mw2, bias=b_proj)
        ctx.save_for_backward(x, act, pre, pt1, mt1, pt2, mt2)
        ctx.shape = input.shape
        ctx.params = (w_fc, b_fc, w_proj, b_proj, into_grad)
        return out.view(*input.shape[:-1], -1)

    @staticmethod
    def backward(ctx, grad_output):
        x, act, pre, pt1, mt1, pt2, mt2 = ctx.saved_tensors
        w_fc, b_fc, w_proj, b_proj, into_grad = ctx.params
        g = grad_output.reshape(-1, grad_output.shape[-1])
        if g.dtype != pt2.dtype:
            g = g.to(pt2.dtype)
        g = g.contiguous()
        need = ctx.needs_input_grad
        d_pre = _spmm_mlp(g, pt2, mt2, epilogue="dgelu", aux=pre)           # gradient of fc's output, (tokens, 4 d)
        gw2, gb2 = _fst_weight_grads(g, act, w_proj, b_proj, into_grad, need[3], need[4])
        grad_input = _spmm(d_pre, pt1, mt1).view(ctx.shape) if need[0] else None
        gw1, gb1 = _fst_weight_grads(d_pre, x, w_fc, b_fc, into_grad, need[1], need[2])
        return grad_input, gw1, gb1, gw2, gb2, None, None, None


def fst_mlp(x, fc, proj):
    """proj(gelu(fc(x), approximate="tanh")) for two ``SparseLinearTranspose`` layers.  Runs the fused epilogues when
    both layers are in sparse mode, their compressed copies are 16-bit and their shapes allow it; otherwise exactly
    the three separate calls.  Counters of both layers advance as in their own ``forward``."""
    w1, w2 = fc.weight, proj.weight
    ok = w1.mode == 'sparse' and w2.mode == 'sparse' and w1.is_cuda and w1.shape[0] % 256 == 0 and w2.shape[0] % 256 == 0 \
        and fc.bias is not None and proj.bias is not None
    if not ok:
        return proj(F.gelu(fc(x), approximate="tanh"))
    fc._ensure_compressed()
    proj._ensure_compressed()
    y = _fst_mlp.apply(x, w1, fc.bias, w2, proj.bias, w1.compressed, w2.compressed,
                       fc.accumulate_into_grad and proj.accumulate_into_grad)
    fc._advance()
    proj._advance()
    return y


class SparseLinearTranspose(nn.Linear):
    """Drop-in for ``nn.Linear`` that trains with 2:4 sparse GEMMs (FST).

    State lives on ``self.weight`` as in the reference listing: ``freq`` (mask refresh period in
    optimizer steps), ``cnt`` (micro-steps since the last optimizer step; the training loop resets it
    to 0 after each optimizer step), ``counter`` (optimizer steps), ``step`` (forward calls),
    ``mask`` (bool, transposable 2:4), ``weight_sparse`` / ``weight_sparse_T`` and ``mode``
    ('sparse' or 'dense').  When both the mask and the compressed copies are due, one fused kernel
    produces all three from a single read of the weight.

    ``materialize_sparse_tensors`` (class attribute, default False): when True the compressed copies are
    also wrapped as ``SparseSemiStructuredTensor`` objects in ``weight.weight_sparse`` /
    ``weight.weight_sparse_T`` after every refresh, as in the listing; the layer itself works on the raw
    buffers (``weight.compressed`` = (packed_w, meta_w, packed_t, meta_t)) to keep the host cost low.
    """

    materialize_sparse_tensors = False
    # How the weight gradient is formed (``weight.weight_grad``, set per layer from this class attribute).  "mvue": the
    # reference recipe, dW = MVUE24(dY^T) X on the sparse tensor cores (README.md:190-192 of the reference).  "dense":
    # the exact dW = dY^T X as a dense GEMM: no estimator noise, and on B200 the faster of the two (the MVUE pass plus
    # the sparse GEMM take longer than the dense GEMM they replace).
    weight_grad = "mvue"
    # True: the weight-gradient GEMM adds straight into an existing fp32 ``weight.grad`` (a trainer that owns flat
    # gradient buffers and needs no autograd hook on the weight, e.g. the graph-replayed one); False: autograd gets it
    accumulate_into_grad = False

    def __init__(self, in_features: int, out_features: int, bias: bool = True, func=lambda step: 'dense', **kwargs):
        super().__init__(in_features, out_features, bias=bias, **kwargs)
        self.weight.freq = 40  # update freq

        self.weight.cnt = 0  # how many steps after an optim step
        self.weight.counter = 0  # how many optim steps
        self.weight.step = 0  # total training step

        self.weight.mask = torch.ones_like(self.weight, dtype=torch.bool)
        self.weight.weight_sparse = None
        self.weight.weight_sparse_T = None
        self.weight.compressed = None
        self.weight.mode = 'sparse'
        self.weight.weight_grad = self.weight_grad
        self.func = func

        self.transposable_sparse = TransposableSparse(abs=True)
        SparseSemiStructuredTensor._FORCE_CUTLASS = True  # kept for parity with the reference; has no effect

    def _refresh(self, reselect: bool):
        w = self.weight
        # a reselected mask overwrites the existing buffer, so w.mask keeps one address for the whole run
        reuse = w.mask if (reselect and w.mask.is_cuda and w.mask.is_contiguous() and w.mask.dtype == torch.bool) else None
        # compressed copies in the autocast dtype when it is bf16 (no cast passes over the activations);
        # fp16 otherwise, like the reference layer (custom_fwd(cast_inputs=torch.float16))
        dtype = torch.float16
        if torch.is_autocast_enabled('cuda') and torch.get_autocast_dtype('cuda') == torch.bfloat16:
            dtype = torch.bfloat16
        mask, (pw, mw), (pt, mt) = select_and_compress(w, mask=None if reselect else w.mask, dtype=dtype,
                                                       mask_out=reuse)
        w.mask = mask
        w.compressed = (pw, mw, pt, mt)
        if not self.materialize_sparse_tensors:
            w.weight_sparse = w.weight_sparse_T = None
            return
        out_f, in_f = w.shape
        w.weight_sparse = SparseSemiStructuredTensor(
            None, original_shape=torch.Size([out_f, in_f]), sparse_tensor_cutlass=pw, meta_tensor_cutlass=mw,
            dtype=dtype)
        w.weight_sparse_T = SparseSemiStructuredTensor(
            None, original_shape=torch.Size([in_f, out_f]), sparse_tensor_cutlass=pt, meta_tensor_cutlass=mt,
            dtype=dtype)

    def _ensure_compressed(self):
        """Rebuild the mask and / or the compressed copies when this forward pass is due to (first micro-step after an
        optimizer step; every ``freq`` optimizer steps with a new mask)."""
        w = self.weight
        if w.mask.device != w.device:
            w.mask = w.mask.to(device=w.device)
        if w.cnt == 0:
            if getattr(w, 'refreshed', False):
                w.refreshed = False      # refresh_sparse_layers has just rebuilt the copies of this step
            else:
                self._refresh(reselect=(w.counter % w.freq == 0))
        elif w.compressed is None:   # state restored in the middle of an accumulation window
            self._refresh(reselect=False)

    def _advance(self):
        w = self.weight
        if self.training:
            if w.cnt == 0:
                w.counter += 1
            w.step += 1
            w.cnt += 1

    def forward(self, x):
        w = self.weight
        if w.mode == 'dense':
            x = F.linear(x, w, self.bias)
        else:
            self._ensure_compressed()
            pw, mw, pt, mt = w.compressed
            x = _fst_linear.apply(x, w, pw, mw, pt, mt, self.bias, self.accumulate_into_grad)
        self._advance()
        return x


def refresh_sparse_layers(model: nn.Module) -> int:
    """What every ``SparseLinearTranspose`` of ``model`` would do at the start of its next forward pass when a
    refresh is due (``cnt`` == 0): reselect the mask if ``counter % freq == 0`` and rebuild the compressed copies
    of W and W^T; done here for all those layers with one kernel launch per 48 weights instead of one per layer.
    Call it right before the forward pass, under the same autocast context.  Layers whose shapes are not
    multiples of 128 are left to refresh themselves.  Returns the number of layers refreshed."""
    from .transposable_semi_structured import select_and_compress_many
    dtype = torch.float16
    if torch.is_autocast_enabled('cuda') and torch.get_autocast_dtype('cuda') == torch.bfloat16:
        dtype = torch.bfloat16
    groups = {}
    for mod in model.modules():
        if not isinstance(mod, SparseLinearTranspose):
            continue
        w = mod.weight
        if w.mode != 'sparse' or w.cnt != 0 or not w.is_cuda or w.shape[0] % 128 or w.shape[1] % 128:
            continue
        if w.mask.device != w.device:
            w.mask = w.mask.to(device=w.device)
        if w.mask.dtype != torch.bool or not w.mask.is_contiguous():
            w.mask = w.mask.to(torch.bool).contiguous()
        groups.setdefault((w.counter % w.freq == 0, w.dtype, w.device), []).append(mod)
    done = 0
    for (reselect, _, _), mods in groups.items():
        res = select_and_compress_many([m.weight for m in mods], [m.weight.mask for m in mods], dtype=dtype,
                                       reselect=reselect)
        for mod, (mask, (pw, mw), (pt, mt)) in zip(mods, res):
            w = mod.weight
            w.compressed = (pw, mw, pt, mt)
            w.refreshed = True
            if mod.materialize_sparse_tensors:
                out_f, in_f = w.shape
                w.weight_sparse = SparseSemiStructuredTensor(
                    None, original_shape=torch.Size([out_f, in_f]), sparse_tensor_cutlass=pw, meta_tensor_cutlass=mw,
                    dtype=dtype)
                w.weight_sparse_T = SparseSemiStructuredTensor(
                    None, original_shape=torch.Size([in_f, out_f]), sparse_tensor_cutlass=pt, meta_tensor_cutlass=mt,
                    dtype=dtype)
            else:
                w.weight_sparse = w.weight_sparse_T = None
            done += 1
    return done


def sparse_state(model: nn.Module) -> dict:
    """Training state the FST layers keep outside ``state_dict()``: per sparse weight its mask, counters,
    refresh period and mode, keyed by parameter name.  Save it next to the checkpoint."""
    out = {}
    for name, p in model.named_parameters():
        if hasattr(p, 'mask'):
            out[name] = {'mask': p.mask.detach().cpu(), 'cnt': p.cnt, 'counter': p.counter, 'step': p.step,
                         'freq': p.freq, 'mode': p.mode}
    return out


def load_sparse_state(model: nn.Module, state: dict) -> None:
    """Inverse of ``sparse_state``; call after ``load_state_dict``.  The compressed copies are dropped,
    so the next forward pass of a layer in the middle of an accumulation window (``cnt`` != 0)
    rebuilds them from the restored weight under the restored mask."""
    params = dict(model.named_parameters())
    for name, st in state.items():
        if name not in params or not hasattr(params[name], 'mask'):
            raise RuntimeError(f"load_sparse_state: {name} is not a sparse weight of this model")
        p = params[name]
        if tuple(st['mask'].shape) != tuple(p.shape):
            raise RuntimeError(f"load_sparse_state: mask of {name} has shape {tuple(st['mask'].shape)}, expected {tuple(p.shape)}")
        p.mask = st['mask'].to(device=p.device, dtype=torch.bool)
        p.cnt, p.counter, p.step, p.freq, p.mode = st['cnt'], st['counter'], st['step'], st['freq'], st['mode']
        p.compressed = None
        p.weight_sparse = p.weight_sparse_T = None
