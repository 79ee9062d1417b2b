"""Masked decay (sparse/decay.py:27-37 of the reference)."""
import torch

from . import _ext


def _storage_order(t: torch.Tensor):
    """``t`` as a flat view over its elements in storage order, or None when its storage is not dense (gaps or
    overlaps).  Tensors with equal sizes and strides keep their element correspondence under this view."""
    if t.is_contiguous():
        return t.view(-1)
    dims = sorted((st, sz) for sz, st in zip(t.shape, t.stride()) if sz != 1)
    expect = 1
    for st, sz in dims:
        if st != expect:
            return None
        expect *= sz
    return t.as_strided((t.numel(),), (1,), t.storage_offset())


def masked_add_(grad: torch.Tensor, p_data: torch.Tensor, p_mask: torch.Tensor, alpha: float = 0):
    '''
    equivalent to
    grad.add_(p.data * (1 - p.mask), alpha=decay)
    '''
    assert grad.is_cuda and p_data.is_cuda and p_mask.is_cuda
    _ext.require_cuda(grad, p_data, p_mask)
    assert (grad.layout, p_data.layout, p_mask.layout) == (torch.strided, torch.strided, torch.strided)
    assert grad.stride() == p_data.stride() == p_mask.stride()
    # like the reference kernel, work on flat storage: any dense layout shared by the three tensors will do
    g, q, m = _storage_order(grad), _storage_order(p_data), _storage_order(p_mask)
    if g is None or q is None or m is None or g.shape != q.shape or g.shape != m.shape:
        raise RuntimeError("masked_add_: tensors must share one dense layout (no gaps, no overlaps)")
    if m.dtype in (torch.bool, torch.uint8, torch.int8):
        itemsize = 1
    elif m.dtype in (torch.float16, torch.bfloat16):
        itemsize = 2
    elif m.dtype == torch.float32:
        itemsize = 4
    else:
        m = m != 0
        itemsize = 1
    # the kernel computes in float32 on float32 tensors; other floating types go through float32 copies and are
    # rounded once on the way back
    g32 = g if g.dtype == torch.float32 else g.float()
    q32 = q if q.dtype == torch.float32 else q.float()
    if g32.data_ptr() % 16 or q32.data_ptr() % 16 or m.data_ptr() % (4 * itemsize):
        g32 = g32.clone() if g32 is g else g32
        q32, m = q32.clone(), m.clone()
    rc = _ext.lib().sp24_masked_add(g32.data_ptr(), q32.data_ptr(), m.data_ptr(), itemsize, g32.numel(), float(alpha),
                                    _ext.stream())
    _ext.check(rc, "sp24_masked_add")
    if g32 is not g:
        g.copy_(g32)


def adamw_masked_decay_(p, grad, exp_avg, exp_avg_sq, *, step, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                        mask=None, alpha=0.0, extra_grad=None):
    """Masked decay (``masked_add_``) and the AdamW update of ``p`` in one pass.  All tensors float32, contiguous,
    same number of elements (``grad`` may also be float16 / bfloat16: what a 16-bit gradient exchange leaves behind);
    ``mask`` bool / uint8 or None.  ``step``: the optimizer step number (int, from 1),
    or a one-element float32 CUDA tensor holding it (read on the device, for CUDA-graph replay).  ``grad`` is
    left unchanged.  ``extra_grad``: a second gradient (float32 / float16 / bfloat16, contiguous, a multiple of four
    elements, at most as many as ``p``) added to ``grad`` on the leading elements it covers, inside the same pass."""
    _ext.require_cuda(p, grad, exp_avg, exp_avg_sq, mask, extra_grad)
    n = p.numel()
    for t in (p, grad, exp_avg, exp_avg_sq):
        ok_dtype = t.dtype == torch.float32 or (t is grad and t.dtype in (torch.float16, torch.bfloat16))
        if not ok_dtype or not t.is_contiguous() or t.numel() != n:
            raise RuntimeError("adamw_masked_decay_: expected contiguous float32 tensors of equal size")
    if mask is not None:
        if mask.dtype not in (torch.bool, torch.uint8) or not mask.is_contiguous() or mask.numel() != n:
            raise RuntimeError("adamw_masked_decay_: mask must be a contiguous bool / uint8 tensor of the same size")
    step_dev, step_host = (step, 1.0) if isinstance(step, torch.Tensor) else (None, float(step))
    if step_dev is not None and (step_dev.dtype != torch.float32 or step_dev.numel() != 1 or not step_dev.is_cuda):
        raise RuntimeError("adamw_masked_decay_: a device step must be a one-element float32 CUDA tensor")
    n2, dt2 = 0, 0
    if extra_grad is not None:
        n2 = extra_grad.numel()
        if extra_grad.dtype not in (torch.float32, torch.float16, torch.bfloat16) or not extra_grad.is_contiguous() \
                or n2 == 0 or n2 > n or n2 % 4:
            raise RuntimeError("adamw_masked_decay_: extra_grad must be a contiguous float tensor of 4 k <= numel(p) elements")
        dt2 = _ext.dt(extra_grad.dtype)
    rc = _ext.lib().sp24_adamw_masked_decay_ex(p.data_ptr(), grad.data_ptr(), _ext.dt(grad.dtype), _ext.ptr(mask), exp_avg.data_ptr(),
                                               exp_avg_sq.data_ptr(), n, lr, betas[0], betas[1], eps, weight_decay, alpha,
                                               step_host, _ext.ptr(step_dev), _ext.ptr(extra_grad), dt2, n2, _ext.stream())
    _ext.check(rc, "sp24_adamw_masked_decay_ex")
    return p
