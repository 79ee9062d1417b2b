"""Masked decay (sparse/decay.py:27-37 of the reference)."""
import torch

from . import _ext


def masked_add_(grad: torch.Tensor, p_data: torch.Tensor, p_mask: torch.Tensor, alpha: float = 0):
    '''
    equivalent to
    grad.add_(p.data * (1 - p.mask), alpha=decay)
    '''
    assert grad.is_cuda and p_data.is_cuda and p_mask.is_cuda
    _ext.require_cuda(grad, p_data, p_mask)
    assert (grad.layout, p_data.layout, p_mask.layout) == (torch.strided, torch.strided, torch.strided)
    assert grad.stride() == p_data.stride() == p_mask.stride()
    if grad.dtype != torch.float32 or p_data.dtype != torch.float32:
        raise RuntimeError("masked_add_: grad and p_data must be float32 (cast the gradient with .float() first)")
    if not grad.is_contiguous():
        # the reference indexes flat storage; only dense storage makes that well defined
        raise RuntimeError("masked_add_: tensors must be contiguous")
    if p_mask.dtype in (torch.bool, torch.uint8, torch.int8):
        itemsize = 1
    elif p_mask.dtype in (torch.float16, torch.bfloat16):
        itemsize = 2
    elif p_mask.dtype == torch.float32:
        itemsize = 4
    else:
        p_mask = p_mask != 0
        itemsize = 1
    rc = _ext.lib().sp24_masked_add(grad.data_ptr(), p_data.data_ptr(), p_mask.data_ptr(), itemsize, grad.numel(),
                                    float(alpha), _ext.stream())
    _ext.check(rc, "sp24_masked_add")


def adamw_masked_decay_(p, grad, exp_avg, exp_avg_sq, *, step, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                        mask=None, alpha=0.0):
    """Masked decay (``masked_add_``) and the AdamW update of ``p`` in one pass.  All tensors float32, contiguous,
    same number of elements; ``mask`` bool / uint8 or None.  ``step``: the optimizer step number (int, from 1),
    or a one-element float32 CUDA tensor holding it (read on the device, for CUDA-graph replay).  ``grad`` is
    left unchanged."""
    _ext.require_cuda(p, grad, exp_avg, exp_avg_sq, mask)
    n = p.numel()
    for t in (p, grad, exp_avg, exp_avg_sq):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n:
            raise RuntimeError("adamw_masked_decay_: expected contiguous float32 tensors of equal size")
    if mask is not None:
        if mask.dtype not in (torch.bool, torch.uint8) or not mask.is_contiguous() or mask.numel() != n:
            raise RuntimeError("adamw_masked_decay_: mask must be a contiguous bool / uint8 tensor of the same size")
    step_dev, step_host = (step, 1.0) if isinstance(step, torch.Tensor) else (None, float(step))
    if step_dev is not None and (step_dev.dtype != torch.float32 or step_dev.numel() != 1 or not step_dev.is_cuda):
        raise RuntimeError("adamw_masked_decay_: a device step must be a one-element float32 CUDA tensor")
    rc = _ext.lib().sp24_adamw_masked_decay(p.data_ptr(), grad.data_ptr(), _ext.ptr(mask), exp_avg.data_ptr(),
                                            exp_avg_sq.data_ptr(), n, lr, betas[0], betas[1], eps, weight_decay, alpha,
                                            step_host, _ext.ptr(step_dev), _ext.stream())
    _ext.check(rc, "sp24_adamw_masked_decay")
    return p
