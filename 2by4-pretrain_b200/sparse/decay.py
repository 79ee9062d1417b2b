"""Masked decay (sparse/decay.py:27-37 of the reference)."""
import torch

from . import _ext


def masked_add_(grad: torch.Tensor, p_data: torch.Tensor, p_mask: torch.Tensor, alpha: float = 0):
    '''
    equivalent to
    grad.add_(p.data * (1 - p.mask), alpha=decay)
    '''
    assert grad.is_cuda and p_data.is_cuda and p_mask.is_cuda
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
