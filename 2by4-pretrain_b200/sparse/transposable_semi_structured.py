"""Transposable 4x4 mask select (sparse/transposable_semi_structured.py:50-200 of the reference)."""
import itertools

import torch
from torch import Tensor, nn

from . import _ext


def _pattern_table() -> torch.Tensor:
    """The 90 4x4 patterns with two ones per row and column, descending lexicographic order."""
    pairs = ((0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3))
    rows = []
    for combo in itertools.product(range(6), repeat=4):
        cnt = [0] * 4
        for i in combo:
            cnt[pairs[i][0]] += 1
            cnt[pairs[i][1]] += 1
        if cnt == [2, 2, 2, 2]:
            bits = []
            for i in combo:
                r = [0, 0, 0, 0]
                r[pairs[i][0]] = r[pairs[i][1]] = 1
                bits += r
            rows.append(bits)
    return torch.tensor(rows, dtype=torch.float32)


def _to_transposable_sparse_semi_structured(dense, mask_pattern=None, abs=True, need_sparse=True):
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    m, k = dense.shape
    if dense.dtype not in [torch.float16, torch.bfloat16, torch.float32]:
        raise RuntimeError(f"Invalid datatype {dense.dtype} of dense matrix")
    if m % 32 != 0:
        raise RuntimeError(f"Number rows columns of dense matrix {m} must be divisible by 32")
    if k % 64 != 0:
        raise RuntimeError(f"Number of columns of dense matrix {k} must be divisible by {64}")
    _ext.require_cuda(dense)
    x = _ext.as_layout(dense.detach(), 0)
    sparse = torch.empty((m, k), dtype=dense.dtype, device=dense.device) if need_sparse else None
    mask = torch.empty((m, k), dtype=torch.bool, device=dense.device)
    rc = _ext.lib().sp24_transposable_select(x.data_ptr(), _ext.dt(x.dtype), m, k, _ext.layout_of(x)[1], 1 if abs else 0,
                                             _ext.ptr(sparse), k, mask.data_ptr(), k, _ext.stream())
    _ext.check(rc, "sp24_transposable_select")
    return sparse, mask


class TransposableSparse(nn.Module):
    r"""
    :return sparse, mask
    """

    def __init__(self, abs=True):
        super().__init__()
        self.abs = abs
        self.mask_pattern = _pattern_table()  # kept for API compatibility; the kernel enumerates it itself

    def forward(self, x: Tensor):
        return _to_transposable_sparse_semi_structured(x, self.mask_pattern, self.abs)


def select_and_compress(weight: Tensor, mask: Tensor = None, dtype: torch.dtype = torch.float16,
                        mask_out: Tensor = None):
    """One pass over ``weight`` (m, k): transposable mask (recomputed when ``mask`` is None, else read)
    plus the 2:4 compression of W and of W^T.  Returns (mask, (packed_w, meta_w), (packed_t, meta_t))
    where packed_t is the column-major (k, m/2) view the reference gets from
    ``to_sparse_semi_structured(W.T, mask=mask.T)``.  ``mask_out`` (bool, contiguous, (m, k)): when the
    mask is recomputed, write it there instead of into a new tensor (a buffer with a fixed address)."""
    _ext.require_cuda(weight, mask, mask_out)
    m, k = weight.shape
    w = _ext.as_layout(weight.detach(), 0)
    select = mask is None
    if select:
        if mask_out is not None:
            if mask_out.dtype != torch.bool or tuple(mask_out.shape) != (m, k) or not mask_out.is_contiguous():
                raise RuntimeError("select_and_compress: mask_out must be a contiguous bool tensor of the weight's shape")
            mask = mask_out
        else:
            mask = torch.empty((m, k), dtype=torch.bool, device=w.device)
    else:
        mask = _ext.as_layout(mask if mask.dtype in (torch.bool, torch.uint8) else mask != 0, 0)
    buf_w = torch.empty(m * k * 9 // 16, dtype=dtype, device=w.device)
    buf_t = torch.empty(m * k * 9 // 16, dtype=dtype, device=w.device)
    packed_w = buf_w[: m * k // 2].view(m, k // 2)
    meta_w = buf_w[m * k // 2:].view(torch.int16).view(m, k // 16)
    packed_t = buf_t[: m * k // 2].view(m // 2, k).t()
    meta_t = buf_t[m * k // 2:].view(torch.int16).view(k, m // 16)
    if m % 128 == 0 and k % 128 == 0:
        # whole tensor-core blocks: the kernel also writes both metadata copies in the order the GEMM reads
        from . import spmm as _spmm
        tc_w = torch.empty(_spmm.tc_bytes(m, k), dtype=torch.uint8, device=w.device)
        tc_t = torch.empty(_spmm.tc_bytes(k, m), dtype=torch.uint8, device=w.device)
        rc = _ext.lib().sp24_select_dual_compress_tc(
            w.data_ptr(), _ext.dt(w.dtype), m, k, _ext.layout_of(w)[1], 1 if select else 0, mask.data_ptr(),
            _ext.layout_of(mask)[1], packed_w.data_ptr(), _ext.dt(dtype), k // 2, meta_w.data_ptr(), packed_t.data_ptr(), k,
            meta_t.data_ptr(), tc_w.data_ptr(), tc_t.data_ptr(), _ext.stream())
        _ext.check(rc, "sp24_select_dual_compress_tc")
        _spmm.register_tc_metadata(meta_w, tc_w)
        _spmm.register_tc_metadata(meta_t, tc_t)
    else:
        rc = _ext.lib().sp24_select_dual_compress(
            w.data_ptr(), _ext.dt(w.dtype), m, k, _ext.layout_of(w)[1], 1 if select else 0, mask.data_ptr(),
            _ext.layout_of(mask)[1], packed_w.data_ptr(), _ext.dt(dtype), k // 2, meta_w.data_ptr(), packed_t.data_ptr(), k,
            meta_t.data_ptr(), _ext.stream())
        _ext.check(rc, "sp24_select_dual_compress")
    return mask, (packed_w, meta_w), (packed_t, meta_t)


def select_and_compress_many(weights, masks, dtype: torch.dtype = torch.float16, reselect: bool = False):
    """``select_and_compress`` for a list of weights of one dtype in one kernel launch per 48 matrices (the
    per-step recompression of all layers of a model, each too small to fill the GPU alone).  ``masks``: one
    contiguous bool (m, k) tensor per weight; read when ``reselect`` is false, overwritten with the newly
    selected mask when it is true.  Every shape must be a multiple of 128 in both dimensions.  Returns a list of
    (mask, (packed_w, meta_w), (packed_t, meta_t)) like the single call."""
    from . import spmm as _spmm
    if len(weights) == 0:
        return []
    if len(masks) != len(weights):
        raise RuntimeError("select_and_compress_many: one mask per weight")
    _ext.require_cuda(*weights, *masks)
    descs = (_ext.DualDesc * len(weights))()
    out, keep = [], []
    for i, (weight, mask) in enumerate(zip(weights, masks)):
        m, k = weight.shape
        if m % 128 or k % 128:
            raise RuntimeError(f"select_and_compress_many: shape {(m, k)} is not a multiple of 128 x 128")
        if weight.dtype != weights[0].dtype or weight.device != weights[0].device:
            raise RuntimeError("select_and_compress_many: all weights must share dtype and device")
        if mask.dtype != torch.bool or tuple(mask.shape) != (m, k) or not mask.is_contiguous():
            raise RuntimeError("select_and_compress_many: masks must be contiguous bool tensors of the weights' shapes")
        w = _ext.as_layout(weight.detach(), 0)
        buf_w = torch.empty(m * k * 9 // 16, dtype=dtype, device=w.device)
        buf_t = torch.empty(m * k * 9 // 16, dtype=dtype, device=w.device)
        packed_w = buf_w[: m * k // 2].view(m, k // 2)
        meta_w = buf_w[m * k // 2:].view(torch.int16).view(m, k // 16)
        packed_t = buf_t[: m * k // 2].view(m // 2, k).t()
        meta_t = buf_t[m * k // 2:].view(torch.int16).view(k, m // 16)
        tc_w = torch.empty(_spmm.tc_bytes(m, k), dtype=torch.uint8, device=w.device)
        tc_t = torch.empty(_spmm.tc_bytes(k, m), dtype=torch.uint8, device=w.device)
        d = descs[i]
        d.w, d.m, d.k, d.ld_w = w.data_ptr(), m, k, _ext.layout_of(w)[1]
        d.mask, d.ld_mask = mask.data_ptr(), k
        d.packed_w, d.ld_packed_w, d.meta_w = packed_w.data_ptr(), k // 2, meta_w.data_ptr()
        d.packed_t, d.ld_packed_t, d.meta_t = packed_t.data_ptr(), k, meta_t.data_ptr()
        d.tc_w, d.tc_t = tc_w.data_ptr(), tc_t.data_ptr()
        keep.append(w)
        out.append((mask, (packed_w, meta_w), (packed_t, meta_t), (tc_w, tc_t)))
    rc = _ext.lib().sp24_select_dual_compress_batch(descs, len(weights), _ext.dt(weights[0].dtype), _ext.dt(dtype),
                                                    1 if reselect else 0, _ext.stream())
    _ext.check(rc, "sp24_select_dual_compress_batch")
    res = []
    for mask, (pw, mw), (pt, mt), (tc_w, tc_t) in out:
        _spmm.register_tc_metadata(mw, tc_w)
        _spmm.register_tc_metadata(mt, tc_t)
        res.append((mask, (pw, mw), (pt, mt)))
    return res
