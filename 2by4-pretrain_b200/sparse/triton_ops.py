"""Dense-shaped 2:4 prune ops.  The function names keep the reference's ``*_triton`` suffix
(sparse/triton_ops.py:55-81, :125-154, :198-227 of the reference) so existing call sites work
unchanged; the implementations are the sm_100a CUDA kernels, there is no Triton here."""
import random
from typing import Optional

import torch

from . import _ext


def _prep(dense: torch.Tensor):
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    _ext.require_cuda(dense)
    rs, cs = dense.stride()
    col_major = 0 if rs > cs else 1  # the reference's layout rule (sparse/triton_ops.py:61-67)
    dense = _ext.as_layout(dense, col_major)
    return dense, col_major, _ext.layout_of(dense)[1]


def _like(dense, col_major):
    m, k = dense.shape
    if col_major:
        return torch.empty((k, m), dtype=dense.dtype, device=dense.device).t()
    return torch.empty((m, k), dtype=dense.dtype, device=dense.device)


def MVUE24_approx_triton(dense, *, uniforms: Optional[torch.Tensor] = None, seed: Optional[int] = None, offset: int = 0,
                         exact: Optional[bool] = None):
    """Minimum-variance unbiased 2:4 estimate of ``dense`` (same shape, zeros where dropped).
    ``uniforms`` / ``seed`` / ``offset`` are optional extras for reproducibility; by default the seed
    comes from Python's ``random`` like the reference (sparse/triton_ops.py:58).

    ``exact``: True = IEEE arithmetic and the 10-round Philox stream, bit-exact against the reference formulas
    (always the case with ``uniforms``); False = the production arithmetic (reciprocal approximations, 7-round
    stream), which is what ``to_sparse_semi_structured(MVUE24=True)`` stores for the same seed.  Default: exact
    only when ``uniforms`` is given."""
    dense, col_major, ld = _prep(dense)
    m, k = dense.shape
    out = _like(dense, col_major)
    if exact is None:
        exact = uniforms is not None
    if uniforms is not None and not exact:
        raise RuntimeError("MVUE24_approx_triton: supplied uniforms drive the exact arithmetic only")
    if seed is None:
        seed = random.randint(0, 2 ** 31 - 1)
    if not exact:
        rc = _ext.lib().sp24_mvue24_dense_fast(dense.data_ptr(), _ext.dt(dense.dtype), m, k, ld, col_major, out.data_ptr(),
                                               _ext.layout_of(out)[1], seed, offset, _ext.stream())
        _ext.check(rc, "sp24_mvue24_dense_fast")
        return out
    ld_u = 0
    if uniforms is not None:
        uniforms = _ext.as_layout(uniforms.float(), col_major)
        ld_u = _ext.layout_of(uniforms)[1]
    rc = _ext.lib().sp24_mvue24_dense(dense.data_ptr(), _ext.dt(dense.dtype), m, k, ld, col_major, out.data_ptr(),
                                      _ext.layout_of(out)[1], _ext.ptr(uniforms), ld_u, seed, offset, _ext.stream())
    _ext.check(rc, "sp24_mvue24_dense")
    return out


def sparse24_triton(dense):
    """Magnitude 2:4 pruning: returns (sparse, mask), mask as 1/0 in ``dense``'s dtype."""
    dense, col_major, ld = _prep(dense)
    m, k = dense.shape
    sparse, mask = _like(dense, col_major), _like(dense, col_major)
    rc = _ext.lib().sp24_sparse24(dense.data_ptr(), _ext.dt(dense.dtype), m, k, ld, col_major, sparse.data_ptr(),
                                  _ext.layout_of(sparse)[1], mask.data_ptr(), _ext.layout_of(mask)[1], _ext.stream())
    _ext.check(rc, "sp24_sparse24")
    return sparse, mask


def soft_threshold24_triton(dense, scale: Optional[float] = None):
    """S-STE soft threshold: returns (sparse, mask).  ``scale`` (optional, not in the reference
    signature) folds the per-tensor S-STE factor into the same pass."""
    dense, col_major, ld = _prep(dense)
    m, k = dense.shape
    sparse, mask = _like(dense, col_major), _like(dense, col_major)
    rc = _ext.lib().sp24_soft_threshold24(dense.data_ptr(), _ext.dt(dense.dtype), m, k, ld, col_major,
                                          sparse.data_ptr(), _ext.layout_of(sparse)[1], mask.data_ptr(),
                                          _ext.layout_of(mask)[1], 0 if scale is None else 1,
                                          0.0 if scale is None else float(scale), _ext.stream())
    _ext.check(rc, "sp24_soft_threshold24")
    return sparse, mask
