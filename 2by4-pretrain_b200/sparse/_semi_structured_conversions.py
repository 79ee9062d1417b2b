"""Dense <-> 2:4 compressed conversion on the GPU.

Keeps the reference module's function names (sparse/_semi_structured_conversions.py of the
reference: ``sparse_semi_structured_from_dense_triton`` :1072-1132,
``sparse_semi_structured_from_dense`` :331-337, ``sparse_semi_structured_to_dense`` :340-346)
but every one of them launches the hand-written sm_100a kernels through the C ABI.
"""
import random
from typing import Optional

import torch
from torch import Tensor

from . import _ext

_META_DTYPE = {torch.float16: torch.int16, torch.bfloat16: torch.int16, torch.int8: torch.int32}
if hasattr(torch, "float8_e4m3fn"):
    _META_DTYPE[torch.float8_e4m3fn] = torch.int32
    _META_DTYPE[torch.float8_e5m2] = torch.int32


# Optional int64 device tensor (one element) whose value is added to the Philox offset of every seeded MVUE
# conversion when the kernel runs.  A training step recorded as a CUDA graph bakes the host-side seeds into the
# graph; bumping this word between replays gives every replay fresh uniforms.
_DEVICE_RNG_OFFSET: Optional[Tensor] = None


def set_device_rng_offset(counter: Optional[Tensor]) -> None:
    """Install (or, with None, remove) the device word added to the MVUE Philox offset."""
    global _DEVICE_RNG_OFFSET
    if counter is not None:
        if counter.dtype != torch.int64 or counter.numel() != 1 or not counter.is_cuda:
            raise RuntimeError("set_device_rng_offset: expected a one-element int64 CUDA tensor")
    _DEVICE_RNG_OFFSET = counter


def prune_compress(dense: Tensor, sparse: Tensor, meta: Tensor, *, mode: int, mask: Optional[Tensor] = None,
                   uniforms: Optional[Tensor] = None, seed: int = 0, offset: int = 0, emit_tc: Optional[bool] = None,
                   row_sums: Optional[Tensor] = None):
    """Low-level entry: fills ``sparse`` (packed values) and ``meta`` (reordered metadata) in place.

    ``dense`` is a logical (m, k) matrix in row- or column-major storage; ``sparse`` must be an
    (m, k/2) view in the same storage order (that is how the reference carves it,
    sparse/semi_structured.py:231-243).  ``uniforms`` (float32, logical (m, k)) is the test hook
    that drives MVUE with caller-supplied randomness; otherwise (seed, offset) key the Philox stream.
    """
    _ext.require_cuda(dense, sparse, meta, mask, uniforms)
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    m, k = dense.shape
    lay = _ext.layout_of(sparse)
    if lay is None:
        raise RuntimeError("packed output must be row- or column-major with unit inner stride")
    col_major, ld_p = lay
    dense = _ext.as_layout(dense, col_major)
    ld_d = _ext.layout_of(dense)[1]
    ld_m = ld_u = 0
    if mask is not None:
        if mask.dtype != torch.bool and mask.dtype != torch.uint8:
            mask = mask != 0
        mask = _ext.as_layout(mask, col_major)
        ld_m = _ext.layout_of(mask)[1]
    if uniforms is not None:
        uniforms = _ext.as_layout(uniforms.float(), col_major)
        ld_u = _ext.layout_of(uniforms)[1]
    if not meta.is_contiguous():
        raise RuntimeError("metadata buffer must be contiguous")
    dev_off = _DEVICE_RNG_OFFSET if mode in (_ext.PRUNE_MVUE, _ext.PRUNE_MVUE_FAST) and uniforms is None else None
    # 16-bit results with whole 128-row blocks can also get their metadata in the order the GEMM reads, in the same
    # pass.  Default: for column-major results (the dY^T operand of the weight-gradient GEMM, consumed at once);
    # row-major results (weights converted once) get it on request, else lazily at their first GEMM.
    e_tc = None
    want_tc = bool(col_major) if emit_tc is None else emit_tc
    if want_tc and sparse.element_size() == 2 and m % 128 == 0:
        from . import spmm as _spmm
        e_tc = torch.empty(_spmm.tc_bytes(m, k), dtype=torch.uint8, device=meta.device)
    if row_sums is not None:
        if not col_major or row_sums.dtype != torch.float32 or row_sums.numel() != m or not row_sums.is_contiguous():
            raise RuntimeError("row_sums: column-major input and a contiguous float32 vector of one value per row")
    if dev_off is not None or e_tc is not None or row_sums is not None:
        rc = _ext.lib().sp24_prune_compress_ex(
            dense.data_ptr(), _ext.dt(dense.dtype), m, k, ld_d, col_major, sparse.data_ptr(), _ext.dt(sparse.dtype), ld_p,
            meta.data_ptr(), mode, _ext.ptr(mask), ld_m, _ext.ptr(uniforms), ld_u, seed & (2 ** 64 - 1),
            offset & (2 ** 64 - 1), _ext.ptr(dev_off), _ext.ptr(e_tc), _ext.ptr(row_sums), _ext.stream())
    else:
        rc = _ext.lib().sp24_prune_compress(
            dense.data_ptr(), _ext.dt(dense.dtype), m, k, ld_d, col_major, sparse.data_ptr(), _ext.dt(sparse.dtype), ld_p,
            meta.data_ptr(), mode, _ext.ptr(mask), ld_m, _ext.ptr(uniforms), ld_u, seed & (2 ** 64 - 1),
            offset & (2 ** 64 - 1), _ext.stream())
    _ext.check(rc, "sp24_prune_compress")
    from .spmm import invalidate_meta, register_tc_metadata
    invalidate_meta(meta)  # a refilled metadata buffer must not reuse a cached tensor-core copy
    if e_tc is not None:
        register_tc_metadata(meta, e_tc)
    return sparse, meta


def sparse_semi_structured_from_dense_triton(dense, sparse, meta, MVUE24: bool = False, mask: Optional[Tensor] = None):
    """Name and arguments of the reference launcher (no Triton inside).  The MVUE seed is drawn from
    Python's ``random`` like the reference does (sparse/_semi_structured_conversions.py:1076)."""
    if mask is not None:
        mode = _ext.PRUNE_MASK
    elif MVUE24:
        mode = _ext.PRUNE_MVUE_FAST   # production arithmetic; PRUNE_MVUE (exact) is reached through prune_compress
    else:
        mode = _ext.PRUNE_MSE
    seed = random.randint(0, 2 ** 31 - 1)
    return prune_compress(dense, sparse, meta, mode=mode, mask=mask, seed=seed)


def sparse_semi_structured_from_dense(dense: Tensor):
    """Magnitude-prune and compress; returns (packed (m, k/2), reordered meta)."""
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    if dense.dtype not in _META_DTYPE:
        raise RuntimeError(f"Invalid datatype {dense.dtype} of dense matrix")
    m, k = dense.shape
    meta_dtype = _META_DTYPE[dense.dtype]
    per = 16 if meta_dtype == torch.int16 else 32
    if m % 32 != 0:
        raise RuntimeError(f"Number rows columns of dense matrix {m} must be divisible by 32")
    if k % (per if per == 32 else 16) != 0:
        raise RuntimeError(f"Number of columns of dense matrix {k} must be divisible by {per}")
    sparse = torch.empty((m, k // 2), dtype=dense.dtype, device=dense.device)
    meta = torch.empty((m, k // per), dtype=meta_dtype, device=dense.device)
    return prune_compress(dense.contiguous(), sparse, meta, mode=_ext.PRUNE_MSE)


def sparse_semi_structured_to_dense(sparse: Tensor, meta_reordered: Tensor):
    """Inverse conversion; ``sparse`` is the packed (m, k/2) matrix."""
    if sparse.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional sparse tensor, got {sparse.dim()}-dimensional tensor")
    if meta_reordered.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional meta tensor, got {meta_reordered.dim()}-dimensional tensor")
    if meta_reordered.device != sparse.device:
        raise RuntimeError(
            f"Expected meta matrix to be on {sparse.device} device, got matrix on {meta_reordered.device} device")
    if meta_reordered.dtype not in (torch.int16, torch.int32):
        raise RuntimeError(f"Invalid datatype {meta_reordered.dtype} of meta matrix")
    _ext.require_cuda(sparse, meta_reordered)
    m, kh = sparse.shape
    k = 2 * kh
    per = 16 if meta_reordered.dtype == torch.int16 else 32
    if meta_reordered.shape[0] != m:
        raise RuntimeError(
            f"Number of rows of meta matrix {meta_reordered.shape[0]} must be equal to number of columns of spase matrix {m}")
    if meta_reordered.shape[1] * per != k:
        raise RuntimeError(
            f"Number of columns of sparse matrix {kh} different from the {meta_reordered.shape[1] * per // 2}, "
            "expected according to the number of columns of meta matrix")
    sparse = sparse.contiguous()
    meta_reordered = meta_reordered.contiguous()
    dense = torch.empty((m, k), dtype=sparse.dtype, device=sparse.device)
    rc = _ext.lib().sp24_to_dense(sparse.data_ptr(), _ext.dt(sparse.dtype), m, k, kh, meta_reordered.data_ptr(),
                                  dense.data_ptr(), k, _ext.stream())
    _ext.check(rc, "sp24_to_dense")
    return dense


_sparse_semi_structured_to_dense_triton = sparse_semi_structured_to_dense
