"""Drop-in ``sparse`` package: the 2:4 sparse-training hot path on B200 (sm_100a) CUDA kernels.

Public names follow sparse/__init__.py of the reference for everything on that path, plus the
classes the reference only lists in its README (``SparseLinearTranspose``,
``sparse_linear_transpose``, ``mask_select``).
"""
from .legacy import MVUE24_approx_torch, sparse24_torch, soft_threshold24_torch
from .triton_ops import MVUE24_approx_triton, sparse24_triton, soft_threshold24_triton
from .decay import masked_add_, adamw_masked_decay_
from .transposable_semi_structured import TransposableSparse, select_and_compress, select_and_compress_many
from .semi_structured import to_sparse_semi_structured, SparseSemiStructuredTensor
from .sparse_ops import (MyLinear, SparseLinear, SparseLinearTranspose, sparse_linear_transpose, sparse_state,
                         load_sparse_state, refresh_sparse_layers, fst_mlp)
from .sste import SoftThreshold, SoftThresholdLinear
from . import fp8  # noqa: F401  (float8 form of the FST layer: sparse.fp8.sparse_linear_transpose_fp8)

mask_select = TransposableSparse()

__all__ = [
    'MyLinear',
    'SparseLinear',
    'SparseLinearTranspose',
    'sparse_linear_transpose',
    'MVUE24_approx_torch',
    'sparse24_torch',
    'soft_threshold24_torch',
    'MVUE24_approx_triton',
    'sparse24_triton',
    'soft_threshold24_triton',
    'masked_add_',
    'adamw_masked_decay_',
    'TransposableSparse',
    'mask_select',
    'select_and_compress',
    'select_and_compress_many',
    'refresh_sparse_layers',
    'fst_mlp',
    'to_sparse_semi_structured',
    'SparseSemiStructuredTensor',
    'SoftThreshold',
    'SoftThresholdLinear',
    'sparse_state',
    'load_sparse_state',
]
