"""``SparseSemiStructuredTensor`` and ``to_sparse_semi_structured``.

Same public surface as sparse/semi_structured.py of the reference (constructor arguments, the
attributes ``sparse_tensor_cutlass`` / ``meta_tensor_cutlass`` / ``compressed_tensor_cusparselt`` /
``transposed`` / ``original_shape``, the class flags, and the ``__torch_dispatch__`` table for
detach / t / mm / addmm / linear / values / indices).  There is one backend: the conversion and the
sparse GEMM are the sm_100a kernels of this package.  ``_FORCE_CUTLASS`` and ``_FUSE_TRANSPOSE`` are
accepted and ignored; the ``*_cutlass`` attribute names are kept because callers read them.
"""
import warnings
from collections import namedtuple
from typing import Any, Optional

import torch

from . import _ext
from .sparse_semi_structured_linear import sparse_semi_structured_linear

__all__ = [
    "SparseSemiStructuredTensor",
    "to_sparse_semi_structured",
]

_SEMI_STRUCTURED_SPARSE_CONFIG = namedtuple(
    "_SEMI_STRUCTURED_SPARSE_CONFIG", "compression_factor sparse_min_rows sparse_min_cols dense_min_rows dense_min_cols"
)
# sparse/semi_structured.py:24-30 of the reference
_DTYPE_TO_SEMI_STRUCTURED_SPARSE_CONFIG = {
    torch.int8: _SEMI_STRUCTURED_SPARSE_CONFIG(10, 32, 128, 16, 16),
    torch.float8_e5m2: _SEMI_STRUCTURED_SPARSE_CONFIG(10, 32, 128, 16, 16),
    torch.float8_e4m3fn: _SEMI_STRUCTURED_SPARSE_CONFIG(10, 32, 128, 16, 16),
    torch.float16: _SEMI_STRUCTURED_SPARSE_CONFIG(9, 32, 64, 8, 8),
    torch.bfloat16: _SEMI_STRUCTURED_SPARSE_CONFIG(9, 32, 64, 8, 8),
}


def _indices_dtype(values_dtype):
    if values_dtype in (torch.int8, torch.float8_e5m2, torch.float8_e4m3fn):
        return torch.int32
    if values_dtype in (torch.float16, torch.bfloat16):
        return torch.int16
    raise RuntimeError(f"Datatype {values_dtype}  is not supported!")


class SparseSemiStructuredTensor(torch.Tensor):
    """2:4 (semi-structured) sparse matrix stored as packed kept values plus 4-bit-per-group metadata.

    A wrapper subclass: ``shape``/``dtype`` describe the logical dense matrix, the data lives in
    ``sparse_tensor_cutlass`` (packed values, (m, k/2), same storage order as the source) and
    ``meta_tensor_cutlass`` (reordered metadata), two views of one allocation of m*k*cf/16 elements.
    """

    _FUSE_TRANSPOSE = False
    _FORCE_CUTLASS = True
    _PROTOTYPE_WARNING_SHOWN = False

    @staticmethod
    def __new__(cls, original_tensor: Optional[torch.Tensor], original_shape: Optional[torch.Size] = None,
                compressed_tensor_cusparselt: Optional[torch.Tensor] = None,
                sparse_tensor_cutlass: Optional[torch.Tensor] = None,
                meta_tensor_cutlass: Optional[torch.Tensor] = None, transposed: bool = False, MVUE24: bool = False,
                mask: Optional[torch.Tensor] = None, dtype: Optional[torch.dtype] = None):
        assert compressed_tensor_cusparselt is None or (sparse_tensor_cutlass is None and meta_tensor_cutlass is None)

        if not cls._PROTOTYPE_WARNING_SHOWN:
            warnings.warn(
                "The PyTorch API of SparseSemiStructuredTensor is in prototype stage "
                "and will change in the near future. Please open a Github issue "
                "for features requests and see our documentation on the torch.sparse "
                "module for further information about the project.",
                UserWarning,
            )
            cls._PROTOTYPE_WARNING_SHOWN = True

        if original_tensor is not None:
            previous_tensor = original_tensor
            original_shape = original_tensor.shape
        elif compressed_tensor_cusparselt is not None:
            previous_tensor = compressed_tensor_cusparselt
        elif sparse_tensor_cutlass is not None:
            previous_tensor = sparse_tensor_cutlass
        else:
            raise ValueError("All of the tensor arguments are None!")

        kwargs = {
            "device": previous_tensor.device,
            "dtype": previous_tensor.dtype if dtype is None else dtype,
            "layout": previous_tensor.layout,
            "requires_grad": False,
        }
        return torch.Tensor._make_wrapper_subclass(cls, original_shape, **kwargs)  # type: ignore[attr-defined]

    def __init__(self, original_tensor: Optional[torch.Tensor], original_shape: Optional[torch.Size] = None,
                 compressed_tensor_cusparselt: Optional[torch.Tensor] = None,
                 sparse_tensor_cutlass: Optional[torch.Tensor] = None,
                 meta_tensor_cutlass: Optional[torch.Tensor] = None, transposed: bool = False, MVUE24: bool = False,
                 mask: Optional[torch.Tensor] = None, dtype: Optional[torch.dtype] = torch.float16) -> None:
        if original_tensor is not None:
            if not original_tensor.is_cuda:
                raise RuntimeError(
                    f"Error original_tensor.device= {original_tensor.device} is not supported! "
                    "Only CUDA tensors are currently supported."
                )
            if original_tensor.dim() != 2:
                raise RuntimeError(
                    f"Error original_tensor.dim = {original_tensor.dim()} is not supported! "
                    "Only 2d tensors are currently supported."
                )
            if dtype not in _DTYPE_TO_SEMI_STRUCTURED_SPARSE_CONFIG:
                raise RuntimeError(
                    f"Error dtype {dtype} is not a supported dtype! "
                    f"dtype must be one of: {list(_DTYPE_TO_SEMI_STRUCTURED_SPARSE_CONFIG)}"
                )
            cfg = _DTYPE_TO_SEMI_STRUCTURED_SPARSE_CONFIG[dtype]
            m, n = original_tensor.shape
            if m < cfg.sparse_min_rows or m % cfg.sparse_min_rows or n < cfg.sparse_min_cols or n % cfg.sparse_min_cols:
                raise RuntimeError(
                    f"Error original_tensor.shape {original_tensor.shape} is not supported! "
                    f"Both dimensions must be larger or equal than and a multiple of "
                    f"({cfg.sparse_min_rows}, {cfg.sparse_min_cols})"
                )
            if mask is not None and MVUE24:
                raise RuntimeError("Error using MVUE24 with mask is not supported! ")

            # one allocation: packed values first, metadata behind (m*n*cf/16 elements of dtype)
            compressed_size = original_tensor.nelement() * cfg.compression_factor // 16
            compressed_tensor = torch.empty((compressed_size,), dtype=dtype, device=original_tensor.device)
            indices_dtype = _indices_dtype(dtype)
            row_stride, col_stride = original_tensor.stride()
            if row_stride > col_stride:
                sparse_tensor_cutlass = compressed_tensor[: m * n // 2].view(m, -1)
            else:
                sparse_tensor_cutlass = compressed_tensor[: m * n // 2].view(-1, m).t()
            meta_tensor_cutlass = compressed_tensor[m * n // 2:].view(indices_dtype).view(m, -1)
            compressed_tensor_cusparselt = None

            from ._semi_structured_conversions import sparse_semi_structured_from_dense_triton
            sparse_semi_structured_from_dense_triton(original_tensor.detach(), sparse_tensor_cutlass,
                                                     meta_tensor_cutlass, MVUE24=MVUE24, mask=mask)

        self.original_tensor = None
        self.compressed_tensor_cusparselt = compressed_tensor_cusparselt
        self.sparse_tensor_cutlass = sparse_tensor_cutlass
        self.meta_tensor_cutlass = meta_tensor_cutlass
        self.transposed = transposed
        self.original_shape = original_shape

    def __tensor_flatten__(self):
        if self.compressed_tensor_cusparselt is None:
            return ['sparse_tensor_cutlass', 'meta_tensor_cutlass'], (self.original_shape, self.transposed)
        return ['compressed_tensor_cusparselt'], (self.original_shape, self.transposed)

    @staticmethod
    def __tensor_unflatten__(inner_tensors, meta, outer_size, outer_stride):
        original_shape, transposed = meta
        if len(inner_tensors) == 2:
            return SparseSemiStructuredTensor(
                None, original_shape=original_shape, sparse_tensor_cutlass=inner_tensors['sparse_tensor_cutlass'],
                meta_tensor_cutlass=inner_tensors['meta_tensor_cutlass'], transposed=transposed)
        if len(inner_tensors) == 1:
            return SparseSemiStructuredTensor(
                None, original_shape=original_shape,
                compressed_tensor_cusparselt=inner_tensors['compressed_tensor_cusparselt'], transposed=transposed)
        raise RuntimeError(f"Expected 1 or 2 inner tensors but got {len(inner_tensors)}")

    def __repr__(self) -> str:  # type: ignore[override]
        return (
            f"SparseSemiStructuredTensor(shape={self.shape}, "
            f"transposed={self.transposed}"
            f"values={self.values()}"
            f"metadata={self.indices()})"
        )

    __torch_function__ = torch._C._disabled_torch_function_impl

    def _copy_with(self, shape, transposed):
        return SparseSemiStructuredTensor(
            self.original_tensor, original_shape=shape,
            compressed_tensor_cusparselt=self.compressed_tensor_cusparselt,
            sparse_tensor_cutlass=self.sparse_tensor_cutlass, meta_tensor_cutlass=self.meta_tensor_cutlass,
            transposed=transposed, dtype=self.dtype)

    def _pad_tensor_for_matmul(self, original_tensor: torch.Tensor) -> torch.Tensor:
        """Pads the dense operand up to the multiples the sparse GEMM wants (8 for 16-bit, 16 for 8-bit).
        The column test deliberately repeats the reference's expression (it tests ``n % min_rows``,
        sparse/semi_structured.py:364); both minima are equal for every supported dtype."""
        assert original_tensor.dim() == 2
        m, n = original_tensor.shape
        cfg = _DTYPE_TO_SEMI_STRUCTURED_SPARSE_CONFIG[original_tensor.dtype]
        min_rows, min_cols = cfg.dense_min_rows, cfg.dense_min_cols
        to_pad_m = -m % min_rows if m < min_rows or m % min_rows else 0
        to_pad_n = -n % min_cols if n < min_cols or n % min_rows else 0
        if to_pad_m or to_pad_n:
            return torch.nn.functional.pad(original_tensor, (0, to_pad_n, 0, to_pad_m))
        return original_tensor

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs) -> Any:
        # below autograd: detach only rewraps the same buffers
        if func is torch.ops.aten.detach.default:
            return args[0]._copy_with(args[0].shape, args[0].transposed)

        # the compressed form cannot be transposed; only the flag and the logical shape flip
        if func is torch.ops.aten.t.default:
            return args[0]._copy_with(torch.Size([args[0].shape[1], args[0].shape[0]]), not args[0].transposed)

        if func is torch.ops.aten.addmm.default:
            bias, input_A, input_B = args
            # F.linear(x) = addmm(bias, x, W.t()) = (W x' + b')'
            if isinstance(input_B, cls) and input_B.transposed:
                row, col = input_A.shape
                input_A_padded = input_B._pad_tensor_for_matmul(input_A)
                assert input_B.sparse_tensor_cutlass is not None and input_B.meta_tensor_cutlass is not None
                res = sparse_semi_structured_linear(input_A_padded, input_B.sparse_tensor_cutlass,
                                                    input_B.meta_tensor_cutlass, bias_opt=bias)
                return res[:row, :]

        if func is torch.ops.aten.mm.default:
            input_A, input_B = args
            # first operand sparse: D = A_sparse @ B
            if isinstance(input_A, cls) and not input_A.transposed:
                row, col = input_B.shape
                input_B_padded = input_A._pad_tensor_for_matmul(input_B)
                assert input_A.sparse_tensor_cutlass is not None and input_A.meta_tensor_cutlass is not None
                res = sparse_semi_structured_linear(input_B_padded.t(), input_A.sparse_tensor_cutlass,
                                                    input_A.meta_tensor_cutlass).t()
                return res[:, :col]
            # second operand sparse and transposed: D = A @ W_sparse.t()
            elif isinstance(input_B, cls) and input_B.transposed:
                row, col = input_A.shape
                input_A_padded = input_B._pad_tensor_for_matmul(input_A)
                assert input_B.sparse_tensor_cutlass is not None and input_B.meta_tensor_cutlass is not None
                res = sparse_semi_structured_linear(input_A_padded, input_B.sparse_tensor_cutlass,
                                                    input_B.meta_tensor_cutlass)
                return res[:row, :]

        # inference mode does not decompose linear into t + addmm
        if func is torch.ops.aten.linear.default:
            input_tensor, weight, bias = args
            shape = input_tensor.shape
            input_tensor_2d = input_tensor.view(-1, shape[-1])
            row, col = input_tensor_2d.shape
            if isinstance(weight, cls):
                input_tensor_2d_padded = weight._pad_tensor_for_matmul(input_tensor_2d)
                assert weight.sparse_tensor_cutlass is not None and weight.meta_tensor_cutlass is not None
                res = sparse_semi_structured_linear(input_tensor_2d_padded, weight.sparse_tensor_cutlass,
                                                    weight.meta_tensor_cutlass, bias_opt=bias)
                return res[:row, :].view(*shape[:-1], -1)

        if func is torch.ops.aten.values.default:
            return args[0].sparse_tensor_cutlass.detach()

        if func is torch.ops.aten.indices.default:
            return args[0].meta_tensor_cutlass

        error_string = "\n".join(
            [f"func {func} with args: "]
            + [f"arg{i}: {arg}" for i, arg in enumerate(args)]
        )
        raise NotImplementedError(error_string)

    def to_dense(self):
        from ._semi_structured_conversions import sparse_semi_structured_to_dense
        return sparse_semi_structured_to_dense(self.sparse_tensor_cutlass.contiguous(),
                                               self.meta_tensor_cutlass.contiguous())


def to_sparse_semi_structured(
        original_tensor: torch.Tensor,
        transposed: bool = False,
        MVUE24: bool = False,
        mask: Optional[torch.Tensor] = None,
        dtype: torch.dtype = torch.float16,
) -> SparseSemiStructuredTensor:
    """Converts a dense 2-D CUDA tensor into a ``SparseSemiStructuredTensor``.

    Pruning rule: ``mask`` given -> keep what the mask says; ``MVUE24=True`` -> minimum-variance
    unbiased 2-of-4 sampling (for gradients); neither -> keep the two largest magnitudes of every
    four.  Values are cast to ``dtype`` on store.  Shape must be a multiple of (32, 64) for 16-bit
    ``dtype`` and (32, 128) for 8-bit.

    Example (the reference's own, sparse/semi_structured.py:603-627)::

        >>> A = torch.Tensor([0, 0, 1, 1]).tile((128, 32)).half().cuda()
        >>> A_sparse = to_sparse_semi_structured(A)
        >>> A_sparse.values()   # all ones, shape (128, 64)
        >>> A_sparse.indices()  # all -4370, shape (128, 8), int16
    """
    return SparseSemiStructuredTensor(
        original_tensor, original_shape=original_tensor.shape, transposed=transposed,
        MVUE24=MVUE24, mask=mask, dtype=dtype)
