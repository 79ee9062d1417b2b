"""Stands where the reference's pybind11 extension module ``sparse.cutlass`` stood
(sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:498-501, :979-981): one function,
``my_sparse_semi_structured_linear(input, weight, meta, bias, activation)``.  There is no CUTLASS
here; the name is kept for callers that import it.  The GEMM is the sm_100a ``tcgen05.mma.sp``
kernel reached through the C ABI."""
from . import spmm


def my_sparse_semi_structured_linear(input, weight, meta, bias_opt=None, activation_opt=None):
    return spmm.sparse_linear(input, weight, meta, bias_opt, activation_opt)
