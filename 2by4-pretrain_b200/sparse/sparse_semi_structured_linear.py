"""Python -> native shim of the sparse GEMM, same name and arguments as
sparse/sparse_semi_structured_linear.py:4-5 of the reference."""
from . import cutlass


def sparse_semi_structured_linear(input, weight, meta, bias_opt=None, activation_opt=None):
    return cutlass.my_sparse_semi_structured_linear(input, weight, meta, bias_opt, activation_opt)
