"""2:4 sparse GEMM host wrapper (placeholder until the kernel entry point is bound)."""


def sparse_linear(input, weight, meta, bias=None, activation=None):
    raise NotImplementedError("the sm_100a 2:4 sparse GEMM is not available in this build")
