"""Host side of the 2:4 sparse GEMM (tcgen05.mma.sp kernel behind ``sp24_spmm``).

``sparse_linear`` has the contract of the reference's only native function,
``my_sparse_semi_structured_linear(input, weight, meta, bias, activation)``
(sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:498-817 of the reference): ``weight`` is the packed
(ms, k/2) matrix (row- or column-major), ``meta`` its reordered metadata, ``input`` the dense (..., k)
operand; the result is (..., ms) = input @ dense(weight).T (+ bias) (activation).
"""
import ctypes
import weakref

import torch

from . import _ext

_i64, _i32, _vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
_ext.register_signature("sp24_meta_to_tc", [_vp, _i32, _i64, _i64, _vp, _vp])
_ext.register_signature("sp24_spmm", [_vp, _i32, _i32, _i64, _vp, _i64, _i64, _vp, _i32, _i64, _i64, _vp, _i32, _i32,
                                      _i64, _vp, _i32, _vp, _vp])

# allocation-free variant (metadata in the reference layout, tensor-core copy kept inside the library)
_ext.register_signature("sp24_spmm_noalloc", [_vp, _i32, _i32, _i64, _vp, _i64, _i64, _vp, _i32, _i64, _i64, _vp, _i32, _i32,
                                              _i64, _vp, _i32, _vp, _vp])

_ext.register_signature("sp24_spmm_scaled", [_vp, _i32, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i32, _i64, _vp, _i32,
                                             ctypes.c_float, _vp, _vp])
_ext.register_signature("sp24_spmm_mlp", [_vp, _i32, _i32, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i32, _i32, _vp,
                                          _i64, _vp, _vp])
_ext.register_signature("sp24_selftest_bounded_wait", [_vp, _i32, _vp])
_ext.register_signature("sp24_spmm_accumulate_f32", [_vp, _i32, _i32, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64,
                                                     _i32, _vp, _vp])

_ACT = {None: 0, "none": 0, "relu": 1, "silu": 2, "gelu": 3}  # gelu (tanh form) is an addition to the reference's set

# Layout of the (tokens, features) result when the dense operand is token-major.  False (default): a
# contiguous (tokens, features) tensor, written by a transposing epilogue.  True: what the reference
# returns (sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:813-815 of the reference), a transposed view
# of the (features, tokens) product; downstream element-wise ops and the next sparse GEMM accept it as is.
RETURN_TRANSPOSED_VIEW = False
# id(meta tensor) -> (weak reference to it, tensor-core copy, (data_ptr, _version) of the metadata when the copy was
# made); tensors do not hash by value.  An in-place write to the metadata (copy_ on a checkpoint restore, a write
# through another view of the same storage) bumps its version counter, and the copy is then rebuilt on the next use.
_tc_meta_cache = {}
_status = {}


def _status_word(device):
    t = _status.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def check_status(device=None):
    """Synchronises and raises if a bounded on-device wait of the sparse GEMM ever gave up."""
    for dev, t in _status.items():
        if device is None or dev == device:
            code = int(t.item())
            if code:
                t.zero_()
                raise RuntimeError(f"sp24_spmm: an on-device wait gave up (role code {code}) on {dev}")


def invalidate_meta(meta):
    """Drop the cached tensor-core copy of ``meta``.  Only needed by code that rewrites the metadata behind torch's
    back (a raw-pointer kernel launch): writes through torch are seen through the tensor's version counter."""
    _tc_meta_cache.pop(id(meta), None)


def _stamp(meta):
    return (meta.data_ptr(), meta._version)


def tc_bytes(ms: int, k: int) -> int:
    lib = _ext.lib()
    lib.sp24_meta_tc_bytes.restype = _i64
    lib.sp24_meta_tc_bytes.argtypes = [_i64, _i64]
    return lib.sp24_meta_tc_bytes(ms, k)


def register_tc_metadata(meta: torch.Tensor, e_tc: torch.Tensor) -> None:
    """Attach a tensor-core-order copy that a compression kernel wrote together with ``meta``."""
    key = id(meta)
    _tc_meta_cache[key] = (weakref.ref(meta, lambda _r, key=key: _tc_meta_cache.pop(key, None)), e_tc, _stamp(meta))


def tc_metadata(meta: torch.Tensor, ms: int, k: int) -> torch.Tensor:
    """Metadata in the order the tensor cores consume (cached per metadata tensor object)."""
    hit = _tc_meta_cache.get(id(meta))
    e = hit[1] if hit is not None and hit[0]() is meta and hit[2] == _stamp(meta) else None
    if e is None:
        lib = _ext.lib()
        e = torch.empty(tc_bytes(ms, k), dtype=torch.uint8, device=meta.device)
        src = meta if meta.is_contiguous() else meta.contiguous()
        _ext.check(lib.sp24_meta_to_tc(src.data_ptr(), src.element_size(), ms, k, e.data_ptr(), _ext.stream()),
                   "sp24_meta_to_tc")
        register_tc_metadata(meta, e)
    return e


def sparse_linear(input, weight, meta, bias=None, activation=None, alpha=None):
    """``alpha`` (float8 operands only, an addition to the reference's contract): the result is
    alpha * (input @ dense(weight).T) (+ bias) (activation), the dequantisation scale applied in the GEMM epilogue."""
    _ext.require_cuda(input, weight, meta, bias)
    if activation not in _ACT:
        raise RuntimeError(f"_sparse_semi_structured_linear: Invalid activation {activation}")
    if weight.dim() != 2:
        raise RuntimeError(f"_sparse_semi_structured_linear: Expected weight argument to be 2D tensor, got {weight.dim()} dims")
    if input.dtype != weight.dtype:
        raise RuntimeError(f"_sparse_semi_structured_linear: Expected input datatype {weight.dtype}, but got {input.dtype}")
    ms, kh = weight.shape
    k = 2 * kh
    sizes = list(input.shape)
    if sizes[-1] != k:
        raise RuntimeError(f"_sparse_semi_structured_linear: Expected weight argument to have {sizes[-1] // 2} columns, but got {kh}")
    x2 = input.reshape(-1, k)
    n = x2.shape[0]
    lay_a = _ext.layout_of(weight)
    if lay_a is None:
        raise RuntimeError(f"_sparse_semi_structured_linear: Invalid strides for weight argument: row stride = "
                           f"{weight.stride(0)}, column stride = {weight.stride(1)}")
    a_mn, ld_a = lay_a
    lay_b = _ext.layout_of(x2)
    if lay_b is None or x2.data_ptr() % 16 or (lay_b[1] * x2.element_size()) % 16:
        x2 = x2.contiguous()
        lay_b = (0, k)
    # layout_of: 0 = rows contiguous along k (K-major for the GEMM), 1 = k strided (the caller passed B.t())
    b_mn, ld_b = lay_b
    f8 = weight.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
    # fp8 operands give fp32, int8 operands int32 (the reference's table,
    # sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:594-637,729,772), 16-bit operands their own type
    out_dtype = torch.float32 if f8 else (torch.int32 if weight.dtype == torch.int8 else weight.dtype)
    if weight.dtype == torch.int8 and (bias is not None or activation not in (None, "none")):
        raise RuntimeError("_sparse_semi_structured_linear: the int8 GEMM on sm_100a takes no bias and no activation")
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != ms:
            raise RuntimeError(f"_sparse_semi_structured_linear: Expected bias argument to have {ms} elements, but got {bias.numel()}")
        if bias.dtype != out_dtype:
            raise RuntimeError(f"two_four_sgemm_cutlass: Expected spars GTEMM bias datatype {out_dtype}, but got {bias.dtype}")
        bias = bias.contiguous()
    if ms % 128:
        raise RuntimeError("sparse GEMM on sm_100a: number of rows of the sparse matrix must be divisible by 128")
    e_tc = tc_metadata(meta, ms, k)
    status = _status_word(weight.device)
    as_view = b_mn or RETURN_TRANSPOSED_VIEW
    if as_view:
        # D (ms, n) row-major, returned as its transposed view (the caller of mm-with-sparse-first
        # transposes it back, so that result ends up contiguous)
        out = torch.empty((ms, n), dtype=out_dtype, device=weight.device)
        trans_out, ld_out = 0, n
    else:
        out = torch.empty((n, ms), dtype=out_dtype, device=weight.device)
        trans_out, ld_out = 1, ms
    if alpha is not None:
        if not f8 or a_mn or b_mn:
            raise RuntimeError("_sparse_semi_structured_linear: alpha is for float8 operands (both K-major) only")
        rc = _ext.lib().sp24_spmm_scaled(weight.data_ptr(), _ext.dt(weight.dtype), ld_a, e_tc.data_ptr(), ms, k, x2.data_ptr(),
                                         ld_b, n, out.data_ptr(), trans_out, ld_out, _ext.ptr(bias), _ACT[activation],
                                         float(alpha), status.data_ptr(), _ext.stream())
        _ext.check(rc, "sp24_spmm_scaled")
    else:
        rc = _ext.lib().sp24_spmm(weight.data_ptr(), _ext.dt(weight.dtype), a_mn, ld_a, e_tc.data_ptr(), ms, k, x2.data_ptr(),
                                  b_mn, ld_b, n, out.data_ptr(), _ext.dt(out_dtype), trans_out, ld_out, _ext.ptr(bias),
                                  _ACT[activation], status.data_ptr(), _ext.stream())
        _ext.check(rc, "sp24_spmm")
    res = out.t() if as_view else out
    sizes[-1] = ms
    return res.reshape(sizes) if len(sizes) != 2 else res


_EPILOGUE = {"none": 0, "gelu": 1, "dgelu": 2}


def mlp_fusable(weight: torch.Tensor, input: torch.Tensor) -> bool:
    """Whether ``sparse_linear_mlp`` can take this GEMM: 16-bit operands, whole 256-row blocks of the sparse operand."""
    return weight.dtype in (torch.float16, torch.bfloat16) and weight.shape[0] % 256 == 0 and input.dtype == weight.dtype


def sparse_linear_mlp(input, weight, meta, bias=None, epilogue="none", aux=None):
    """``sparse_linear`` with the neighbours of a transformer MLP's GEMMs fused into the epilogue (``sp24_spmm_mlp``).

    ``epilogue``: "none"  -> returns input @ W_s^T + bias; ``bias`` may be float32 (no cast launch);
                  "gelu"  -> returns (gelu(h), h) with h = input @ W_s^T + bias rounded to the operand dtype (tanh
                             form of GELU, evaluated on the rounded h);
                  "dgelu" -> returns (input @ W_s^T) * gelu'(aux), ``aux`` shaped like the result: the input
                             gradient of a layer fed with gelu(aux), as the gradient with respect to aux.
    ``input``: (tokens, k) contiguous, 16-bit; ``weight`` / ``meta``: the compressed (ms, k/2) operand, ms % 256 == 0."""
    _ext.require_cuda(input, weight, meta, bias, aux)
    if epilogue not in _EPILOGUE:
        raise RuntimeError(f"sparse_linear_mlp: unknown epilogue {epilogue}")
    if not mlp_fusable(weight, input):
        raise RuntimeError("sparse_linear_mlp: 16-bit operands of one dtype and sparse rows % 256 == 0 required")
    ms, kh = weight.shape
    k = 2 * kh
    x2 = input.reshape(-1, k)
    if x2.stride(1) != 1 or x2.data_ptr() % 16 or (x2.stride(0) * x2.element_size()) % 16:
        x2 = x2.contiguous()
    n = x2.shape[0]
    lay_a = _ext.layout_of(weight)
    if lay_a is None:
        raise RuntimeError("sparse_linear_mlp: invalid strides for the packed values")
    a_mn, ld_a = lay_a
    bias_f32 = 0
    if bias is not None:
        if bias.dim() != 1 or bias.shape[0] != ms or epilogue == "dgelu":
            raise RuntimeError("sparse_linear_mlp: bias must have one value per output feature (none with dgelu)")
        if bias.dtype == torch.float32:
            bias_f32 = 1
        elif bias.dtype != weight.dtype:
            raise RuntimeError(f"sparse_linear_mlp: bias must be float32 or {weight.dtype}, got {bias.dtype}")
        bias = bias.contiguous()
    out = torch.empty((n, ms), dtype=weight.dtype, device=weight.device)
    if epilogue == "gelu":
        aux = torch.empty((n, ms), dtype=weight.dtype, device=weight.device)
    elif epilogue == "dgelu":
        if aux is None or tuple(aux.shape) != (n, ms) or aux.dtype != weight.dtype or not aux.is_contiguous():
            raise RuntimeError("sparse_linear_mlp: dgelu needs a contiguous aux of the result's shape and dtype")
    e_tc = tc_metadata(meta, ms, k)
    status = _status_word(weight.device)
    rc = _ext.lib().sp24_spmm_mlp(weight.data_ptr(), _ext.dt(weight.dtype), a_mn, ld_a, e_tc.data_ptr(), ms, k, x2.data_ptr(),
                                  x2.stride(0), n, out.data_ptr(), ms, _ext.ptr(bias), bias_f32, _EPILOGUE[epilogue],
                                  _ext.ptr(aux), ms, status.data_ptr(), _ext.stream())
    _ext.check(rc, "sp24_spmm_mlp")
    return (out, aux) if epilogue == "gelu" else out


def sparse_mm_accumulate_(out: torch.Tensor, weight: torch.Tensor, meta: torch.Tensor, dense: torch.Tensor,
                          k_splits: int = 0) -> torch.Tensor:
    """out (ms, n) fp32 += sparse (ms, k) @ dense (k, n).  ``weight`` / ``meta`` are the compressed sparse
    operand (row- or column-major packed values), ``dense`` is row-major.  K is split over idle SMs and the
    partial products are added with fp32 reductions, so ``out`` may already hold a gradient to add to."""
    _ext.require_cuda(out, weight, meta, dense)
    if out.dtype != torch.float32 or out.dim() != 2 or out.stride(1) != 1:
        raise RuntimeError("sparse_mm_accumulate_: out must be a row-major fp32 matrix")
    if weight.dtype not in (torch.float16, torch.bfloat16) or dense.dtype != weight.dtype:
        raise RuntimeError(f"sparse_mm_accumulate_: expected matching fp16 / bf16 operands, got {weight.dtype} and {dense.dtype}")
    ms, kh = weight.shape
    k = 2 * kh
    if dense.dim() != 2 or dense.shape[0] != k:
        raise RuntimeError(f"sparse_mm_accumulate_: dense operand must have {k} rows, got {tuple(dense.shape)}")
    n = dense.shape[1]
    if tuple(out.shape) != (ms, n):
        raise RuntimeError(f"sparse_mm_accumulate_: out must be {(ms, n)}, got {tuple(out.shape)}")
    lay_a = _ext.layout_of(weight)
    if lay_a is None:
        raise RuntimeError("sparse_mm_accumulate_: invalid strides for the packed values")
    a_mn, ld_a = lay_a
    if dense.stride(1) != 1 or dense.data_ptr() % 16 or (dense.stride(0) * dense.element_size()) % 16:
        dense = dense.contiguous()
    e_tc = tc_metadata(meta, ms, k)
    status = _status_word(weight.device)
    rc = _ext.lib().sp24_spmm_accumulate_f32(weight.data_ptr(), _ext.dt(weight.dtype), a_mn, ld_a, e_tc.data_ptr(), ms, k,
                                             dense.data_ptr(), dense.stride(0), n, out.data_ptr(), out.stride(0),
                                             k_splits, status.data_ptr(), _ext.stream())
    _ext.check(rc, "sp24_spmm_accumulate_f32")
    return out
