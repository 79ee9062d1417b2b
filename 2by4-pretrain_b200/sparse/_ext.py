"""Loader of the C-ABI kernel library (``lib/libsparse24_b200.so``) and thin ctypes call helpers.

The Python layer never computes on the CPU: if the library is missing every op raises, it does
not fall back.  Tensors are passed as raw device pointers plus sizes; the current torch CUDA
stream is passed as the stream handle, so calls are asynchronous like any torch op.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libsparse24_b200.so")

F32, F16, BF16, E4M3, E5M2, I8, I32 = 0, 1, 2, 3, 4, 5, 6
PRUNE_MSE, PRUNE_MASK, PRUNE_MVUE, PRUNE_MVUE_FAST = 0, 1, 2, 3

_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int8: I8, torch.int32: I32}
if hasattr(torch, "float8_e4m3fn"):
    _DT[torch.float8_e4m3fn] = E4M3
    _DT[torch.float8_e5m2] = E5M2

_lib = None

_i64, _i32, _u64, _vp, _f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_float

class DualDesc(ctypes.Structure):
    """``sp24_dual_desc`` of the C header: one matrix of a batched select + dual compress call."""
    _fields_ = [("w", _vp), ("m", _i64), ("k", _i64), ("ld_w", _i64), ("mask", _vp), ("ld_mask", _i64),
                ("packed_w", _vp), ("ld_packed_w", _i64), ("meta_w", _vp), ("packed_t", _vp), ("ld_packed_t", _i64),
                ("meta_t", _vp), ("tc_w", _vp), ("tc_t", _vp)]


_SIGNATURES = {
    "sp24_prune_compress": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i32, _i64, _vp, _i32, _vp, _i64, _vp, _i64,
                            _u64, _u64, _vp],
    "sp24_prune_compress_ex": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i32, _i64, _vp, _i32, _vp, _i64, _vp, _i64,
                               _u64, _u64, _vp, _vp, _vp, _vp],
    "sp24_prune_compress_q8": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i32, _i64, _vp, _i32, _vp, _i64, _f32, _u64, _u64, _vp],
    "sp24_soft_threshold24_compress": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i32, _i64, _vp, _i32, _f32, _vp, _vp],
    "sp24_layernorm_fwd": [_vp, _vp, _vp, _vp, _i32, _vp, _vp, _i64, _i64, _f32, _vp],
    "sp24_layernorm_bwd": [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp],
    "sp24_add_layernorm_fwd": [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i64, _i64, _f32, _vp],
    "sp24_add_layernorm_bwd": [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp],
    "sp24_cross_entropy_fwd": [_vp, _i32, _vp, _vp, _vp, _i64, _i64, _i64, _vp],
    "sp24_cross_entropy_bwd": [_vp, _i32, _vp, _vp, _vp, _f32, _vp, _i64, _i64, _i64, _i64, _vp],
    "sp24_adamw_masked_decay": [_vp, _vp, _vp, _vp, _vp, _i64, _f32, _f32, _f32, _f32, _f32, _f32, _f32, _vp, _vp],
    "sp24_adamw_masked_decay_ex": [_vp, _vp, _i32, _vp, _vp, _vp, _i64, _f32, _f32, _f32, _f32, _f32, _f32, _f32, _vp, _vp, _i32,
                                   _i64, _vp],
    "sp24_to_dense": [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _i64, _vp],
    "sp24_mvue24_dense": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _i64, _u64, _u64, _vp],
    "sp24_mvue24_dense_fast": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i64, _u64, _u64, _vp],
    "sp24_sparse24": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _i64, _vp],
    "sp24_soft_threshold24": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _i64, _i32, _f32, _vp],
    "sp24_transposable_select": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _i64, _vp],
    "sp24_select_dual_compress": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _i32, _i64, _vp, _vp, _i64,
                                  _vp, _vp],
    "sp24_select_dual_compress_tc": [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _i64, _vp, _i32, _i64, _vp, _vp, _i64,
                                     _vp, _vp, _vp, _vp],
    "sp24_select_dual_compress_batch": [ctypes.POINTER(DualDesc), _i32, _i32, _i32, _i32, _vp],
    "sp24_masked_add": [_vp, _vp, _vp, _i32, _i64, _f32, _vp],
    "sp24_cross_entropy_fused": [_vp, _i32, _vp, _vp, _vp, _f32, _vp, _i64, _i64, _i64, _i64, _vp],
    "sp24_scale_unless_one": [_vp, _i32, _vp, _i64, _vp],
    "sp24_gelu": [_vp, _vp, _vp, _i32, _i64, _vp],
    "sp24_ipc_open": [_vp, _i32, ctypes.POINTER(ctypes.c_void_p)],
    "sp24_ipc_close": [_vp],
    "sp24_embedding_fwd": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp],
    "sp24_embedding_bwd": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp],
}


def lib():
    """The loaded library; raises RuntimeError (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"sparse24_b200 kernel library not found at {LIB_PATH}; build it with "
                f"`python {os.path.join(os.path.dirname(_HERE), 'build.py')}` (needs nvcc). "
                "There is no CPU or Triton fallback.")
        h = ctypes.CDLL(LIB_PATH)
        h.sp24_strerror.restype = ctypes.c_char_p
        h.sp24_strerror.argtypes = [_i32]
        h.sp24_abi_version.restype = _i32
        h.sp24_meta_tc_bytes.restype = _i64
        h.sp24_meta_tc_bytes.argtypes = [_i64, _i64]
        for name, args in _SIGNATURES.items():
            fn = getattr(h, name, None)
            if fn is not None:
                fn.restype = _i32
                fn.argtypes = args
        _lib = h
    return _lib


def register_signature(name, argtypes):
    """Used by modules that bind further entry points (e.g. the sparse GEMM)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = _i32
        fn.argtypes = argtypes


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what}: {lib().sp24_strerror(rc).decode()} (code {rc})")


def dt(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise RuntimeError(f"Datatype {dtype} is not supported!") from None


def stream() -> int:
    """Raw handle of the current CUDA stream of the current device."""
    try:
        return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())
    except AttributeError:  # older / newer torch without the private fast path
        return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return 0 if t is None else t.data_ptr()


def require_cuda(*tensors):
    """Every tensor (``None`` entries skipped) must be a CUDA tensor on the CURRENT device: the kernels run on the
    current device's current stream and dereference raw addresses, so a tensor of another GPU would be an illegal
    address on the device instead of a Python error.  Select the device first (``torch.cuda.device(t.device)``)."""
    current = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"Error tensor.device= {t.device} is not supported! Only CUDA tensors are currently supported.")
        if current is None:
            current = torch.cuda.current_device()
        if t.device.index != current:
            raise RuntimeError(f"tensor on {t.device} but the current CUDA device is cuda:{current}: the sparse24 kernels "
                               "launch on the current device; wrap the call in torch.cuda.device(tensor.device)")


def layout_of(t: torch.Tensor):
    """(col_major, leading dimension) of a 2-D tensor with one unit stride, or None."""
    rs, cs = t.stride()
    m, k = t.shape
    if cs == 1 and (rs >= k or m == 1):
        return 0, max(rs, k)
    if rs == 1 and (cs >= m or k == 1):
        return 1, max(cs, m)
    return None


def as_layout(t: torch.Tensor, col_major: int) -> torch.Tensor:
    """Same logical matrix stored densely in the requested order (no copy when already so)."""
    lay = layout_of(t)
    if lay is not None and lay[0] == col_major and t.data_ptr() % 16 == 0 and (lay[1] * t.element_size()) % 16 == 0:
        return t
    return t.contiguous() if not col_major else t.t().contiguous().t()
