"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header declares,
and rejects bad arguments before touching a GPU (argument checks come first in every entry point)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sparse24_b200.h")


@pytest.fixture(scope="module")
def lib():
    from sparse import _ext
    if not os.path.exists(_ext.LIB_PATH):
        import importlib.util
        spec = importlib.util.spec_from_file_location("sp24_build", os.path.join(ROOT, "2by4-pretrain_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return _ext.lib()


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(sp24_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/sparse24_b200.h but not exported"


def test_python_signatures_cover_header(lib):
    from sparse import _ext
    from sparse import spmm  # noqa: F401  (binds the GEMM entry points)
    bound = set(_ext._SIGNATURES) | {"sp24_strerror", "sp24_abi_version", "sp24_meta_tc_bytes", "sp24_spmm_noalloc_max_bytes"}
    assert set(declared_symbols()) <= bound


def test_error_strings(lib):
    assert lib.sp24_strerror(0) == b"ok"
    for code in range(-8, 0):
        assert len(lib.sp24_strerror(code)) > 5
    assert lib.sp24_abi_version() >= 1


def test_bad_arguments_are_rejected_without_a_gpu(lib):
    buf = ctypes.create_string_buffer(1 << 16)
    base = (ctypes.addressof(buf) + 15) & ~15
    p = ctypes.c_void_p(base)
    q = ctypes.c_void_p(base + 4096)
    r = ctypes.c_void_p(base + 8192)
    F32, F16 = 0, 1
    # rows not a multiple of 32
    assert lib.sp24_prune_compress(p, F16, 33, 64, 64, 0, q, F16, 32, r, 0, None, 0, None, 0, 0, 0, None) == -1
    # k not a multiple of 64
    assert lib.sp24_prune_compress(p, F16, 32, 48, 48, 0, q, F16, 24, r, 0, None, 0, None, 0, 0, 0, None) == -1
    # leading dimension smaller than the row
    assert lib.sp24_prune_compress(p, F16, 32, 64, 32, 0, q, F16, 32, r, 0, None, 0, None, 0, 0, 0, None) == -2
    # fp32 packed output does not exist
    assert lib.sp24_prune_compress(p, F16, 32, 64, 64, 0, q, F32, 32, r, 0, None, 0, None, 0, 0, 0, None) == -3
    # misaligned pointer
    assert lib.sp24_prune_compress(ctypes.c_void_p(base + 2), F16, 32, 64, 64, 0, q, F16, 32, r, 0, None, 0, None, 0, 0,
                                   0, None) == -4
    # mask mode without a mask, mask with another mode, null output
    assert lib.sp24_prune_compress(p, F16, 32, 64, 64, 0, q, F16, 32, r, 1, None, 0, None, 0, 0, 0, None) == -5
    assert lib.sp24_prune_compress(p, F16, 32, 64, 64, 0, q, F16, 32, r, 0, r, 64, None, 0, 0, 0, None) == -5
    assert lib.sp24_prune_compress(p, F16, 32, 64, 64, 0, None, F16, 32, r, 0, None, 0, None, 0, 0, 0, None) == -5
    assert lib.sp24_transposable_select(p, F16, 32, 96, 96, 1, None, 0, q, 96, None) == -1
    assert lib.sp24_select_dual_compress(p, F16, 32, 64, 64, 1, q, 64, q, F16, 32, r, q, 64, r, None) == -1
    assert lib.sp24_masked_add(p, q, r, 3, 16, 0.5, None) == -3
    assert lib.sp24_masked_add(p, q, r, 1, 0, 0.5, None) == 0  # empty input is a no-op
    assert lib.sp24_sparse24(p, F16, 32, 12, 12, 0, q, 12, r, 12, None) == -1
    assert lib.sp24_to_dense(p, F32, 32, 64, 32, q, r, 64, None) == -3
    # the newer entry points validate in the same way
    from sparse import spmm  # noqa: F401  (binds the GEMM signatures)
    I8, I32, BF16 = 5, 6, 2
    st = ctypes.c_void_p(base + 12288)
    # sparse GEMM: rows of the sparse operand not a multiple of 128; int8 wants an int32 output and no bias
    assert lib.sp24_spmm(p, F16, 0, 64, q, 64, 128, r, 0, 128, 8, st, F16, 1, 64, None, 0, None, None) == -1
    assert lib.sp24_spmm(p, I8, 0, 64, q, 128, 128, r, 0, 128, 8, st, F32, 1, 128, None, 0, None, None) == -3
    assert lib.sp24_spmm(p, I8, 0, 64, q, 128, 128, r, 0, 128, 8, st, I32, 1, 128, r, 0, None, None) == -5
    # the allocation-free GEMM runs the same checks before it touches its scratch array or the device
    noalloc = lib.sp24_spmm_noalloc
    noalloc.restype = ctypes.c_int
    noalloc.argtypes = lib.sp24_spmm.argtypes
    assert noalloc(p, F16, 0, 64, q, 64, 128, r, 0, 128, 8, st, F16, 1, 64, None, 0, None, None) == -1
    assert noalloc(p, I8, 0, 64, q, 128, 128, r, 0, 128, 8, st, F32, 1, 128, None, 0, None, None) == -3
    assert noalloc(p, F16, 0, 64, q, 128, 128, r, 0, 128, 8, None, F16, 1, 128, None, 0, None, None) == -5
    assert noalloc(p, F16, 0, 64, None, 128, 128, r, 0, 128, 8, st, F16, 1, 128, None, 0, None, None) == -5
    assert noalloc(p, F16, 0, 4096, q, 8192, 8192, r, 0, 8192, 8, st, F16, 1, 8192, None, 0, None, None) == -8
    # accumulating form: fp8 is not accepted, n must keep 16-byte rows
    assert lib.sp24_spmm_accumulate_f32(p, 3, 0, 64, q, 128, 128, r, 8, 8, st, 8, 0, st, None) == -3
    assert lib.sp24_spmm_accumulate_f32(p, BF16, 0, 64, q, 128, 128, r, 12, 12, st, 12, 0, st, None) == -1
    # fused optimizer: null moments, unaligned mask, step 0
    assert lib.sp24_adamw_masked_decay(p, q, None, None, r, 16, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.0, 1.0, None, None) == -5
    assert lib.sp24_adamw_masked_decay(p, q, ctypes.c_void_p(base + 1), r, st, 16, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.0, 1.0, None,
                                       None) == -4
    assert lib.sp24_adamw_masked_decay(p, q, None, r, st, 16, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.0, 0.0, None, None) == -5
    # second gradient: 16- or 32-bit floats, a multiple of four elements, no longer than the range
    assert lib.sp24_adamw_masked_decay_ex(p, q, F32, None, r, st, 16, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.0, 1.0, None, q, 5, 8, None) == -3
    assert lib.sp24_adamw_masked_decay_ex(p, q, F32, None, r, st, 16, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.0, 1.0, None, q, 2, 6, None) == -1
    assert lib.sp24_adamw_masked_decay_ex(p, q, F32, None, r, st, 16, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.0, 1.0, None, q, 2, 32, None) == -1
    assert lib.sp24_adamw_masked_decay_ex(p, q, I8, None, r, st, 16, 1e-3, 0.9, 0.95, 1e-8, 0.0, 0.0, 1.0, None, None, 0, 0, None) == -3
    # tensor-core metadata copies need whole 128-row / 128-column blocks
    assert lib.sp24_select_dual_compress_tc(p, F16, 64, 128, 128, 1, q, 128, q, F16, 64, r, q, 128, r, st, st, None) == -1
    assert lib.sp24_prune_compress_ex(p, F16, 64, 64, 64, 0, q, F16, 32, r, 0, None, 0, None, 0, 0, 0, None, st, None, None) == -5
    # batched select + dual compress: empty batch, descriptors that disagree about the tensor-core copies, bad shape
    from sparse._ext import DualDesc
    descs = (DualDesc * 2)()
    for d in descs:
        d.w, d.m, d.k, d.ld_w, d.mask, d.ld_mask = base, 128, 128, 128, base, 128
        d.packed_w, d.ld_packed_w, d.meta_w, d.packed_t, d.ld_packed_t, d.meta_t = base, 64, base, base, 128, base
    assert lib.sp24_select_dual_compress_batch(descs, 0, F16, F16, 0, None) == -5
    descs[1].tc_w = descs[1].tc_t = base
    assert lib.sp24_select_dual_compress_batch(descs, 2, F16, F16, 0, None) == -5
    descs[1].tc_w = descs[1].tc_t = None
    descs[1].m = 96
    assert lib.sp24_select_dual_compress_batch(descs, 2, F16, F16, 0, None) == -1
    # entry points added for the float8 backward pass, the one-pass S-STE forward and the fused MLP epilogues
    E4M3 = 3
    # q8: float8 outputs only; a quantisation scale must be positive; k a multiple of 128
    assert lib.sp24_prune_compress_q8(p, F16, 32, 128, 128, 0, q, F16, 64, r, 0, None, 0, 1.0, 0, 0, None) == -3
    assert lib.sp24_prune_compress_q8(p, F16, 32, 128, 128, 0, q, E4M3, 64, r, 0, None, 0, 0.0, 0, 0, None) == -5
    assert lib.sp24_prune_compress_q8(p, F16, 32, 64, 64, 1, q, E4M3, 32, r, 0, None, 0, 1.0, 0, 0, None) == -1
    # the fast MVUE mode takes no uniforms; mode codes beyond the public enum are refused
    assert lib.sp24_prune_compress(p, F16, 32, 64, 64, 0, q, F16, 32, r, 3, None, 0, r, 64, 0, 0, None) == -5
    assert lib.sp24_prune_compress(p, F16, 32, 64, 64, 0, q, F16, 32, r, 4, None, 0, None, 0, 0, 0, None) == -5
    assert lib.sp24_mvue24_dense_fast(p, F16, 32, 12, 12, 0, q, 12, 0, 0, None) == -1
    # soft threshold + compress: 16-bit packed types only
    assert lib.sp24_soft_threshold24_compress(p, F32, 32, 64, 64, 0, q, E4M3, 32, r, 0, 0.0, None, None) == -3
    assert lib.sp24_soft_threshold24_compress(p, F32, 33, 64, 64, 0, q, F16, 32, r, 0, 0.0, None, None) == -1
    # scaled float8 GEMM: 16-bit operands are refused; fused MLP epilogues: 16-bit only, dgelu takes no bias, and the
    # second tensor is mandatory
    assert lib.sp24_spmm_scaled(p, F16, 64, q, 128, 128, r, 128, 8, st, 1, 128, None, 0, 1.0, None, None) == -3
    assert lib.sp24_spmm_mlp(p, E4M3, 0, 64, q, 256, 128, r, 128, 8, st, 256, None, 0, 0, None, 0, None, None) == -3
    assert lib.sp24_spmm_mlp(p, F16, 0, 64, q, 256, 128, r, 128, 8, st, 256, r, 0, 2, st, 256, None, None) == -5
    assert lib.sp24_spmm_mlp(p, F16, 0, 64, q, 256, 128, r, 128, 8, st, 256, None, 0, 1, None, 0, None, None) == -5
    assert lib.sp24_spmm_mlp(p, F16, 0, 64, q, 128, 128, r, 128, 8, st, 128, None, 0, 1, st, 128, None, None) == -5
    # row sums exist for column-major storage only
    assert lib.sp24_prune_compress_ex(p, F16, 128, 64, 64, 0, q, F16, 32, r, 0, None, 0, None, 0, 0, 0, None, None, st, None) == -5
    # trainer kernels: row length a multiple of 128 up to 1024; the residual forms want both extra tensors; cross
    # entropy takes 16-bit logits with classes % 8 == 0 and a row pitch that covers them
    assert lib.sp24_layernorm_fwd(p, q, r, st, BF16, st, st, 8, 100, 1e-5, None) == -1
    assert lib.sp24_layernorm_fwd(p, q, r, st, BF16, st, st, 8, 2048, 1e-5, None) == -1
    assert lib.sp24_layernorm_fwd(p, q, r, st, I8, st, st, 8, 128, 1e-5, None) == -3
    assert lib.sp24_add_layernorm_fwd(p, None, st, q, r, st, BF16, st, st, 8, 128, 1e-5, None) == -5
    assert lib.sp24_add_layernorm_fwd(p, q, None, q, r, st, BF16, st, st, 8, 128, 1e-5, None) == -5
    assert lib.sp24_add_layernorm_fwd(p, ctypes.c_void_p(base + 2), st, q, r, st, BF16, st, st, 8, 128, 1e-5, None) == -4
    assert lib.sp24_add_layernorm_bwd(p, BF16, None, q, r, st, st, None, None, st, st, 8, 128, None) == -5
    assert lib.sp24_add_layernorm_bwd(p, BF16, None, q, r, st, st, st, None, st, st, 8, 96, None) == -1
    assert lib.sp24_cross_entropy_fused(p, F32, q, r, st, 1.0, p, 4, 64, 64, 64, None) == -3
    assert lib.sp24_cross_entropy_fused(p, BF16, q, r, st, 1.0, p, 4, 60, 64, 64, None) == -1
    assert lib.sp24_cross_entropy_fused(p, BF16, q, r, st, 1.0, p, 4, 64, 32, 64, None) == -2
    assert lib.sp24_cross_entropy_fused(p, BF16, q, r, st, 1.0, None, 4, 64, 64, 64, None) == -5
    assert lib.sp24_scale_unless_one(p, BF16, None, 64, None) == -5
    assert lib.sp24_scale_unless_one(p, BF16, q, 60, None) == -1
    # peer memory: a handle is the 64 bytes of a cudaIpcMemHandle_t
    out_ptr = ctypes.c_void_p()
    assert lib.sp24_ipc_open(None, 64, ctypes.byref(out_ptr)) == -5
    assert lib.sp24_ipc_open(p, 63, ctypes.byref(out_ptr)) == -5
    assert lib.sp24_ipc_close(None) == -5
    assert lib.sp24_gelu(p, None, q, F32, 64, None) == -3
    assert lib.sp24_gelu(p, None, q, BF16, 60, None) == -1
    assert lib.sp24_gelu(p, None, None, BF16, 64, None) == -5
    assert lib.sp24_embedding_fwd(p, q, r, st, 8, 4, 30, 100, None) == -1
    assert lib.sp24_embedding_fwd(p, q, r, None, 8, 4, 32, 100, None) == -5
    assert lib.sp24_embedding_bwd(p, q, ctypes.c_void_p(base + 4), st, 8, 4, 32, 100, None) == -4


def test_missing_library_fails_loudly(monkeypatch):
    from sparse import _ext
    monkeypatch.setattr(_ext, "_lib", None)
    monkeypatch.setattr(_ext, "LIB_PATH", "/nonexistent/libsparse24_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or Triton fallback"):
        _ext.lib()
