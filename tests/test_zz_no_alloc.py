"""GPU test of ``sp24_spmm_noalloc``, the sparse-GEMM entry point for callers that cannot allocate
device memory at call time (hosts replaying a fixed memory plan, loops that must not touch the
allocator, plug-ins inside an application that owns the GPU's memory).

It is driven through the C ABI with ctypes and compared with the regular entry point ``sp24_spmm``,
which gets its tensor-core metadata scratch from the caller.  Both run the same kernel, so the outputs
must be identical bit for bit.  Two calls in a row with different problems check that what the first
call left in the library's fixed scratch array does not leak into the second.  The file name sorts
last so that a run stopping at the first failure has already exercised every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bind():
    from sparse import _ext, spmm  # noqa: F401  (spmm binds sp24_spmm / sp24_meta_to_tc)
    lib = _ext.lib()
    i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
    lib.sp24_spmm_noalloc.restype = i32
    lib.sp24_spmm_noalloc.argtypes = [vp, i32, i32, i64, vp, i64, i64, vp, i32, i64, i64, vp, i32, i32, i64, vp, i32, vp, vp]
    lib.sp24_spmm_noalloc_max_bytes.restype = i64
    lib.sp24_spmm_noalloc_max_bytes.argtypes = []
    return lib, _ext


def _problem(ms, k, n, dtype, seed):
    import sparse
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(ms, k, generator=g).to(dtype).to(DEV)
    x = torch.randn(n, k, generator=g).to(dtype).to(DEV)
    sp = sparse.to_sparse_semi_structured(w, dtype=dtype)
    return sp.sparse_tensor_cutlass, sp.meta_tensor_cutlass, x, sp


def _run_both(lib, _ext, packed, meta, x, trans_out):
    ms, kh = packed.shape
    k, n = 2 * kh, x.shape[0]
    dt = _ext.dt(packed.dtype)
    stream = torch.cuda.current_stream().cuda_stream
    shape = (n, ms) if trans_out else (ms, n)
    ld_out = ms if trans_out else n
    # regular entry point: the caller allocates the scratch and fills it with sp24_meta_to_tc
    e_tc = torch.empty(lib.sp24_meta_tc_bytes(ms, k), dtype=torch.uint8, device=DEV)
    assert lib.sp24_meta_to_tc(meta.data_ptr(), 2, ms, k, e_tc.data_ptr(), stream) == 0
    ref = torch.full(shape, float("nan"), dtype=packed.dtype, device=DEV)
    rc = lib.sp24_spmm(packed.data_ptr(), dt, 0, kh, e_tc.data_ptr(), ms, k, x.data_ptr(), 0, k, n, ref.data_ptr(), dt,
                       trans_out, ld_out, None, 0, None, stream)
    assert rc == 0
    # the entry point under test: no scratch argument, nothing allocated between here and the launch
    out = torch.full(shape, float("nan"), dtype=packed.dtype, device=DEV)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = lib.sp24_spmm_noalloc(packed.data_ptr(), dt, 0, kh, meta.data_ptr(), ms, k, x.data_ptr(), 0, k, n,
                               out.data_ptr(), dt, trans_out, ld_out, None, 0, None, stream)
    assert rc == 0
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    return out, ref


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    lib, _ext = _bind()
    assert lib.sp24_spmm_noalloc_max_bytes() == 4 << 20
    # first call: a problem with ragged K (832 = 6.5 metadata atoms) and ragged N
    packed, meta, x, sp = _problem(384, 832, 200, torch.float16, 1)
    out, ref = _run_both(lib, _ext, packed, meta, x, trans_out=1)
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    dense = sp.to_dense().float()
    assert float((out.float() - x.float() @ dense.t()).abs().max() / (x.float() @ dense.t()).abs().max()) < 1e-3
    # second call right after it: smaller, different data and layout; stale scratch contents must not matter
    packed, meta, x, sp = _problem(128, 256, 64, torch.bfloat16, 2)
    out, ref = _run_both(lib, _ext, packed, meta, x, trans_out=0)
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    dense = sp.to_dense().float()
    assert float((out.float() - dense @ x.float().t()).abs().max() / (dense @ x.float().t()).abs().max()) < 8e-3


def test_noalloc_rejects_problems_beyond_the_fixed_scratch():
    lib, _ext = _bind()
    dummy = torch.zeros(64, dtype=torch.float16, device=DEV)
    p = dummy.data_ptr()
    # 8192 x 8192 needs 8 MiB of tensor-core metadata: more than the 4 MiB array
    rc = lib.sp24_spmm_noalloc(p, 1, 0, 4096, p, 8192, 8192, p, 0, 8192, 8, p, 1, 1, 8192, None, 0, None, None)
    assert rc == -8
    assert b"capacity" in lib.sp24_strerror(rc)
