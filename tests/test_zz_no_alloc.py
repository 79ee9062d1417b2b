"""GPU test of ``sp24_spmm_noalloc``, the sparse-GEMM entry point for callers that cannot allocate
device memory at call time (hosts replaying a fixed memory plan, loops that must not touch the
allocator, plug-ins inside an application that owns the GPU's memory).

It is driven through the C ABI with ctypes and compared with the regular entry point ``sp24_spmm``,
which gets its tensor-core metadata scratch from the caller.  Both run the same kernel, so the outputs
must be identical bit for bit.  Calls in a row with different problems (16-bit, fp8 and int8 operands)
check that what one call left in the library's fixed scratch array does not leak into the next.  The
file name sorts last so that a run stopping at the first failure has already exercised every other
test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

OUT_OF = {torch.float16: torch.float16, torch.bfloat16: torch.bfloat16, torch.float8_e4m3fn: torch.float32,
          torch.float8_e5m2: torch.float32, torch.int8: torch.int32}


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
    if dtype == torch.int8:
        w = torch.randint(-128, 128, (ms, k), generator=g, dtype=torch.int32).to(torch.int8).to(DEV)
        x = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int32).to(torch.int8).to(DEV)
        sp = sparse.to_sparse_semi_structured(w, dtype=dtype)
    elif dtype in (torch.float16, torch.bfloat16):
        w = torch.randn(ms, k, generator=g).to(dtype).to(DEV)
        x = torch.randn(n, k, generator=g).to(dtype).to(DEV)
        sp = sparse.to_sparse_semi_structured(w, dtype=dtype)
    else:
        w = torch.randn(ms, k, generator=g).to(DEV)
        x = torch.randn(n, k, generator=g).to(DEV).to(dtype)
        sp = sparse.to_sparse_semi_structured(w, dtype=dtype)
    return sp.sparse_tensor_cutlass, sp.meta_tensor_cutlass, x, sp


def _free_bytes():
    return torch.cuda.mem_get_info(torch.device(DEV))[0]


def _run_both(lib, _ext, packed, meta, x, trans_out):
    ms, kh = packed.shape
    k, n = 2 * kh, x.shape[0]
    dt = _ext.dt(packed.dtype)
    out_dtype = OUT_OF[packed.dtype]
    odt = _ext.dt(out_dtype)
    fill = float("nan") if out_dtype.is_floating_point else -7
    stream = torch.cuda.current_stream().cuda_stream
    shape = (n, ms) if trans_out else (ms, n)
    ld_out = ms if trans_out else n
    # regular entry point: the caller allocates the scratch and fills it with sp24_meta_to_tc
    e_tc = torch.empty(lib.sp24_meta_tc_bytes(ms, k), dtype=torch.uint8, device=DEV)
    assert lib.sp24_meta_to_tc(meta.data_ptr(), meta.element_size(), ms, k, e_tc.data_ptr(), stream) == 0
    ref = torch.full(shape, fill, dtype=out_dtype, device=DEV)
    rc = lib.sp24_spmm(packed.data_ptr(), dt, 0, kh, e_tc.data_ptr(), ms, k, x.data_ptr(), 0, k, n, ref.data_ptr(), odt,
                       trans_out, ld_out, None, 0, None, stream)
    assert rc == 0
    # the entry point under test: no scratch argument.  Two things are watched around the call: torch's own
    # allocator, and the device's free memory as the driver reports it (which also sees allocations made behind
    # torch's back; the slack covers what other processes on the device may do meanwhile)
    out = torch.full(shape, fill, dtype=out_dtype, device=DEV)
    torch.cuda.synchronize()
    before, free_before = torch.cuda.memory_allocated(), _free_bytes()
    rc = lib.sp24_spmm_noalloc(packed.data_ptr(), dt, 0, kh, meta.data_ptr(), ms, k, x.data_ptr(), 0, k, n,
                               out.data_ptr(), odt, trans_out, ld_out, None, 0, None, stream)
    assert rc == 0
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    return out, ref, free_before - _free_bytes()


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    lib, _ext = _bind()
    assert lib.sp24_spmm_noalloc_max_bytes() == 4 << 20
    # first call: a problem with ragged K (832 = 6.5 metadata atoms) and ragged N
    packed, meta, x, sp = _problem(384, 832, 200, torch.float16, 1)
    out, ref, _ = _run_both(lib, _ext, packed, meta, x, trans_out=1)   # first call on the device: module load, set-up
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    dense = sp.to_dense().float()
    assert float((out.float() - x.float() @ dense.t()).abs().max() / (x.float() @ dense.t()).abs().max()) < 1e-3
    # second call right after it: smaller, different data and layout; stale scratch contents must not matter
    packed, meta, x, sp = _problem(128, 256, 64, torch.bfloat16, 2)
    out, ref, taken = _run_both(lib, _ext, packed, meta, x, trans_out=0)
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    dense = sp.to_dense().float()
    assert float((out.float() - dense @ x.float().t()).abs().max() / (dense @ x.float().t()).abs().max()) < 8e-3
    assert taken < (2 << 20), f"device free memory dropped by {taken} bytes across a steady-state call"


def test_noalloc_eight_bit_operands_after_a_sixteen_bit_call():
    """fp8 and int8 operands carry 32-bit metadata words; the scratch array still holds the 16-bit atoms of the
    call before.  e4m3: bit-equal to sp24_spmm and within 1e-5 of the fp32 product of the dequantised operands;
    int8: equal to the int64 matmul."""
    lib, _ext = _bind()
    packed, meta, x, sp = _problem(256, 512, 96, torch.float16, 3)
    _run_both(lib, _ext, packed, meta, x, trans_out=1)
    packed, meta, x, sp = _problem(256, 896, 208, torch.float8_e4m3fn, 4)
    assert meta.dtype == torch.int32
    out, ref, _ = _run_both(lib, _ext, packed, meta, x, trans_out=1)
    assert torch.equal(out.view(torch.int32), ref.view(torch.int32))
    want = x.float() @ sp.to_dense().float().t()
    assert float((out - want).abs().max() / want.abs().max()) <= 1e-5
    packed, meta, x, sp = _problem(384, 1024, 72, torch.int8, 5)
    assert meta.dtype == torch.int32
    for trans_out in (1, 0):
        out, ref, _ = _run_both(lib, _ext, packed, meta, x, trans_out=trans_out)
        assert torch.equal(out, ref)
        want = x.cpu().long() @ sp.to_dense().cpu().long().t()
        assert torch.equal(out.cpu().long(), want if trans_out else want.t())


def test_noalloc_rejects_problems_beyond_the_fixed_scratch():
    lib, _ext = _bind()
    dummy = torch.zeros(64, dtype=torch.float16, device=DEV)
    p = dummy.data_ptr()
    # 8192 x 8192 needs 8 MiB of tensor-core metadata: more than the 4 MiB array
    rc = lib.sp24_spmm_noalloc(p, 1, 0, 4096, p, 8192, 8192, p, 0, 8192, 8, p, 1, 1, 8192, None, 0, None, None)
    assert rc == -8
    assert b"capacity" in lib.sp24_strerror(rc)


def test_noalloc_refuses_what_sp24_spmm_refuses():
    """Every argument check of sp24_spmm runs before the metadata conversion into the shared array, so a refused
    call launches nothing (the CPU suite shows the same codes coming back on a machine without a GPU)."""
    lib, _ext = _bind()
    p2, m2, x2, _ = _problem(256, 512, 64, torch.float16, 7)
    out = torch.empty(64, 256, dtype=torch.float16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    # null output, output pitch that breaks the 16-byte rule, unknown activation, fp16 operands with an fp32 output
    assert lib.sp24_spmm_noalloc(p2.data_ptr(), 1, 0, 256, m2.data_ptr(), 256, 512, x2.data_ptr(), 0, 512, 64, None, 1, 1, 256,
                                 None, 0, None, st) == -5
    assert lib.sp24_spmm_noalloc(p2.data_ptr(), 1, 0, 256, m2.data_ptr(), 256, 512, x2.data_ptr(), 0, 512, 64, out.data_ptr(), 1,
                                 1, 100, None, 0, None, st) == -2
    assert lib.sp24_spmm_noalloc(p2.data_ptr(), 1, 0, 256, m2.data_ptr(), 256, 512, x2.data_ptr(), 0, 512, 64, out.data_ptr(), 1,
                                 1, 256, None, 9, None, st) == -5
    assert lib.sp24_spmm_noalloc(p2.data_ptr(), 1, 0, 256, m2.data_ptr(), 256, 512, x2.data_ptr(), 0, 512, 64, out.data_ptr(), 0,
                                 1, 256, None, 0, None, st) == -3
    torch.cuda.synchronize()
