"""Regenerates the golden fixtures in this folder from the reference project's own code.

Run where a checkout of the reference project is available (its path in REFERENCE_ROOT), no GPU needed:

    REFERENCE_ROOT=<checkout of huyz2023/2by4-pretrain> TRITON_INTERPRET=1 python tests/golden/make_golden.py

What is executed is the reference, not this repository:
  * its pure-PyTorch converter ``_sparse_semi_structured_from_dense`` /
    ``_sparse_semi_structured_to_dense`` (sparse/_semi_structured_conversions.py:10-328);
  * its Triton kernels, run on CPU tensors by the Triton interpreter (the
    autotuned ones through ``kernel.fn[grid]`` with a fixed BLOCK_SIZE);
  * its ``legacy.py`` torch functions where the interpreter cannot be trusted
    (bf16 stores) or would be too slow.
MVUE has no entry point taking uniforms in the reference, so a small harness
kernel defined here loads x and u and calls the reference's own
``utils._MVUE24_approx`` device function.

The reference package cannot be imported as ``sparse`` (its native extension is
not built), so its modules are loaded by path under the alias ``_ref_sparse``.
Outputs: one ``.npz`` per case (bf16 / int16 payloads stored as raw integer bits).
"""
import importlib
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(os.path.join(REF, "sparse")):
    raise SystemExit("make_golden.py: set REFERENCE_ROOT to a checkout of the reference project (the folder holding sparse/)")
HERE = os.path.dirname(os.path.abspath(__file__))


def load_ref():
    pkg = types.ModuleType("_ref_sparse")
    pkg.__path__ = [os.path.join(REF, "sparse")]
    sys.modules["_ref_sparse"] = pkg
    mods = {}
    for name in ("_semi_structured_conversions", "utils", "triton_ops", "decay",
                 "transposable_semi_structured", "legacy"):
        mods[name] = importlib.import_module(f"_ref_sparse.{name}")
    return mods


R = load_ref()
conv = R["_semi_structured_conversions"]


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as a numpy integer / float array."""
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    if t.dtype == torch.bool:
        return t.numpy()
    return t.numpy()


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    print("wrote", name, {k: (v.shape, str(v.dtype)) for k, v in arrays.items()})


def randn(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def with_ties(x: torch.Tensor, seed: int) -> torch.Tensor:
    """Plant equal magnitudes, zeros and sign flips so that tie-breaking is exercised."""
    g = torch.Generator().manual_seed(seed)
    x = x.clone()
    m, k = x.shape
    x4 = x.view(m, k // 4, 4)
    sel = torch.rand(m, k // 4, generator=g)
    x4[sel < 0.10, 1] = x4[sel < 0.10, 0]
    x4[(sel >= 0.10) & (sel < 0.15), 3] = -x4[(sel >= 0.10) & (sel < 0.15), 2]
    x4[(sel >= 0.15) & (sel < 0.20)] = 0
    x4[(sel >= 0.20) & (sel < 0.23)] = x4[(sel >= 0.20) & (sel < 0.23), 0:1]
    return x


# ---------------------------------------------------------------------------
# 1. pure-PyTorch converter (magnitude pruning) and its inverse
# ---------------------------------------------------------------------------
def case_from_dense_torch():
    for tag, dtype, shape, seed in (("f16", torch.float16, (64, 128), 100),
                                    ("bf16", torch.bfloat16, (96, 192), 101),
                                    ("i8", torch.int8, (32, 128), 102)):
        if dtype == torch.int8:
            g = torch.Generator().manual_seed(seed)
            x = torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)
        else:
            x = with_ties(randn(shape, seed), seed + 1000).to(dtype)
        packed, meta = conv._sparse_semi_structured_from_dense(x)
        back = conv._sparse_semi_structured_to_dense(packed, meta)
        save(f"from_dense_torch_{tag}", dense=bits(x), packed=bits(packed), meta=bits(meta), back=bits(back))


# ---------------------------------------------------------------------------
# 2. Triton conversion kernels under the interpreter
# ---------------------------------------------------------------------------
def run_k1(dense, out_dtype, prune, mask=None, col=False, block=8):
    """Launch the reference conversion kernel the way its launcher does
    (sparse/_semi_structured_conversions.py:1072-1125) but with a fixed BLOCK_SIZE."""
    m, k = dense.shape
    is8 = out_dtype in (torch.int8,)
    width = 32 if is8 else 16
    meta_dtype = torch.int32 if is8 else torch.int16
    if col:
        dense = dense.t().contiguous().t()  # column-major storage of the same logical matrix
        packed = torch.empty(k // 2, m, dtype=out_dtype).t()
        if mask is not None:
            mask = mask.t().contiguous().t()
    else:
        packed = torch.empty(m, k // 2, dtype=out_dtype)
    meta = torch.zeros(m, k // width, dtype=meta_dtype)
    layout = "col" if col else "row"
    grid = (triton.cdiv(m, block), k // width) if col else (m, triton.cdiv(k, width * block))
    kern = conv._sparse_semi_structured_from_dense_triton_8 if is8 else conv._sparse_semi_structured_from_dense_triton_16
    kern.fn[grid](dense, packed, meta, mask,
                  dense.stride(0), packed.stride(0), mask.stride(0) if mask is not None else None,
                  dense.stride(1), packed.stride(1), mask.stride(1) if mask is not None else None,
                  m, k, 1234, BLOCK_SIZE=block, PRUNE=prune, ARRAY_LAYOUT=layout)
    return packed.contiguous(), meta


def case_triton_convert():
    x16 = with_ties(randn((64, 128), 110), 1110).half()
    x32 = with_ties(randn((64, 128), 111), 1111)
    g = torch.Generator().manual_seed(112)
    # masks: valid 2:4 patterns plus a few groups with 0, 1, 3 and 4 set bits (fall-back encodings)
    mask = conv_mask_random((64, 128), g)
    for tag, x, od in (("f16_f16", x16, torch.float16), ("f32_f16", x32, torch.float16)):
        for col in (False, True):
            lay = "col" if col else "row"
            p, me = run_k1(x, od, "mse", col=col)
            save(f"k1_mse_{tag}_{lay}", dense=bits(x), packed=bits(p), meta=bits(me))
            p, me = run_k1(x, od, "mask", mask=mask, col=col)
            save(f"k1_mask_{tag}_{lay}", dense=bits(x), mask=bits(mask), packed=bits(p), meta=bits(me))
    g = torch.Generator().manual_seed(113)
    xi = torch.randint(-127, 128, (32, 256), generator=g, dtype=torch.int8)
    for col in (False, True):
        p, me = run_k1(xi, torch.int8, "mse", col=col)
        save(f"k2_mse_i8_{'col' if col else 'row'}", dense=bits(xi), packed=bits(p), meta=bits(me))


def conv_mask_random(shape, g):
    m, k = shape
    pats = torch.tensor([[1, 1, 0, 0], [1, 0, 1, 0], [1, 0, 0, 1], [0, 1, 1, 0], [0, 1, 0, 1], [0, 0, 1, 1]],
                        dtype=torch.bool)
    idx = torch.randint(0, 6, (m, k // 4), generator=g)
    mask = pats[idx]
    odd = torch.rand(m, k // 4, generator=g) < 0.08
    anyp = torch.rand(m, k // 4, 4, generator=g) < 0.5
    mask = torch.where(odd.unsqueeze(-1), anyp, mask)
    return mask.reshape(m, k).contiguous()


# ---------------------------------------------------------------------------
# 3. MVUE through the reference's own device function, with supplied uniforms
# ---------------------------------------------------------------------------
_MVUE = R["utils"]._MVUE24_approx


@triton.jit
def _mvue_harness(x_ptr, u_ptr, v_ptr, m_ptr, n_groups, BLOCK: tl.constexpr):
    g = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    ok = g < n_groups
    x0 = tl.load(x_ptr + g * 4 + 0, mask=ok)
    x1 = tl.load(x_ptr + g * 4 + 1, mask=ok)
    x2 = tl.load(x_ptr + g * 4 + 2, mask=ok)
    x3 = tl.load(x_ptr + g * 4 + 3, mask=ok)
    u0 = tl.load(u_ptr + g * 4 + 0, mask=ok)
    u1 = tl.load(u_ptr + g * 4 + 1, mask=ok)
    a0, a1, a2, a3, m0, m1, m2, m3 = _MVUE(x0, x1, x2, x3, u0, u1)
    tl.store(v_ptr + g * 4 + 0, a0, mask=ok)
    tl.store(v_ptr + g * 4 + 1, a1, mask=ok)
    tl.store(v_ptr + g * 4 + 2, a2, mask=ok)
    tl.store(v_ptr + g * 4 + 3, a3, mask=ok)
    tl.store(m_ptr + g * 4 + 0, m0.to(tl.int8), mask=ok)
    tl.store(m_ptr + g * 4 + 1, m1.to(tl.int8), mask=ok)
    tl.store(m_ptr + g * 4 + 2, m2.to(tl.int8), mask=ok)
    tl.store(m_ptr + g * 4 + 3, m3.to(tl.int8), mask=ok)


def case_mvue():
    g = torch.Generator().manual_seed(120)
    for tag, dtype in (("f16", torch.float16), ("f32", torch.float32)):
        shape = (64, 256)
        x = randn(shape, 121, 1e-3)
        big = torch.rand(shape, generator=g) < 0.02
        x = torch.where(big, x * 100, x)
        x.view(-1, 4)[:16] = 0  # all-zero groups
        x = x.to(dtype)
        u = torch.rand(shape, generator=g)
        u.view(-1, 4)[16:24, 1] = 0.0  # u1 == 0: second pick can coincide with the first
        u.view(-1, 4)[24:32, 0] = 0.0
        n_groups = x.numel() // 4
        vals = torch.zeros(shape, dtype=torch.float32)
        msk = torch.zeros(shape, dtype=torch.int8)
        _mvue_harness[(triton.cdiv(n_groups, 256),)](x, u, vals, msk, n_groups, BLOCK=256)
        save(f"mvue_groups_{tag}", x=bits(x), u=bits(u), vals=bits(vals), mask=bits(msk))


# ---------------------------------------------------------------------------
# 4. dense-shaped prune ops
# ---------------------------------------------------------------------------
def run_dense_op(kernel, x, col=False):
    m, k = x.shape
    if col:
        x = x.t().contiguous().t()
    sparse = torch.zeros_like(x)
    mask = torch.zeros_like(x)
    block = 64
    grid = (triton.cdiv(m, block), k // 4) if col else (m, triton.cdiv(k, 4 * block))
    kernel[grid](x, sparse, mask, x.stride(0), sparse.stride(0), mask.stride(0),
                 x.stride(1), sparse.stride(1), mask.stride(1), m, k,
                 BLOCK_SIZE=block, ARRAY_LAYOUT="col" if col else "row")
    return sparse.contiguous(), mask.contiguous()


def case_dense_ops():
    ops = R["triton_ops"]
    leg = R["legacy"]
    for tag, dtype in (("f16", torch.float16), ("f32", torch.float32)):
        x = with_ties(randn((32, 256), 130), 1130).to(dtype)
        for col in (False, True):
            lay = "col" if col else "row"
            s, mk = run_dense_op(ops._sparse24_triton, x, col)
            save(f"sparse24_{tag}_{lay}", x=bits(x), sparse=bits(s), mask=bits(mk))
            s, mk = run_dense_op(ops._soft_threshold24_triton, x, col)
            save(f"soft_threshold24_{tag}_{lay}", x=bits(x), sparse=bits(s), mask=bits(mk))
    # bf16: the interpreter truncates bf16 stores, so the reference's torch implementation is used.
    # Random values without planted ties (argsort's tie order is not the kernels' tie order).
    x = randn((32, 256), 131).bfloat16()
    s, mk = leg.soft_threshold24_torch(x)
    save("soft_threshold24_bf16_legacy", x=bits(x), sparse=bits(s), mask=mk.numpy().astype(np.int8))
    s, mk = leg.sparse24_torch(x)
    save("sparse24_bf16_legacy", x=bits(x), sparse=bits(s), mask=mk.numpy().astype(np.int8))


# ---------------------------------------------------------------------------
# 5. transposable mask select
# ---------------------------------------------------------------------------
def case_transposable():
    ts = R["transposable_semi_structured"]
    leg = R["legacy"]
    mod = ts.TransposableSparse(abs=True)
    for tag, dtype, scale in (("f16", torch.float16, 0.02), ("f32", torch.float32, 0.02)):
        x = randn((64, 128), 140, scale).to(dtype)
        pat = mod.mask_pattern.to(x)
        m, k = x.shape
        sparse = torch.zeros_like(x)
        mask = torch.zeros_like(x, dtype=torch.bool)
        ts._to_transposable_sparse_semi_structured_kernel[(m // 32, k // 64)](
            x, sparse, pat, mask, x.stride(0), x.stride(1), sparse.stride(0), sparse.stride(1),
            pat.stride(0), pat.stride(1), mask.stride(0), mask.stride(1), m, k, 90, 1,
            num_warps=4, BLOCK_SIZE=128)
        save(f"transposable_k7_{tag}", x=bits(x), sparse=bits(sparse), mask=bits(mask))
    save("transposable_patterns", patterns=mod.mask_pattern.numpy().astype(np.uint8))
    x = randn((256, 256), 141, 0.02).half()
    s, mk = leg.transposable_sparse(x.float(), abs=True)
    save("transposable_legacy_f16", x=bits(x), mask=mk.bool().numpy())


# ---------------------------------------------------------------------------
# 6. masked decay
# ---------------------------------------------------------------------------
def case_masked_add():
    dec = R["decay"]
    n = 5000  # not a multiple of the block size
    g = torch.Generator().manual_seed(150)
    grad = torch.randn(n, generator=g) * 1e-3
    p = torch.randn(n, generator=g) * 0.02
    mask = torch.rand(n, generator=g) < 0.5
    out = grad.clone()
    dec.masked_add_kernel[(triton.cdiv(n, 1024),)](out, p, mask, n, 2e-4, BLOCK_SIZE=1024)
    save("masked_add_f32", grad=bits(grad), p=bits(p), mask=bits(mask), out=bits(out), alpha=np.float64(2e-4))
    # the reference's own four-element example (sparse/decay.py:41-45)
    grad = torch.tensor([1., 1., 1., 1.])
    p = torch.tensor([1., 2., 3., 4.])
    mask = torch.tensor([1., 0., 1., 0.])
    out = grad.clone()
    dec.masked_add_kernel[(1,)](out, p, mask, 4, 0.03, BLOCK_SIZE=1024)
    save("masked_add_example", grad=bits(grad), p=bits(p), mask=bits(mask), out=bits(out), alpha=np.float64(0.03))


if __name__ == "__main__":
    only = sys.argv[1:]
    cases = dict(from_dense_torch=case_from_dense_torch, triton_convert=case_triton_convert, mvue=case_mvue,
                 dense_ops=case_dense_ops, transposable=case_transposable, masked_add=case_masked_add)
    for name, fn in cases.items():
        if not only or name in only:
            fn()
