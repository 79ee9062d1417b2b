"""GPU parity tests: every CUDA kernel, called through the C ABI (ctypes), against the committed
golden fixtures (outputs of the reference's own code) and against the CPU oracle on seeded inputs.
Bit-exact throughout: masks, packed values, metadata, and the float results of MVUE / soft threshold /
masked decay."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from _golden import load, t, same_bits
from oracle import sp24_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def S():
    import sparse
    return sparse


def randn(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def with_ties(x, seed):
    g = torch.Generator().manual_seed(seed)
    x = x.clone()
    m, k = x.shape
    x4 = x.view(m, k // 4, 4)
    sel = torch.rand(m, k // 4, generator=g)
    x4[sel < 0.10, 1] = x4[sel < 0.10, 0]
    x4[(sel >= 0.10) & (sel < 0.15), 3] = -x4[(sel >= 0.10) & (sel < 0.15), 2]
    x4[(sel >= 0.15) & (sel < 0.20)] = 0
    return x


def gpu_compress(dense_cpu, out_dtype, *, col=False, mode=0, mask=None, U=None, seed=0, offset=0):
    """Runs sp24_prune_compress on the logical matrix in the requested storage order; returns CPU
    (packed (m, k/2) contiguous, meta)."""
    from sparse._semi_structured_conversions import prune_compress
    m, k = dense_cpu.shape
    d = dense_cpu.to(DEV)
    if col:
        d = d.t().contiguous().t()
        packed = torch.empty(k // 2, m, dtype=out_dtype, device=DEV).t()
    else:
        packed = torch.empty(m, k // 2, dtype=out_dtype, device=DEV)
    per = 16 if out_dtype in (torch.float16, torch.bfloat16) else 32
    meta = torch.zeros(m, k // per, dtype=torch.int16 if per == 16 else torch.int32, device=DEV)
    prune_compress(d, packed, meta, mode=mode, mask=None if mask is None else mask.to(DEV),
                   uniforms=None if U is None else U.to(DEV), seed=seed, offset=offset)
    torch.cuda.synchronize()
    return packed.contiguous().cpu(), meta.cpu()


# ------------------------------------------------------------------------------------------------
# golden fixtures (reference outputs)
# ------------------------------------------------------------------------------------------------
def test_docstring_known_answer(S):
    a = torch.tensor([0, 0, 1, 1.]).tile((128, 32)).half().to(DEV)
    sp = S.to_sparse_semi_structured(a)
    assert sp.shape == (128, 128) and sp.dtype == torch.float16
    assert bool((sp.values() == 1).all()) and bool((sp.indices() == -4370).all())
    assert sp.indices().dtype == torch.int16 and sp.indices().shape == (128, 8)
    assert torch.equal(sp.to_dense(), a)


@pytest.mark.parametrize("tag,bf", [("f16", False), ("bf16", True), ("i8", False)])
def test_golden_pure_torch_converter(tag, bf):
    g = load(f"from_dense_torch_{tag}")
    dense = t(g["dense"], bf)
    p, me = gpu_compress(dense, dense.dtype)
    assert same_bits(p, t(g["packed"], bf)) and same_bits(me, t(g["meta"]))
    from sparse._semi_structured_conversions import sparse_semi_structured_to_dense
    back = sparse_semi_structured_to_dense(t(g["packed"], bf).to(DEV), t(g["meta"]).to(DEV)).cpu()
    assert same_bits(back, t(g["back"], bf))


@pytest.mark.parametrize("lay", ["row", "col"])
@pytest.mark.parametrize("tag", ["f16_f16", "f32_f16"])
def test_golden_triton_convert(tag, lay):
    g = load(f"k1_mse_{tag}_{lay}")
    p, me = gpu_compress(t(g["dense"]), torch.float16, col=lay == "col")
    assert same_bits(p, t(g["packed"])) and same_bits(me, t(g["meta"]))
    g = load(f"k1_mask_{tag}_{lay}")
    p, me = gpu_compress(t(g["dense"]), torch.float16, col=lay == "col", mode=1, mask=t(g["mask"]))
    assert same_bits(p, t(g["packed"])) and same_bits(me, t(g["meta"]))


@pytest.mark.parametrize("lay", ["row", "col"])
def test_golden_triton_convert_int8(lay):
    g = load(f"k2_mse_i8_{lay}")
    p, me = gpu_compress(t(g["dense"]), torch.int8, col=lay == "col")
    assert same_bits(p, t(g["packed"])) and same_bits(me, t(g["meta"]))


@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_golden_mvue_device_function(S, tag):
    g = load(f"mvue_groups_{tag}")
    x, u = t(g["x"]), t(g["u"])
    out = S.MVUE24_approx_triton(x.to(DEV), uniforms=u.to(DEV)).cpu()
    vals = torch.from_numpy(g["vals"])
    want = torch.where(torch.from_numpy(g["mask"].astype(bool)), vals.to(x.dtype), torch.zeros((), dtype=x.dtype))
    assert same_bits(out, want)


@pytest.mark.parametrize("lay", ["row", "col"])
@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_golden_dense_prune_ops(S, tag, lay):
    for name, fn in (("sparse24", S.sparse24_triton), ("soft_threshold24", S.soft_threshold24_triton)):
        g = load(f"{name}_{tag}_{lay}")
        x = t(g["x"]).to(DEV)
        if lay == "col":
            x = x.t().contiguous().t()
        s, mk = fn(x)
        assert s.stride() == x.stride()
        assert same_bits(s.cpu().contiguous(), t(g["sparse"])) and same_bits(mk.cpu().contiguous(), t(g["mask"]))


def test_golden_dense_prune_ops_bf16(S):
    g = load("soft_threshold24_bf16_legacy")
    x = t(g["x"], True).to(DEV)
    s, mk = S.soft_threshold24_triton(x)
    assert torch.equal(mk.cpu().bool(), t(g["mask"]).bool())
    assert torch.equal(s.cpu().float(), t(g["sparse"], True).float())


@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_golden_transposable_kernel(S, tag):
    g = load(f"transposable_k7_{tag}")
    s, mk = S.mask_select(t(g["x"]).to(DEV))
    assert mk.dtype == torch.bool
    assert torch.equal(mk.cpu(), t(g["mask"])) and same_bits(s.cpu(), t(g["sparse"]))


def test_golden_transposable_legacy(S):
    g = load("transposable_legacy_f16")
    _, mk = S.TransposableSparse(abs=True)(t(g["x"]).to(DEV))
    assert torch.equal(mk.cpu(), t(g["mask"]))


@pytest.mark.parametrize("name", ["masked_add_f32", "masked_add_example"])
def test_golden_masked_add(S, name):
    g = load(name)
    grad = t(g["grad"]).to(DEV)
    S.masked_add_(grad, t(g["p"]).to(DEV), t(g["mask"]).to(DEV), alpha=float(g["alpha"]))
    assert same_bits(grad.cpu(), t(g["out"]))


# ------------------------------------------------------------------------------------------------
# oracle parity on seeded inputs: every dtype pair, both storage orders, all three pruning modes
# ------------------------------------------------------------------------------------------------
IN_DTYPES = [torch.float32, torch.float16, torch.bfloat16]
OUT_DTYPES = [torch.float16, torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2]


@pytest.mark.parametrize("col", [False, True])
@pytest.mark.parametrize("od", OUT_DTYPES)
@pytest.mark.parametrize("idt", IN_DTYPES)
def test_compress_matches_oracle(idt, od, col):
    m, k = 96, 640  # 640 = one full 512-wide tile + a ragged one; 96 = three row groups
    x = with_ties(randn((m, k), 200), 1200).to(idt)
    g = torch.Generator().manual_seed(201)
    pats = torch.tensor([[1, 1, 0, 0], [1, 0, 1, 0], [1, 0, 0, 1], [0, 1, 1, 0], [0, 1, 0, 1], [0, 0, 1, 1]], dtype=torch.bool)
    mask = pats[torch.randint(0, 6, (m, k // 4), generator=g)].reshape(m, k)
    bad = torch.rand(m, k // 4, generator=g) < 0.05
    mask = torch.where(bad.repeat_interleave(4, 1), torch.rand(m, k, generator=g) < 0.5, mask)
    U = torch.rand(m, k, generator=g)
    p, me = gpu_compress(x, od, col=col)
    wp, wm = O.prune_compress(x, od)
    assert same_bits(p, wp) and same_bits(me, wm)
    p, me = gpu_compress(x, od, col=col, mode=1, mask=mask)
    wp, wm = O.prune_compress(x, od, mask=mask)
    assert same_bits(p, wp) and same_bits(me, wm)
    xs = (x.float() * 1e-2).to(idt)
    p, me = gpu_compress(xs, od, col=col, mode=2, U=U)
    wp, wm = O.prune_compress(xs, od, mvue=True, U=U)
    assert same_bits(p, wp) and same_bits(me, wm)
    p, me = gpu_compress(xs, od, col=col, mode=2, seed=0x1234_5678_9ABC, offset=77)
    wp, wm = O.prune_compress(xs, od, mvue=True, seed=0x1234_5678_9ABC, offset=77)
    assert same_bits(p, wp) and same_bits(me, wm)


@pytest.mark.parametrize("shape", [(32, 64), (32, 128), (64, 64), (32, 1088), (2048, 64)])
def test_compress_edge_shapes(shape):
    x = randn(shape, 210).half()
    for col in (False, True):
        p, me = gpu_compress(x, torch.float16, col=col)
        wp, wm = O.prune_compress(x, torch.float16)
        assert same_bits(p, wp) and same_bits(me, wm)


def test_compress_padded_leading_dimension():
    from sparse._semi_structured_conversions import prune_compress
    m, k = 64, 128
    big = randn((m, k + 64), 211).half().to(DEV)
    x = big[:, :k]  # row stride k + 64
    packed = torch.empty(m, k // 2 + 8, dtype=torch.float16, device=DEV)[:, : k // 2]
    meta = torch.empty(m, k // 16, dtype=torch.int16, device=DEV)
    prune_compress(x, packed, meta, mode=0)
    wp, wm = O.prune_compress(x.cpu().contiguous(), torch.float16)
    assert same_bits(packed.cpu().contiguous(), wp) and same_bits(meta.cpu(), wm)


def test_to_sparse_semi_structured_api(S):
    w = randn((128, 256), 220, 0.02).to(DEV)  # fp32 master weight, fp16 compressed copy
    _, mask = S.mask_select(w)
    a = S.to_sparse_semi_structured(w, mask=mask, dtype=torch.float16)
    b = S.to_sparse_semi_structured(w.T, mask=mask.T, dtype=torch.float16)
    assert a.shape == (128, 256) and b.shape == (256, 128)
    assert a.sparse_tensor_cutlass.stride() == (128, 1)
    assert b.sparse_tensor_cutlass.stride() == (1, 256)  # column-major packed, mirrors the W.T view
    wp, wm = O.prune_compress(w.cpu(), torch.float16, mask=mask.cpu())
    assert same_bits(a.values().cpu(), wp) and same_bits(a.indices().cpu(), wm)
    wp, wm = O.prune_compress(w.cpu().t().contiguous(), torch.float16, mask=mask.cpu().t().contiguous())
    assert same_bits(b.values().cpu().contiguous(), wp) and same_bits(b.indices().cpu(), wm)
    want = torch.where(mask.cpu(), w.cpu(), torch.zeros(())).half()
    assert same_bits(a.to_dense().cpu(), want) and same_bits(b.to_dense().cpu(), want.t().contiguous())
    at = a.t()
    assert at.shape == (256, 128) and at.transposed and at.sparse_tensor_cutlass is a.sparse_tensor_cutlass
    with pytest.raises(RuntimeError, match="MVUE24 with mask"):
        S.to_sparse_semi_structured(w, mask=mask, MVUE24=True)
    with pytest.raises(RuntimeError, match="is not supported"):
        S.to_sparse_semi_structured(w[:, :48])
    with pytest.raises(RuntimeError, match="Only CUDA"):
        S.to_sparse_semi_structured(w.cpu())
    with pytest.raises(RuntimeError, match="Only 2d"):
        S.to_sparse_semi_structured(w.view(2, 64, 256))


@pytest.mark.parametrize("col", [False, True])
@pytest.mark.parametrize("dt", IN_DTYPES)
def test_dense_ops_match_oracle(S, dt, col):
    m, k = 160, 264
    x = with_ties(randn((m, k), 230), 1230).to(dt)
    xg = x.to(DEV)
    if col:
        xg = xg.t().contiguous().t()
    s, mk = S.sparse24_triton(xg)
    ws, wm = O.sparse24(x)
    assert same_bits(s.cpu().contiguous(), ws) and same_bits(mk.cpu().contiguous(), wm)
    s, mk = S.soft_threshold24_triton(xg)
    ws, wm = O.soft_threshold24(x)
    assert same_bits(s.cpu().contiguous(), ws) and same_bits(mk.cpu().contiguous(), wm)
    s, mk = S.soft_threshold24_triton(xg, scale=1.37)
    ws, wm = O.soft_threshold24(x, scale=1.37)
    assert same_bits(s.cpu().contiguous(), ws)
    g = torch.Generator().manual_seed(231)
    U = torch.rand(m, k, generator=g)
    out = S.MVUE24_approx_triton(xg, uniforms=U.to(DEV))
    assert same_bits(out.cpu().contiguous(), O.mvue24_dense(x, U=U))
    out = S.MVUE24_approx_triton(xg, seed=99, offset=5, exact=True)
    assert same_bits(out.cpu().contiguous(), O.mvue24_dense(x, seed=99, offset=5))


@pytest.mark.parametrize("dt", IN_DTYPES)
def test_transposable_matches_oracle(S, dt):
    x = randn((96, 192), 240, 0.02).to(dt)
    x.view(-1)[::97] = 0
    x[4:8, 8:12] = x[4, 8]  # a block of equal magnitudes: first pattern must win
    for use_abs in (True, False):
        s, mk = S.TransposableSparse(abs=use_abs)(x.to(DEV))
        ws, wm = O.transposable_sparse(x, abs=use_abs)
        assert torch.equal(mk.cpu(), wm) and same_bits(s.cpu(), ws)


@pytest.mark.parametrize("dt", IN_DTYPES)
@pytest.mark.parametrize("od", [torch.float16, torch.bfloat16])
def test_fused_select_dual_compress(S, dt, od):
    m, k = 128, 320
    w = randn((m, k), 250, 0.02).to(dt)
    mask, (pw, mw), (pt, mt) = S.select_and_compress(w.to(DEV), dtype=od)
    wm = O.transposable_mask(w)
    assert torch.equal(mask.cpu(), wm)
    a, b = O.compress_with_mask(w, wm, od)
    assert same_bits(pw.cpu(), a) and same_bits(mw.cpu(), b)
    a, b = O.compress_with_mask(w.t().contiguous(), wm.t().contiguous(), od)
    assert pt.shape == (k, m // 2) and pt.stride() == (1, k)
    assert same_bits(pt.cpu().contiguous(), a) and same_bits(mt.cpu(), b)
    # reuse of a given mask (no re-selection)
    g = torch.Generator().manual_seed(251)
    w2 = randn((m, k), 252, 0.02).to(dt)
    mask2, (pw2, mw2), (pt2, mt2) = S.select_and_compress(w2.to(DEV), mask=mask, dtype=od)
    a, b = O.compress_with_mask(w2, wm, od)
    assert same_bits(pw2.cpu(), a) and same_bits(mw2.cpu(), b)
    a, b = O.compress_with_mask(w2.t().contiguous(), wm.t().contiguous(), od)
    assert same_bits(pt2.cpu().contiguous(), a) and same_bits(mt2.cpu(), b)


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096 + 5])
@pytest.mark.parametrize("mdt", [torch.bool, torch.float16, torch.float32])
def test_masked_add_matches_oracle(S, n, mdt):
    g = torch.Generator().manual_seed(260 + n)
    grad, p = torch.randn(n, generator=g) * 1e-3, torch.randn(n, generator=g) * 0.02
    mask = (torch.rand(n, generator=g) < 0.5).to(mdt)
    if mdt != torch.bool and n > 2:
        mask[1] = -0.0  # negative zero counts as zero
    gg = grad.to(DEV)
    S.masked_add_(gg, p.to(DEV), mask.to(DEV), alpha=2e-4)
    assert same_bits(gg.cpu(), O.masked_add(grad, p, mask != 0, 2e-4))


def test_masked_add_layouts_and_types(S):
    """Strides must agree (as in the reference); any dense layout the three tensors share works (flat storage
    order); 16-bit gradients and weights go through float32 and are rounded once; gapped storage is refused."""
    a = torch.zeros(8, 8, device=DEV)
    with pytest.raises(AssertionError):
        S.masked_add_(a, a.t(), a.bool(), alpha=0.1)
    g = torch.Generator().manual_seed(12)
    grad, p = torch.randn(48, 80, generator=g).to(DEV), torch.randn(48, 80, generator=g).to(DEV)
    mask = (torch.rand(48, 80, generator=g) < 0.5).to(DEV)
    want = grad + 0.3 * p * (~mask)
    gt = grad.t().contiguous().t()                                   # column-major storage, shared by all three
    S.masked_add_(gt, p.t().contiguous().t(), mask.t().contiguous().t(), alpha=0.3)
    assert torch.allclose(gt, want, atol=1e-6)
    for dt in (torch.float16, torch.bfloat16):
        g16 = grad.to(dt)
        S.masked_add_(g16, p.to(dt), mask, alpha=0.3)
        ref = (grad.to(dt).float() + 0.3 * p.to(dt).float() * (~mask)).to(dt)
        assert g16.dtype == dt and float((g16.float() - ref.float()).abs().max()) <= float(ref.abs().max()) * 2 ** -8
    wide, wide_mask = torch.zeros(8, 16, device=DEV), torch.zeros(8, 16, dtype=torch.bool, device=DEV)
    with pytest.raises(RuntimeError, match="dense layout"):
        S.masked_add_(wide[:, ::2], wide[:, ::2], wide_mask[:, ::2], alpha=0.1)


# ------------------------------------------------------------------------------------------------
# full-size configurations: size-independent properties + spot parity on a slab
# ------------------------------------------------------------------------------------------------
def _two_per_group(mask_bool):
    m, k = mask_bool.shape
    return bool((mask_bool.view(m, k // 4, 4).sum(-1) == 2).all())


def test_config1_roundtrip(S):
    g = torch.Generator().manual_seed(0)
    w = torch.randn(1024, 1024, generator=g).half()
    sp = S.to_sparse_semi_structured(w.to(DEV))
    assert sp.values().shape == (1024, 512) and sp.indices().shape == (1024, 64)
    wp, wm = O.prune_compress(w, torch.float16)
    assert same_bits(sp.values().cpu(), wp) and same_bits(sp.indices().cpu(), wm)
    dense = sp.to_dense().cpu()
    want = torch.where(O.magnitude_mask24(w), w, torch.zeros((), dtype=w.dtype))
    assert same_bits(dense, want)


def test_config2_full_size_properties(S):
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(4096, 4096, generator=g) * 0.02).half().to(DEV)
    mask, (pw, mw), (pt, mt) = S.select_and_compress(w)
    mk4 = mask.view(1024, 4, 1024, 4)
    assert bool((mk4.sum(1) == 2).all()) and bool((mk4.sum(3) == 2).all())
    # the fused kernel equals the three-launch sequence it replaces
    _, mask2 = S.mask_select(w)
    assert torch.equal(mask, mask2)
    a = S.to_sparse_semi_structured(w, mask=mask)
    b = S.to_sparse_semi_structured(w.T, mask=mask.T)
    assert torch.equal(pw, a.values()) and torch.equal(mw, a.indices())
    assert torch.equal(pt, b.values()) and torch.equal(mt, b.indices())
    # round trip
    from sparse._semi_structured_conversions import sparse_semi_structured_to_dense
    want = torch.where(mask, w, torch.zeros((), dtype=w.dtype, device=DEV))
    assert torch.equal(sparse_semi_structured_to_dense(pw, mw), want)
    assert torch.equal(sparse_semi_structured_to_dense(pt.contiguous(), mt), want.t())
    # oracle parity on a 256-row slab (independent 4x4 blocks and row groups make slabs self-contained)
    sl = w[1024:1280].cpu()
    assert torch.equal(mask[1024:1280].cpu(), O.transposable_mask(sl))
    # a transposable mask cannot keep more magnitude than unconstrained row-wise 2:4 pruning, and on
    # Gaussian weights it keeps most of it
    kept = float((sl.float().abs() * mask[1024:1280].cpu()).sum())
    bound = float((sl.float().abs() * O.magnitude_mask24(sl)).sum())
    assert 0.9 * bound < kept <= bound


def test_config3_full_size_properties(S):
    g = torch.Generator().manual_seed(3)
    G = torch.randn(8192, 4096, generator=g) * 1e-3
    pos = torch.randperm(G.numel(), generator=torch.Generator().manual_seed(4))[: G.numel() // 100]
    G.view(-1)[pos] *= 100
    G = G.bfloat16()
    U = torch.rand(8192, 4096, generator=torch.Generator().manual_seed(5))
    Gg, Ug = G.to(DEV), U.to(DEV)
    # MVUE compress, driven by U; parity on a slab, structure on everything
    from sparse._semi_structured_conversions import prune_compress, sparse_semi_structured_to_dense
    packed = torch.empty(8192, 2048, dtype=torch.bfloat16, device=DEV)
    meta = torch.empty(8192, 256, dtype=torch.int16, device=DEV)
    prune_compress(Gg, packed, meta, mode=2, uniforms=Ug)
    dense = sparse_semi_structured_to_dense(packed, meta)
    d_ref = S.MVUE24_approx_triton(Gg, uniforms=Ug)
    assert torch.equal(dense, d_ref)  # compress then expand == dense-shaped MVUE with the same U
    sl = slice(4096, 4096 + 128)
    assert same_bits(d_ref[sl].cpu(), O.mvue24_dense(G[sl], U=U[sl]))
    # unbiasedness over independent seeds, fp32 in/out so that output rounding adds no bias.  With the
    # analytic inclusion probabilities p (oracle), E[out] = x and Var[out] = x^2 (1/p - 1): the signed
    # sum of the errors over a slab and the kept-frequency sum must sit within 6 sigma (within-group
    # correlation bounded by a factor 4 on the variance).
    # Both arithmetic modes are held to it: the exact one and the fast one the training layer uses.
    xs = Gg[:256].float()
    n = 300
    x_cpu = xs.cpu()
    p = torch.from_numpy(O.mvue24_probabilities(x_cpu.reshape(256, -1, 4).numpy())).reshape(x_cpu.shape).double()
    var = (x_cpu.double() ** 2) * (1 / p - 1).clamp_min(0)
    nz = x_cpu != 0
    for exact in (True, False):
        acc = torch.zeros_like(xs)
        freq = torch.zeros_like(xs)
        for i in range(n):
            d = S.MVUE24_approx_triton(xs, seed=1234, offset=i, exact=exact)
            acc += d
            freq += (d != 0).float()
        err = float(((acc.cpu().double() / n) - x_cpu.double()).sum())
        assert abs(err) <= 6 * float((4 * var.sum() / n).sqrt()), (exact, err, float((4 * var.sum() / n).sqrt()))
        ferr = float(((freq.cpu().double() / n) - p)[nz].sum())
        assert abs(ferr) <= 6 * float((4 * (p * (1 - p))[nz].sum() / n).sqrt()), (exact, ferr)
    assert abs(float(p.reshape(-1, 4).sum(-1).mean()) - 2.0) < 1e-3  # two kept per group on average

    # soft threshold: parity on a slab, mask structure everywhere
    s, mk = S.soft_threshold24_triton(Gg)
    assert _two_per_group(mk.bool())
    ws, wm = O.soft_threshold24(G[sl])
    assert same_bits(s[sl].cpu(), ws) and same_bits(mk[sl].cpu(), wm)
    # masked decay with the transposable mask of p itself
    p = (torch.randn(8192, 4096, generator=torch.Generator().manual_seed(6)) * 0.02).to(DEV)
    _, pm = S.mask_select(p)
    grad = Gg.float()
    before = grad.clone()
    S.masked_add_(grad, p, pm, alpha=2e-4)
    assert torch.equal(grad[pm], before[pm])
    assert same_bits(grad[sl].cpu(), O.masked_add(before[sl].cpu(), p[sl].cpu(), pm[sl].cpu(), 2e-4))
    ident = before + (p * 2e-4) * (~pm)
    assert torch.equal(grad, ident)


@pytest.mark.parametrize("col", [False, True])
def test_mvue_fast_mode_tracks_the_exact_arithmetic(S, col):
    """SP24_PRUNE_MVUE_FAST / sp24_mvue24_dense_fast (reciprocal approximations, sums ordered against cancellation,
    7-round Philox with 23-bit uniforms) against a float64 evaluation of the reference formulas on the same
    uniforms.  Stated tolerances: the kept positions agree on at least 99.99 % of the groups (a decision can flip
    only where a uniform falls within float32 rounding of an interval boundary); where both keep a position the
    stored float32 value is within 4e-6 relative of the float64 one (the reference's own float32 operation order
    is up to ~1e-4 off in groups that one magnitude dominates, which is reported, not asserted).  And the
    compressing kernel stores exactly what the dense-shaped kernel writes."""
    from sparse import _ext
    from sparse._semi_structured_conversions import prune_compress, sparse_semi_structured_to_dense
    m, k = 512, 1024
    g = torch.Generator().manual_seed(77)
    x = torch.randn(m, k, generator=g) * 1e-3
    pos = torch.randperm(x.numel(), generator=g)[: x.numel() // 100]
    x.view(-1)[pos] *= 100
    x.view(-1)[::1013] = 0
    xg = x.to(DEV)
    if col:
        xg = xg.t().contiguous().t()
    out = S.MVUE24_approx_triton(xg, seed=4321, offset=9).cpu().contiguous()       # default for seeded calls: fast
    assert torch.equal(out, S.MVUE24_approx_triton(xg, seed=4321, offset=9, exact=False).cpu().contiguous())
    want, wkept = O.mvue24_dense_f64(x, seed=4321, offset=9)
    kept = (out != 0).reshape(m, k // 4, 4)
    zero = (x == 0).reshape(m, k // 4, 4)                                            # kept zeros are not visible
    same_group = ((kept == wkept.reshape(m, k // 4, 4)) | zero).all(-1)
    assert float(same_group.float().mean()) >= 0.9999, float(same_group.float().mean())
    both = (out != 0) & wkept
    rel = ((out.double() - want).abs() / want.abs().clamp_min(1e-300))[both]
    assert float(rel.max()) <= 4e-6, float(rel.max())
    assert int((out != 0).reshape(-1, 4).sum(-1).max()) <= 2
    # bf16: compress with the fast mode, expand, compare with the dense-shaped fast kernel bit for bit
    xb = xg.bfloat16()
    if col:
        packed = torch.empty(k // 2, m, dtype=torch.bfloat16, device=DEV).t()
    else:
        packed = torch.empty(m, k // 2, dtype=torch.bfloat16, device=DEV)
    meta = torch.empty(m, k // 16, dtype=torch.int16, device=DEV)
    prune_compress(xb, packed, meta, mode=_ext.PRUNE_MVUE_FAST, seed=4321, offset=9, emit_tc=False)
    dense = sparse_semi_structured_to_dense(packed.contiguous(), meta)
    assert same_bits(dense.cpu(), S.MVUE24_approx_triton(xb, seed=4321, offset=9, exact=False).cpu().contiguous())
    # the fast mode is seeded only
    U = torch.rand(m, k, device=DEV)
    with pytest.raises(RuntimeError):
        prune_compress(xb, packed, meta, mode=_ext.PRUNE_MVUE_FAST, uniforms=U)
    with pytest.raises(RuntimeError):
        S.MVUE24_approx_triton(xb, uniforms=U, exact=False)


# ------------------------------------------------------------------------------------------------
# degenerate and special-value inputs
# ------------------------------------------------------------------------------------------------
def test_all_zero_and_all_equal_inputs(S):
    z = torch.zeros(64, 128, dtype=torch.float16)
    p, me = gpu_compress(z, torch.float16)
    wp, wm = O.prune_compress(z, torch.float16)
    assert same_bits(p, wp) and same_bits(me, wm) and bool((me == -4370).all())  # ties keep elements 2, 3
    s, mk = S.mask_select(z.to(DEV))
    assert torch.equal(mk.cpu(), O.transposable_mask(z))  # every score ties: the first pattern wins
    blk = mk.cpu().view(16, 4, 32, 4).permute(0, 2, 1, 3)[0, 0]
    assert blk.int().tolist() == [[1, 1, 0, 0], [1, 1, 0, 0], [0, 0, 1, 1], [0, 0, 1, 1]]
    one = torch.full((64, 128), -3.0)
    for fn, ofn in ((S.sparse24_triton, O.sparse24), (S.soft_threshold24_triton, O.soft_threshold24)):
        a, b = fn(one.to(DEV))
        wa, wb = ofn(one)
        assert same_bits(a.cpu(), wa) and same_bits(b.cpu(), wb)


@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
def test_transposable_special_values_match_flat_scan(S, dt):
    """NaN, infinities, negative zeros, huge dynamic range (rounding ties) and small integers (exact ties):
    the hierarchical search must return what the scan over all 90 patterns returns."""
    g = torch.Generator().manual_seed(77)
    x = torch.randn(128, 256, generator=g)
    x[0:32] = torch.randint(0, 3, (32, 256), generator=g).float()              # many exact ties
    x[32:64] = x[32:64].abs() * torch.tensor([1e-6, 1.0, 1e4])[torch.randint(0, 3, (32, 256), generator=g)]
    x[64, 0] = float("nan"); x[68, 5] = float("inf"); x[72, 9] = float("-inf"); x[76:80, 16:20] = float("nan")
    x[80:84, 20:24] = float("inf"); x[84, 24:28] = -0.0
    x = x.to(dt)
    for use_abs in (True, False):
        s, mk = S.TransposableSparse(abs=use_abs)(x.to(DEV))
        assert torch.equal(mk.cpu(), O.transposable_mask(x, abs=use_abs))


def test_large_matrix_round_trip(S):
    """8192 x 8192 bf16 (128 MiB) in both storage orders: structure and round trip."""
    from sparse._semi_structured_conversions import sparse_semi_structured_to_dense
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(8192, 8192, device=DEV, generator=g).bfloat16()
    a = S.to_sparse_semi_structured(x, dtype=torch.bfloat16)
    b = S.to_sparse_semi_structured(x.t(), dtype=torch.bfloat16)      # column-major view, groups along rows of x
    da = a.to_dense()
    assert _two_per_group(da != 0) or bool(((da != 0).view(8192, 2048, 4).sum(-1) <= 2).all())
    keep = (da != 0)
    assert torch.equal(torch.where(keep, x, torch.zeros((), dtype=x.dtype, device=DEV)), da)
    frac = float(da.float().abs().sum()) / float(x.float().abs().sum())
    assert 0.73 < frac < 0.76   # keeping the two largest of four Gaussians keeps ~74.5 % of the L1 mass
    db = sparse_semi_structured_to_dense(b.values().contiguous(), b.indices())
    sl = x[:, :256].t().contiguous().cpu()                                       # first 256 rows of x^T
    wp, wm = O.prune_compress(sl, torch.bfloat16)
    assert same_bits(db[:256].cpu(), O.to_dense(wp, wm))


@pytest.mark.parametrize("n", [4096 * 3, 1001])
def test_fused_masked_decay_adamw_matches_the_two_pass_recipe(S, n):
    """masked_add_ followed by torch.optim.AdamW (the reference recipe) against the one-pass kernel, five steps:
    same parameters and moments to float32 rounding of the differently ordered arithmetic."""
    g = torch.Generator().manual_seed(n)
    p0 = torch.randn(n, generator=g) * 0.02
    mask = (torch.rand(n, generator=g) < 0.5)
    grads = [torch.randn(n, generator=g) * 1e-3 for _ in range(5)]
    lr, betas, eps, wd, alpha = 6e-4, (0.9, 0.95), 1e-8, 0.1, 2e-4
    # reference: two passes
    pr = torch.nn.Parameter(p0.clone().to(DEV))
    opt = torch.optim.AdamW([pr], lr=lr, betas=betas, eps=eps, weight_decay=wd)
    for gr in grads:
        pr.grad = gr.clone().to(DEV)
        S.masked_add_(pr.grad, pr.data, mask.to(DEV), alpha=alpha)
        opt.step()
    # one pass, host step number and device step number
    for dev_step in (False, True):
        p = p0.clone().to(DEV)
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        mk = mask.to(DEV)
        st = torch.zeros(1, device=DEV)
        for i, gr in enumerate(grads):
            gd = gr.clone().to(DEV)
            keep = gd.clone()
            st += 1
            S.adamw_masked_decay_(p, gd, m, v, step=st if dev_step else i + 1, lr=lr, betas=betas, eps=eps, weight_decay=wd,
                                  mask=mk, alpha=alpha)
            assert torch.equal(gd, keep)          # the gradient is read only
        state = opt.state[pr]
        assert torch.allclose(p, pr.data, rtol=2e-5, atol=1e-8)
        assert torch.allclose(m, state["exp_avg"], rtol=2e-5, atol=1e-10)
        assert torch.allclose(v, state["exp_avg_sq"], rtol=2e-5, atol=1e-14)
    # without a mask it is plain AdamW
    p = p0.clone().to(DEV)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    pr2 = torch.nn.Parameter(p0.clone().to(DEV))
    opt2 = torch.optim.AdamW([pr2], lr=lr, betas=betas, eps=eps, weight_decay=wd)
    for i, gr in enumerate(grads):
        pr2.grad = gr.clone().to(DEV)
        opt2.step()
        S.adamw_masked_decay_(p, gr.clone().to(DEV), m, v, step=i + 1, lr=lr, betas=betas, eps=eps, weight_decay=wd)
    assert torch.allclose(p, pr2.data, rtol=2e-5, atol=1e-8)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_adamw_second_gradient_equals_adding_it_first(S, dt):
    """extra_grad: the update with a second gradient on the leading elements is bit-identical to adding that gradient
    (converted to float32) to the first one beforehand."""
    g = torch.Generator().manual_seed(31)
    n, n2 = 4099, 2048
    p0 = (torch.randn(n, generator=g) * 0.02).to(DEV)
    grad = (torch.randn(n, generator=g) * 1e-3).to(DEV)
    extra = (torch.randn(n2, generator=g) * 1e-3).to(dt).to(DEV)
    mask = (torch.rand(n, generator=g) < 0.5).to(DEV)
    kw = dict(step=3, lr=6e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, mask=mask, alpha=2e-4)
    pa, ma, va = p0.clone(), torch.full_like(p0, 1e-4), torch.full_like(p0, 1e-7)
    pb, mb, vb = p0.clone(), ma.clone(), va.clone()
    S.adamw_masked_decay_(pa, grad, ma, va, extra_grad=extra, **kw)
    summed = grad.clone()
    summed[:n2] += extra.float()
    S.adamw_masked_decay_(pb, summed, mb, vb, **kw)
    assert torch.equal(pa, pb) and torch.equal(ma, mb) and torch.equal(va, vb)
    with pytest.raises(RuntimeError):
        S.adamw_masked_decay_(pa, grad, ma, va, extra_grad=extra[:6], **kw)
    if dt != torch.float32:
        # a 16-bit main gradient (what a 16-bit exchange leaves behind) = the same values handed over as float32
        pc, mc, vc = p0.clone(), torch.full_like(p0, 1e-4), torch.full_like(p0, 1e-7)
        pd, md, vd = p0.clone(), mc.clone(), vc.clone()
        S.adamw_masked_decay_(pc, grad.to(dt), mc, vc, extra_grad=extra, **kw)
        S.adamw_masked_decay_(pd, grad.to(dt).float(), md, vd, extra_grad=extra, **kw)
        assert torch.equal(pc, pd) and torch.equal(mc, md) and torch.equal(vc, vd)


def test_prune_compress_random_shapes_match_the_oracle(S):
    """Twenty-four seeded random conversions (shape, dtype pair, storage order, pruning rule): packed values and
    reordered metadata equal the oracle's bit for bit."""
    import random as _r
    from sparse._semi_structured_conversions import prune_compress
    from sparse import _ext
    rng = _r.Random(4242)
    g = torch.Generator().manual_seed(17)
    for case in range(24):
        m = 32 * rng.randint(1, 9)
        k = 64 * rng.randint(1, 9)
        din = rng.choice([torch.float32, torch.float16, torch.bfloat16])
        dout = rng.choice([torch.float16, torch.bfloat16])
        col = rng.random() < 0.5
        mode = rng.choice(["mse", "mask", "mvue"])
        x = (torch.randn(m, k, generator=g) * rng.choice([1e-3, 1.0, 50.0])).to(din)
        xin = x.t().contiguous().t() if col else x
        packed = (torch.empty(k // 2, m, dtype=dout, device=DEV).t() if col else torch.empty(m, k // 2, dtype=dout, device=DEV))
        meta = torch.empty(m, k // 16, dtype=torch.int16, device=DEV)
        kwargs, okw = {}, {}
        if mode == "mask":
            pats = torch.tensor([[1, 1, 0, 0], [1, 0, 1, 0], [1, 0, 0, 1], [0, 1, 1, 0], [0, 1, 0, 1], [0, 0, 1, 1]], dtype=torch.bool)
            mk = pats[torch.randint(0, 6, (m, k // 4), generator=g)].reshape(m, k)
            kwargs["mask"] = (mk.t().contiguous().t() if col else mk).to(DEV)
            okw["mask"] = mk
        if mode == "mvue":
            kwargs["seed"], kwargs["offset"] = 1000 + case, case
            okw.update(mvue=True, seed=1000 + case, offset=case)
        code = {"mse": _ext.PRUNE_MSE, "mask": _ext.PRUNE_MASK, "mvue": _ext.PRUNE_MVUE}[mode]
        prune_compress(xin.to(DEV), packed, meta, mode=code, **kwargs)
        op, om = O.prune_compress(x, dout, **okw)[:2]
        assert same_bits(packed.cpu().contiguous(), op), (case, m, k, din, dout, col, mode)
        assert torch.equal(meta.cpu(), om), (case, m, k, din, dout, col, mode)


@pytest.mark.parametrize("din", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode", ["mse", "mvue"])
def test_row_sums_come_out_of_the_column_major_compress(S, din, mode):
    """The optional row-sum output of the column-major conversion: fp32 sums of the unpruned values added to what
    the buffer held (rtol 1e-5 on sum|x|, the order of the fp32 additions is free), packed values and metadata
    bit-identical to the call without it; row counts that leave the last CTA ragged; row-major input refused."""
    from sparse._semi_structured_conversions import prune_compress
    from sparse import _ext
    g = torch.Generator().manual_seed(91)
    code = {"mse": _ext.PRUNE_MSE, "mvue": _ext.PRUNE_MVUE}[mode]
    for m, k in [(32, 64), (96, 640), (160, 1088), (2048, 64), (736, 4096)]:
        x = torch.randn(k, m, generator=g).to(din).to(DEV).t()         # (m, k) column-major
        outs = []
        for with_sums in (False, True):
            packed = torch.empty(k // 2, m, dtype=torch.float16, device=DEV).t()
            meta = torch.empty(m, k // 16, dtype=torch.int16, device=DEV)
            sums = torch.full((m,), 3.0, dtype=torch.float32, device=DEV) if with_sums else None
            prune_compress(x, packed, meta, mode=code, seed=5, offset=9, row_sums=sums)
            outs.append((packed.clone(), meta.clone(), sums))
        assert torch.equal(outs[0][0].view(torch.int16), outs[1][0].view(torch.int16))
        assert torch.equal(outs[0][1], outs[1][1])
        want = x.double().sum(1) + 3.0
        err = (outs[1][2].double() - want).abs()
        assert bool((err <= 1e-5 * (x.double().abs().sum(1) + 3.0)).all()), (m, k, float(err.max()))
    x = torch.randn(64, 128, generator=g).half().to(DEV)
    with pytest.raises(RuntimeError):
        prune_compress(x, torch.empty(64, 64, dtype=torch.float16, device=DEV),
                       torch.empty(64, 8, dtype=torch.int16, device=DEV), mode=_ext.PRUNE_MSE,
                       row_sums=torch.zeros(64, device=DEV))


# ------------------------------------------------------------------------------------------------
# S-STE forward in one pass: soft threshold (+ frozen scale) fused with the 2:4 compression
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("idt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("odt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("scale", [None, 1.37])
def test_soft_threshold_compress_matches_the_three_pass_sequence(S, idt, odt, scale):
    """sp24_soft_threshold24_compress against the oracle (soft_threshold24, then compress_with_mask with the cast to
    the packed type) and against the kernels it replaces, values and metadata bit for bit; ties included."""
    from sparse.sste import soft_threshold24_compress
    from sparse.spmm import tc_metadata
    m, k = 256, 320
    x = with_ties(randn((m, k), 910), 911).to(idt)
    packed, meta = soft_threshold24_compress(x.to(DEV), scale=scale, dtype=odt)
    ws, wm = O.soft_threshold24(x, scale=scale)
    op, om = O.compress_with_mask(ws, wm != 0, odt)
    assert same_bits(packed.cpu().contiguous(), op) and same_bits(meta.cpu(), om)
    # the sequence the layer used to run: dense-shaped kernel, cast, mask-mode compression
    s3, m3 = S.soft_threshold24_triton(x.to(DEV), scale=scale)
    sp = S.to_sparse_semi_structured(s3.to(odt), mask=m3 != 0, dtype=odt)
    assert same_bits(packed.cpu().contiguous(), sp.sparse_tensor_cutlass.cpu().contiguous())
    assert same_bits(meta.cpu(), sp.meta_tensor_cutlass.cpu())
    # and the tensor-core order written by the same pass equals the converted one
    from sparse import spmm as _spmm
    fused_tc = _spmm._tc_meta_cache[id(meta)][1]
    _spmm.invalidate_meta(meta)
    assert torch.equal(fused_tc, tc_metadata(meta, m, k))


# ------------------------------------------------------------------------------------------------
# trainer kernels around the GEMMs: layer norm and cross entropy (float arithmetic: torch fp32 references)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d", [128, 768, 1024])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16, torch.float16])
def test_layer_norm_kernels_match_torch_fp32(d, odt):
    """sp24_layernorm_fwd / _bwd against F.layer_norm and autograd in float32.  Tolerances: output within one rounding
    of the output type of the fp32 result (1e-5 relative for fp32 out, 2^-8 / 2^-11 for bf16 / fp16); dx, dgamma, dbeta
    within 2e-5 of the largest magnitude for an fp32 dy, 1e-2 / 2e-3 when dy is first rounded to bf16 / fp16."""
    from sparse.train_ops import _layer_norm
    g = torch.Generator().manual_seed(d)
    rows = 1000                                                    # not a multiple of the 8 rows per block
    x = (torch.randn(rows, d, generator=g) * 2 + 0.5).to(DEV).requires_grad_(True)
    w = (torch.randn(d, generator=g) * 0.5 + 1).to(DEV).requires_grad_(True)
    b = torch.randn(d, generator=g).to(DEV).requires_grad_(True)
    dy = torch.randn(rows, d, generator=g).to(DEV)
    y = _layer_norm.apply(x, w, b, 1e-5, odt)
    assert y.dtype == odt and y.shape == x.shape
    y.backward(dy.to(odt))
    got = (y.detach().float(), x.grad.clone(), w.grad.clone(), b.grad.clone())
    x.grad = w.grad = b.grad = None
    ref = F.layer_norm(x, (d,), w, b, 1e-5)
    ref.backward(dy.to(odt).float())
    tol_y = {torch.float32: 1e-5, torch.bfloat16: 2 ** -8, torch.float16: 2 ** -11}[odt]
    assert float((got[0] - ref.detach()).abs().max() / ref.detach().abs().max()) <= tol_y
    tol_g = 2e-5
    for a, r in zip(got[1:], (x.grad, w.grad, b.grad)):
        assert float((a - r).abs().max() / r.abs().max()) <= tol_g, float((a - r).abs().max() / r.abs().max())


def test_layer_norm_module_under_autocast_and_fallback():
    from sparse.train_ops import LayerNorm
    ln = LayerNorm(256).to(DEV)
    x = torch.randn(4, 10, 256, device=DEV)
    assert ln(x).dtype == torch.float32
    with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
        y = ln(x)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    assert float((y.float() - F.layer_norm(x, (256,), ln.weight, ln.bias)).abs().max()) < 0.05
    odd = LayerNorm(100).to(DEV)                                   # not a multiple of 128: the parent's implementation
    z = torch.randn(3, 100, device=DEV)
    assert torch.allclose(odd(z), F.layer_norm(z, (100,), odd.weight, odd.bias), atol=1e-6)


@pytest.mark.parametrize("d,dt", [(768, torch.bfloat16), (256, torch.float16), (1024, torch.float32)])
def test_add_layer_norm_matches_the_separate_ops(d, dt):
    """sp24_add_layernorm_fwd / _bwd: (x + delta, layer_norm(x + delta)) and its backward pass with a gradient arriving
    along the residual stream, against torch in float32 on the same (rounded) inputs.  Tolerances: residual within
    1e-6 relative; normalised output within one rounding of its type; dx within 2e-5 of the largest magnitude, the
    branch gradient within one rounding of its type of dx; dgamma / dbeta within 2e-5."""
    from sparse.train_ops import _add_layer_norm
    g = torch.Generator().manual_seed(d)
    rows = 1003
    x = (torch.randn(rows, d, generator=g) * 2).to(DEV).requires_grad_(True)
    delta = torch.randn(rows, d, generator=g).to(dt).to(DEV).requires_grad_(True)
    w = (torch.randn(d, generator=g) * 0.5 + 1).to(DEV).requires_grad_(True)
    b = torch.randn(d, generator=g).to(DEV).requires_grad_(True)
    dy = torch.randn(rows, d, generator=g).to(dt).to(DEV)
    dres = torch.randn(rows, d, generator=g).to(DEV)
    res, y = _add_layer_norm.apply(x, delta, w, b, 1e-5)
    assert res.dtype == torch.float32 and y.dtype == dt
    torch.autograd.backward([res, y], [dres, dy])
    got = (res.detach(), y.detach().float(), x.grad.clone(), delta.grad.clone(), w.grad.clone(), b.grad.clone())
    assert got[3].dtype == dt
    x.grad = delta.grad = w.grad = b.grad = None
    d32 = delta.detach().float().requires_grad_(True)
    r_ref = x + d32
    y_ref = F.layer_norm(r_ref, (d,), w, b, 1e-5)
    torch.autograd.backward([r_ref, y_ref], [dres, dy.float()])
    tol = {torch.float32: 1e-5, torch.bfloat16: 2 ** -8, torch.float16: 2 ** -11}[dt]
    assert float((got[0] - r_ref.detach()).abs().max() / r_ref.detach().abs().max()) <= 1e-6
    assert float((got[1] - y_ref.detach()).abs().max() / y_ref.detach().abs().max()) <= tol
    assert float((got[2] - x.grad).abs().max() / x.grad.abs().max()) <= 2e-5
    assert float((got[3].float() - d32.grad).abs().max() / d32.grad.abs().max()) <= max(tol, 2e-5)
    for a, r in ((got[4], w.grad), (got[5], b.grad)):
        assert float((a - r).abs().max() / r.abs().max()) <= 2e-5
    # without a gradient along the residual stream (the last norm of a model)
    x.grad = delta.grad = w.grad = b.grad = None
    res, y = _add_layer_norm.apply(x, delta, w, b, 1e-5)
    y.backward(dy)
    want = torch.autograd.grad(F.layer_norm(x + delta.detach().float(), (d,), w, b, 1e-5), x, dy.float())[0]
    assert float((x.grad - want).abs().max() / want.abs().max()) <= 2e-5


def test_layer_norm_affine_gradients_added_into_existing_buffers():
    """accumulate_into_grad: gamma / beta gradients are added by the kernel to the float32 .grad buffers in place (two
    backward passes add up); autograd hands nothing over."""
    from sparse.train_ops import LayerNorm, add_layer_norm
    torch.manual_seed(2)
    a, b = LayerNorm(384).to(DEV), LayerNorm(384).to(DEV)
    b.accumulate_into_grad = True
    b.weight.grad, b.bias.grad = torch.zeros_like(b.weight), torch.zeros_like(b.bias)
    bufs = (b.weight.grad, b.bias.grad)
    x = torch.randn(50, 384, device=DEV)
    delta = torch.randn(50, 384, device=DEV)
    for _ in range(2):
        for ln in (a, b):
            ln(x).square().sum().backward()
            add_layer_norm(x, delta, ln)[1].square().sum().backward()
    assert b.weight.grad is bufs[0] and b.bias.grad is bufs[1]
    assert float((a.weight.grad - b.weight.grad).abs().max() / a.weight.grad.abs().max()) < 1e-5
    assert float((a.bias.grad - b.bias.grad).abs().max() / a.bias.grad.abs().max()) < 1e-5


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_gelu_kernel_matches_torch_fp32(dt):
    """sp24_gelu forward and backward against F.gelu(approximate="tanh") and autograd in float32 on the same 16-bit
    inputs: within one rounding of the output type plus the 2^-11 of tanh.approx (bf16 2^-8, fp16 2^-10 of the largest
    magnitude); an odd element count goes to torch."""
    from sparse.train_ops import gelu
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(257, 3072, generator=g) * 2).to(dt).to(DEV).requires_grad_(True)
    dy = torch.randn(257, 3072, generator=g).to(dt).to(DEV)
    y = gelu(x)
    y.backward(dy)
    x32 = x.detach().float().requires_grad_(True)
    ref = F.gelu(x32, approximate="tanh")
    ref.backward(dy.float())
    tol = {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -10}[dt]
    assert y.dtype == dt and float((y.float() - ref).abs().max() / ref.abs().max()) <= tol
    assert float((x.grad.float() - x32.grad).abs().max() / x32.grad.abs().max()) <= tol
    odd = torch.randn(7, device=DEV).to(dt)
    assert torch.equal(gelu(odd), F.gelu(odd, approximate="tanh"))


def test_token_and_position_embedding_kernels():
    """sp24_embedding_fwd / _bwd against nn.Embedding + autograd: the forward sum is exact; the gradient tables agree to
    float32 summation order (1e-6 of the largest entry), repeated tokens included; into_grad adds into existing buffers."""
    from sparse.train_ops import embed_tokens
    g = torch.Generator().manual_seed(9)
    vocab, t, d, batch = 1000, 48, 192, 6
    wte = torch.randn(vocab, d, generator=g).to(DEV).requires_grad_(True)
    wpe = torch.randn(64, d, generator=g).to(DEV).requires_grad_(True)          # more positions than t
    ids = torch.randint(0, 40, (batch, t), generator=g).to(DEV)                  # few distinct tokens: many collisions
    ids[0, 0] = vocab - 1
    dy = torch.randn(batch, t, d, generator=g).to(DEV)
    out = embed_tokens(ids, wte, wpe)
    ref = F.embedding(ids, wte) + F.embedding(torch.arange(t, device=DEV), wpe)
    assert torch.equal(out, ref)
    out.backward(dy)
    got = (wte.grad.clone(), wpe.grad.clone())
    wte.grad = wpe.grad = None
    ref.backward(dy)
    for a, r in zip(got, (wte.grad, wpe.grad)):
        assert float((a - r).abs().max() / r.abs().max()) < 1e-6
    bufs = (wte.grad, wpe.grad)                                                  # now holding one gradient each
    embed_tokens(ids, wte, wpe, into_grad=True).backward(dy)
    assert wte.grad is bufs[0] and wpe.grad is bufs[1]
    assert float((wte.grad - 2 * got[0]).abs().max() / got[0].abs().max()) < 2e-6
    with pytest.raises(RuntimeError):
        embed_tokens(ids.int(), wte, wpe)
    with pytest.raises(RuntimeError):
        embed_tokens(torch.zeros(2, 65, dtype=torch.long, device=DEV), wte, wpe)


def test_add_layer_norm_wrapper_and_fallback():
    from sparse.train_ops import add_layer_norm, LayerNorm
    ln = LayerNorm(256).to(DEV)
    x = torch.randn(2, 9, 256, device=DEV)
    delta = torch.randn(2, 9, 256, device=DEV)
    res, y = add_layer_norm(x, delta, ln)                          # float32 outside autocast: the kernel
    assert torch.allclose(res, x + delta) and torch.allclose(y, F.layer_norm(x + delta, (256,), ln.weight, ln.bias), atol=1e-5)
    with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
        res, y = add_layer_norm(x, delta.bfloat16(), ln)
        assert res.dtype == torch.float32 and y.dtype == torch.bfloat16
        res2, y2 = add_layer_norm(x, delta, ln)                    # float32 branch under autocast: the separate ops
        assert torch.allclose(res2, x + delta)
    odd = torch.nn.LayerNorm(100).to(DEV)
    z = torch.randn(3, 100, device=DEV)
    r, o = add_layer_norm(z, z, odd)
    assert torch.allclose(r, 2 * z) and torch.allclose(o, odd(2 * z))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,v,fused", [(37, 512, True), (256, 50304, True), (64, 65536, True), (256, 50304, False),
                                          (37, 512, False)])
def test_cross_entropy_fused_gradient_for_unit_upstream(dt, rows, v, fused):
    """loss.backward() directly on the loss (upstream gradient 1): the fused form writes the gradient in its forward
    launch (row staged in shared memory up to 110 KB, re-read beyond: v = 65536); one rounding of the logits' type."""
    from sparse.train_ops import cross_entropy
    g = torch.Generator().manual_seed(rows + v + 1)
    logits = (torch.randn(rows, v, generator=g) * 3).to(dt).to(DEV).requires_grad_(True)
    tgt = torch.randint(0, v, (rows,), generator=g).to(DEV)
    loss = cross_entropy(logits, tgt, fused=fused)
    loss.backward()
    l32 = logits.detach().float().requires_grad_(True)
    ref = F.cross_entropy(l32, tgt)
    ref.backward()
    assert abs(float(loss) - float(ref)) <= 1e-5 * abs(float(ref))
    tol = {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -11}[dt]
    assert float((logits.grad.float() - l32.grad).abs().max() / l32.grad.abs().max()) <= tol
    with torch.no_grad():                                          # no gradient wanted: the forward-only kernel
        assert abs(float(cross_entropy(logits, tgt)) - float(ref)) <= 1e-5 * abs(float(ref))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,v", [(37, 512), (256, 50304)])
def test_cross_entropy_kernels_match_torch_fp32(dt, rows, v):
    """sp24_cross_entropy_fwd / _bwd against F.cross_entropy on the float32 copy of the same 16-bit logits: loss within
    1e-5 relative (float32 summation order), gradient within one rounding of the logits' type of the fp32 gradient
    (2^-8 / 2^-11 of the largest magnitude), including a scaled upstream gradient and a padded row pitch.  The fused
    form rounds twice when the upstream gradient is not 1 (once in the forward launch, once when rescaled): two
    roundings, 2^-7 / 2^-10."""
    from sparse.train_ops import cross_entropy
    g = torch.Generator().manual_seed(rows + v)
    buf = torch.zeros(rows, v + 16, dtype=dt, device=DEV)
    logits = buf[:, :v]                                             # row pitch v + 16
    logits.copy_((torch.randn(rows, v, generator=g) * 3).to(dt))
    logits.requires_grad_(True)
    tgt = torch.randint(0, v, (rows,), generator=g).to(DEV)
    l32 = logits.detach().float().contiguous().requires_grad_(True)
    ref = F.cross_entropy(l32, tgt)
    (ref * 0.37).backward()
    for fused, roundings in ((False, 1), (True, 2)):
        logits.grad = None
        loss = cross_entropy(logits, tgt, fused=fused)
        (loss * 0.37).backward()
        assert abs(float(loss) - float(ref)) <= 1e-5 * abs(float(ref))
        tol = roundings * {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -11}[dt]
        assert float((logits.grad.float() - l32.grad).abs().max() / l32.grad.abs().max()) <= tol
        assert logits.grad.dtype == dt
