"""CPU tests: the oracle restatement against fixtures produced by the reference's own code
(tests/golden/make_golden.py) and against the known answers the reference states."""
import numpy as np
import pytest
import torch

from oracle import sp24_oracle as O
from _golden import load, t, same_bits


def test_docstring_known_answer():
    # sparse/semi_structured.py:603-627 of the reference: values all 1, metadata all -4370
    a = torch.tensor([0, 0, 1, 1.]).tile((128, 32)).half()
    packed, meta = O.prune_compress(a, torch.float16)
    assert packed.shape == (128, 64) and meta.shape == (128, 8) and meta.dtype == torch.int16
    assert bool((packed == 1).all()) and bool((meta == -4370).all())


def test_encoding_truth_table():
    # sparse/_semi_structured_conversions.py:46-71 of the reference
    table = {(1, 1, 0, 0): 0b0100, (1, 0, 1, 0): 0b1000, (0, 1, 1, 0): 0b1001, (1, 0, 0, 1): 0b1100,
             (0, 1, 0, 1): 0b1101, (0, 0, 1, 1): 0b1110,
             (0, 0, 0, 0): 0b1110, (0, 0, 0, 1): 0b1110, (0, 0, 1, 0): 0b1110, (0, 1, 0, 0): 0b1101,
             (0, 1, 1, 1): 0b1001, (1, 0, 0, 0): 0b1100, (1, 0, 1, 1): 0b1000, (1, 1, 0, 1): 0b0100,
             (1, 1, 1, 0): 0b1000, (1, 1, 1, 1): 0b1000}
    for bits, code in table.items():
        _, _, nib = O.encode_mask_groups(torch.tensor(bits, dtype=torch.bool).view(1, 4))
        assert int(nib) == code, bits


def test_readme_masked_add_identity():
    # README.md:108 of the reference: masked_add_ == grad.add_(p * (1 - mask), alpha=decay)
    g = torch.Generator().manual_seed(0)
    grad, p = torch.randn(4096, generator=g), torch.randn(4096, generator=g)
    mask = torch.rand(4096, generator=g) < 0.5
    want = grad.clone().add_(p * (1 - mask.float()), alpha=2e-4)
    got = O.masked_add(grad, p, mask, 2e-4)
    kept = mask
    assert torch.equal(got[kept], grad[kept])
    assert torch.allclose(got, want, rtol=0, atol=1e-7)


@pytest.mark.parametrize("tag,bf", [("f16", False), ("bf16", True), ("i8", False)])
def test_pure_torch_converter(tag, bf):
    g = load(f"from_dense_torch_{tag}")
    dense, packed, meta = t(g["dense"], bf), t(g["packed"], bf), t(g["meta"])
    if tag == "i8":
        mk = O.magnitude_mask24(dense)
        p, me = O.compress_with_mask(dense, mk, torch.int8)
    else:
        p, me = O.prune_compress(dense, dense.dtype)
    assert same_bits(p, packed) and same_bits(me, meta)
    assert same_bits(O.to_dense(packed, meta), t(g["back"], bf))


@pytest.mark.parametrize("lay", ["row", "col"])
@pytest.mark.parametrize("tag", ["f16_f16", "f32_f16"])
def test_triton_convert_kernels(tag, lay):
    g = load(f"k1_mse_{tag}_{lay}")
    p, me = O.prune_compress(t(g["dense"]), torch.float16)
    assert same_bits(p, t(g["packed"])) and same_bits(me, t(g["meta"]))
    g = load(f"k1_mask_{tag}_{lay}")
    p, me = O.prune_compress(t(g["dense"]), torch.float16, mask=t(g["mask"]))
    assert same_bits(p, t(g["packed"])) and same_bits(me, t(g["meta"]))


@pytest.mark.parametrize("lay", ["row", "col"])
def test_triton_convert_int8(lay):
    g = load(f"k2_mse_i8_{lay}")
    dense = t(g["dense"])
    p, me = O.compress_with_mask(dense, O.magnitude_mask24(dense), torch.int8)
    assert same_bits(p, t(g["packed"])) and same_bits(me, t(g["meta"]))


@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_mvue_device_function(tag):
    g = load(f"mvue_groups_{tag}")
    x, u = t(g["x"]), t(g["u"])
    u0, u1 = O._uniform_pairs_from_tensor(u)
    m, k = x.shape
    vals, mask = O.mvue24_groups(x.float().reshape(m, k // 4, 4).numpy(), u0, u1)
    assert np.array_equal(mask.reshape(m, k), g["mask"].astype(bool))
    assert np.array_equal(vals.reshape(m, k).view(np.int32), g["vals"].view(np.int32))
    # exactly two kept unless the second draw coincides with the first (u1 == 0 rows)
    cnt = mask.sum(-1)
    assert set(np.unique(cnt)) <= {1, 2}


@pytest.mark.parametrize("lay", ["row", "col"])
@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_dense_prune_ops(tag, lay):
    g = load(f"sparse24_{tag}_{lay}")
    s, mk = O.sparse24(t(g["x"]))
    assert same_bits(s, t(g["sparse"])) and same_bits(mk, t(g["mask"]))
    g = load(f"soft_threshold24_{tag}_{lay}")
    s, mk = O.soft_threshold24(t(g["x"]))
    assert same_bits(s, t(g["sparse"])) and same_bits(mk, t(g["mask"]))


def test_dense_prune_ops_bf16_legacy():
    g = load("soft_threshold24_bf16_legacy")
    x = t(g["x"], True)
    s, mk = O.soft_threshold24(x)
    want = t(g["sparse"], True)
    assert torch.equal(mk.bool(), t(g["mask"]).bool())
    assert torch.equal(s.float(), want.float())  # the legacy function leaves -0 at pruned slots
    g = load("sparse24_bf16_legacy")
    s, mk = O.sparse24(x)
    assert torch.equal(mk.bool(), t(g["mask"]).bool()) and torch.equal(s.float(), t(g["sparse"], True).float())


def test_transposable_patterns_table():
    assert np.array_equal(O.transposable_patterns(), load("transposable_patterns")["patterns"])


@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_transposable_kernel(tag):
    g = load(f"transposable_k7_{tag}")
    s, mk = O.transposable_sparse(t(g["x"]))
    assert torch.equal(mk, t(g["mask"])) and same_bits(s, t(g["sparse"]))


def test_transposable_legacy():
    g = load("transposable_legacy_f16")
    assert torch.equal(O.transposable_mask(t(g["x"])), t(g["mask"]))
    mk = t(g["mask"]).view(64, 4, 64, 4)
    assert bool((mk.sum(1) == 2).all()) and bool((mk.sum(3) == 2).all())


@pytest.mark.parametrize("name", ["masked_add_f32", "masked_add_example"])
def test_masked_add(name):
    g = load(name)
    out = O.masked_add(t(g["grad"]), t(g["p"]), t(g["mask"]), float(g["alpha"]))
    assert same_bits(out, t(g["out"]))


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    z = np.zeros(1, np.uint32)
    assert [int(v[0]) for v in O.philox4x32_10(z, 0, 0, 0, 0, 0)] == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    f = 0xffffffff
    assert [int(v[0]) for v in O.philox4x32_10(z + f, f, f, f, f, f)] == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]


def test_mvue_unbiased_with_own_stream():
    # mean over many independent draws approaches x: |mean - x| within 5 sigma of the estimator
    x = torch.tensor([[0.5, -0.25, 0.125, 1.0] * 16] * 32)
    acc = torch.zeros_like(x)
    n = 400
    sq = torch.zeros_like(x)
    for i in range(n):
        d = O.mvue24_dense(x, seed=7, offset=i)
        acc += d
        sq += d * d
    mean = acc / n
    var = (sq / n - mean * mean).clamp_min(0)
    # average over the 512 identical groups as well
    gm = mean.view(-1, 4).mean(0)
    gv = var.view(-1, 4).mean(0) / (n * 512)
    assert bool(((gm - x.view(-1, 4)[0]).abs() <= 5 * gv.sqrt() + 1e-6).all())
