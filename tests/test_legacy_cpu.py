"""CPU tests of the plain-torch compatibility functions (sparse/legacy.py) against the oracle, on inputs
without ties (ties are broken by torch.argsort there, by position in the kernels)."""
import numpy as np
import torch

from oracle import sp24_oracle as O


def _no_ties(shape, seed):
    g = torch.Generator().manual_seed(seed)
    n = int(np.prod(shape))
    mag = (torch.randperm(n, generator=g).float() + 1.0) / 64.0          # distinct, exactly representable
    sign = torch.where(torch.rand(n, generator=g) < 0.5, -1.0, 1.0)
    return (mag * sign).reshape(shape)


def test_names_are_exported_like_the_reference_package():
    import sparse
    for name in ("sparse24_torch", "soft_threshold24_torch", "MVUE24_approx_torch"):
        assert callable(getattr(sparse, name))


def test_sparse24_and_soft_threshold_match_the_oracle():
    from sparse.legacy import sparse24_torch, soft_threshold24_torch
    x = _no_ties((64, 128), 3)
    got, mask = sparse24_torch(x)
    want, wmask = O.sparse24(x)
    assert torch.equal(got, want) and torch.equal(mask.bool(), wmask.bool()) and mask.dtype == torch.int32
    got, mask = soft_threshold24_torch(x)
    want, wmask = O.soft_threshold24(x)
    assert torch.equal(got, want.to(got.dtype)) and torch.equal(mask.bool(), wmask.bool())


def test_transposable_sparse_matches_the_oracle_when_sums_are_exact():
    from sparse.legacy import transposable_sparse
    x = _no_ties((32, 64), 5)            # multiples of 1/64 below 64: every 8-term sum is exact in fp32
    got, mask = transposable_sparse(x)
    want = O.transposable_mask(x)
    assert torch.equal(mask.bool(), want)
    assert torch.equal(got, torch.where(want, x, torch.zeros(())))
    blocks = mask.reshape(8, 4, 16, 4)
    assert bool((blocks.sum(1) == 2).all()) and bool((blocks.sum(3) == 2).all())


def test_mvue_approx_is_two_of_four_and_unbiased():
    from sparse.legacy import MVUE24_approx_torch
    torch.manual_seed(11)
    x = torch.tensor([[0.5, -1.0, 2.0, 0.25]]).repeat(20000, 1)
    y = MVUE24_approx_torch(x)
    assert bool(((y != 0).sum(1) == 2).all())
    p = torch.from_numpy(O.mvue24_probabilities(x[:1].numpy()))[0]
    # kept entries are x_i / p_i, so every column's mean estimates x_i
    assert torch.allclose(y.mean(0), x[0], rtol=0.05, atol=0.02)
    kept = y[:, 2][y[:, 2] != 0]
    assert torch.allclose(kept, (x[0, 2] / p[2]).expand_as(kept), rtol=1e-5)
