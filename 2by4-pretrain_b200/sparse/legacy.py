"""Plain-torch formulations kept for API compatibility (sparse/legacy.py of the reference).

The reference exports ``sparse24_torch``, ``soft_threshold24_torch`` and ``MVUE24_approx_torch`` from its
package (sparse/__init__.py:1) and keeps a matmul-based ``transposable_sparse`` beside them
(sparse/legacy.py:271-354).  None of them is on the training path: they are the slow formulations the
kernels were derived from, useful for cross-checks on any device.  They are written here with ordinary torch
operators on whatever device the argument lives on; the training path uses the CUDA kernels behind
``sparse24_triton``, ``soft_threshold24_triton``, ``MVUE24_approx_triton`` and ``TransposableSparse``.

Differences a caller may see against the kernels: groups of four are taken over the flattened tensor
(= along the last dimension of a contiguous tensor), ties are broken by ``torch.argsort`` (unspecified order)
instead of by position, masks are int32 tensors, and ``MVUE24_approx_torch`` draws from torch's global
generator with ``torch.multinomial``.
"""
import itertools

import torch

_PAIRS = [(0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3)]


def _keep_two_largest(magnitude: torch.Tensor):
    """(groups, 4) magnitudes -> (int32 keep mask, argsort indices ascending)."""
    order = torch.argsort(magnitude, dim=1)
    keep = torch.ones(magnitude.shape, device=magnitude.device, dtype=torch.int)
    keep.scatter_(1, order[:, :2], 0)
    return keep, order


def sparse24_torch(weight: torch.Tensor):
    """Magnitude 2:4 pruning (sparse/legacy.py:26-38): returns (weight * mask, mask)."""
    keep, _ = _keep_two_largest(weight.abs().reshape(-1, 4))
    keep = keep.reshape(weight.shape)
    return weight * keep, keep


def soft_threshold24_torch(weight: torch.Tensor):
    """S-STE soft threshold (sparse/legacy.py:96-114): the second-smallest magnitude of each group is
    subtracted from the two kept magnitudes, signs restored; returns (pruned, mask)."""
    magnitude = weight.detach().abs().reshape(-1, 4)
    keep, order = _keep_two_largest(magnitude)
    threshold = torch.gather(magnitude, 1, order[:, 1:2])
    shrunk = (magnitude - threshold).reshape(weight.shape)
    keep = keep.reshape(weight.shape)
    return torch.sign(weight) * shrunk * keep, keep


def MVUE24_approx_torch(weight: torch.Tensor):
    """Approximate minimum-variance unbiased 2:4 estimator (sparse/legacy.py:227-268): two positions per
    group sampled without replacement with probability proportional to |x| + eps, the survivors divided by
    their inclusion probability."""
    eps = 1.19209e-07
    shape = weight.shape
    x = weight.reshape(-1, 4)
    sign = torch.sign(x)
    a = x.abs() + eps
    first = a / a.sum(dim=1, keepdim=True)             # P(position drawn first)
    inclusion = first.clone()
    for j in range(4):
        rest = a.clone()
        rest[:, j] = 0
        inclusion = inclusion + first[:, j:j + 1] * rest / rest.sum(dim=1, keepdim=True)
    pool = a.clone()
    pool.scatter_(1, torch.multinomial(pool, 1), 0)
    pool.scatter_(1, torch.multinomial(pool, 1), 0)
    kept = a - pool                                    # the two drawn magnitudes, zero elsewhere
    return (kept / inclusion * sign).view(shape)


def _transposable_table(device) -> torch.Tensor:
    """(90, 16) float32: the 4x4 0/1 matrices with two ones in every row and column, in descending
    lexicographic order of the row-major bit string (the order of the reference's table, so that argmax ties
    fall on the same pattern)."""
    rows = [tuple(1 if j in p else 0 for j in range(4)) for p in _PAIRS]
    table = [sum(r, ()) for r in itertools.product(rows, repeat=4)
             if all(sum(row[j] for row in r) == 2 for j in range(4))]
    table.sort(reverse=True)
    return torch.tensor(table, dtype=torch.float32, device=device)


def transposable_sparse(weight: torch.Tensor, abs: bool = True):
    """Transposable 2:4 mask by exhaustive scoring (sparse/legacy.py:271-354): every 4x4 block is scored
    against the 90 admissible patterns with one fp32 matrix product and takes the best; returns
    (weight * mask, mask).  The product's summation order is the GEMM library's, so near-ties can fall
    differently than in ``TransposableSparse``, which adds in a fixed order."""
    m, k = weight.shape
    score_in = weight.detach().abs() if abs else weight.detach()
    blocks = score_in.float().reshape(m // 4, 4, k // 4, 4).permute(0, 2, 1, 3).reshape(-1, 16)
    table = _transposable_table(weight.device)
    best = torch.argmax(blocks @ table.t(), dim=-1)
    mask = table[best].reshape(m // 4, k // 4, 4, 4).permute(0, 2, 1, 3).reshape(m, k).to(weight.dtype)
    return weight * mask, mask
