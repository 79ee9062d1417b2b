"""CPU oracle for the 2:4 sparse-training hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain numpy / CPU torch, the arithmetic of the
reference project's 2:4 prune / compress / metadata kernels so that the CUDA
kernels can be checked bit-for-bit.  Nothing in the shipped package imports
it: only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark do, and there only as the checker (or as the thing timed as "CPU").

Each function cites the reference lines it follows (paths are relative to the
reference project root).  Pinning: the functions here are compared against
outputs of the reference's own code (its pure-PyTorch converter and its Triton
kernels run under the Triton CPU interpreter), stored as fixtures under
``tests/golden`` together with the script that produced them, and against the
reference's docstring known-answer (metadata -4370 for the [0,0,1,1] tile).

Conventions
-----------
* every array is a CPU ``torch.Tensor``; float work that must be IEEE-exact is
  done in numpy float32 with one rounding per operation (no fused multiply-add);
* ``meta`` always means the *reordered* metadata buffer in the layout the
  reference exposes (``sparse/_semi_structured_conversions.py:639-661``),
  viewed as ``(m, k/16)`` int16 or ``(m, k/32)`` int32.
"""
from __future__ import annotations

import itertools
from typing import Optional, Tuple

import numpy as np
import torch

MVUE_EPS = np.float32(1.19209e-07)  # sparse/utils.py:8

_F8 = tuple(getattr(torch, n) for n in ("float8_e4m3fn", "float8_e5m2") if hasattr(torch, n))


# ---------------------------------------------------------------------------
# A.1  magnitude top-2-of-4 mask
# ---------------------------------------------------------------------------
def _six_compares(a0, a1, a2, a3):
    return a0 > a1, a0 > a2, a0 > a3, a1 > a2, a1 > a3, a2 > a3


def mask_from_magnitudes(a0, a1, a2, a3):
    """sparse/utils.py:63-69 and sparse/_semi_structured_conversions.py:42-44.

    Six strict comparisons; ties keep the higher index.  Inputs are magnitudes
    (any float dtype that compares exactly); returns four bool arrays.
    """
    x1, x2, x3, x4, x5, x6 = _six_compares(a0, a1, a2, a3)
    m0 = x2 & x3 | x1 & x2 | x1 & x3
    m1 = ~x1 & x5 | x4 & x5 | ~x1 & x4
    m2 = ~x2 & ~x4 | ~x2 & x6 | ~x4 & x6
    m3 = ~x3 & ~x5 | ~x3 & ~x6 | ~x5 & ~x6
    return m0, m1, m2, m3


def magnitude_mask24(x: torch.Tensor) -> torch.Tensor:
    """Bool mask (same shape as ``x``) keeping the two largest |x| of every 4 along dim 1."""
    m, k = x.shape
    a = x.float().abs().reshape(m, k // 4, 4)
    ms = mask_from_magnitudes(a[..., 0], a[..., 1], a[..., 2], a[..., 3])
    return torch.stack(ms, dim=-1).reshape(m, k)


# ---------------------------------------------------------------------------
# A.2  group encoding
# ---------------------------------------------------------------------------
def encode_mask_groups(mask4: torch.Tensor):
    """sparse/_semi_structured_conversions.py:77-88.

    ``mask4``: bool (..., 4).  Returns (idx0, idx1, nibble) as int64 tensors.
    Masks with other than two set bits follow the reference fall-back table
    (``:56-71``) because the same boolean formulas are used.
    """
    m0, m1, m2, _ = mask4.unbind(-1)
    bit0 = ~m0 & m1
    bit1 = ~m0 & ~m1
    bit2 = bit1 | ~m2
    bit3 = bit0 | ~m1 | m2
    idx0 = bit0.to(torch.int64) | (bit1.to(torch.int64) << 1)
    idx1 = bit2.to(torch.int64) | (bit3.to(torch.int64) << 1)
    return idx0, idx1, idx0 | (idx1 << 2)


# ---------------------------------------------------------------------------
# A.3  metadata placement
# ---------------------------------------------------------------------------
def meta_scatter_offsets(m: int, ncols: int, itemsize: int) -> torch.Tensor:
    """Flat destination offset of logical metadata element (r, c).

    sparse/_semi_structured_conversions.py:639-661 (int16) / :1047-1069 (int32);
    same arithmetic as ``reorder_meta`` in
    sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:826-851 followed by the
    column-major-interleaved-by-2 placement.
    """
    group, inter = (32, 4) if itemsize == 2 else (16, 2)
    r = torch.arange(m, dtype=torch.int64)[:, None].expand(m, ncols)
    c = torch.arange(ncols, dtype=torch.int64)[None, :].expand(m, ncols)
    dr = r // group * group + (r % 8) * inter + (r % group) // 8
    topright = ((dr % 2 == 0) & (c % 2 == 1)).to(torch.int64)
    bottomleft = ((dr % 2 == 1) & (c % 2 == 0)).to(torch.int64)
    dr = dr + topright - bottomleft
    dc = c - topright + bottomleft
    return (dc // 2) * m * 2 + dr * 2 + dc % 2


def reorder_meta(meta_logical: torch.Tensor) -> torch.Tensor:
    m, ncols = meta_logical.shape
    off = meta_scatter_offsets(m, ncols, meta_logical.element_size())
    out = torch.empty(m * ncols, dtype=meta_logical.dtype)
    out[off.reshape(-1)] = meta_logical.reshape(-1)
    return out.view(m, ncols)


def unreorder_meta(meta_reordered: torch.Tensor) -> torch.Tensor:
    m, ncols = meta_reordered.shape
    off = meta_scatter_offsets(m, ncols, meta_reordered.element_size())
    return meta_reordered.reshape(-1)[off.reshape(-1)].view(m, ncols)


def _meta_dtype_for(out_dtype: torch.dtype) -> torch.dtype:
    """sparse/semi_structured.py:323-331."""
    if out_dtype in (torch.float16, torch.bfloat16):
        return torch.int16
    if out_dtype == torch.int8 or out_dtype in _F8:
        return torch.int32
    raise RuntimeError(f"unsupported packed dtype {out_dtype}")


def pack_nibbles(nibbles: torch.Tensor, meta_dtype: torch.dtype) -> torch.Tensor:
    """(m, k/4) nibbles -> (m, k/16) int16 or (m, k/32) int32, nibble j at bits 4j
    (sparse/_semi_structured_conversions.py:88-108, :623-632, :1023-1040)."""
    m, ng = nibbles.shape
    per = 4 if meta_dtype == torch.int16 else 8
    n = nibbles.view(m, ng // per, per)
    acc = torch.zeros(m, ng // per, dtype=torch.int64)
    for j in range(per):
        acc |= n[..., j] << (4 * j)
    if meta_dtype == torch.int16:
        acc = torch.where(acc >= 1 << 15, acc - (1 << 16), acc)
    else:
        acc = torch.where(acc >= 1 << 31, acc - (1 << 32), acc)
    return acc.to(meta_dtype)


def cast_store(values: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """The cast the reference applies on store (``tl.store`` converts to the
    pointer's element type, sparse/_semi_structured_conversions.py:614-621):
    round-to-nearest-even from the value's own precision.  float8 inputs must be
    finite and in range (the GPU conversion saturates, torch's does not)."""
    if values.dtype == out_dtype:
        return values
    if out_dtype in _F8:
        v = values.float()
        lim = 448.0 if out_dtype == torch.float8_e4m3fn else 57344.0
        return v.clamp(-lim, lim).to(out_dtype)
    return values.float().to(out_dtype)


def compress_with_mask(values: torch.Tensor, mask: torch.Tensor, out_dtype: torch.dtype
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Select two values per group of 4 (along dim 1) according to ``mask`` and
    emit packed values plus reordered metadata.

    sparse/_semi_structured_conversions.py:570-661: the value taken is the one
    at idx0 / idx1 of the encoding, whatever the mask's population count.
    ``values`` is what gets stored (the dense input, or the MVUE-rescaled fp32
    values); it is cast to ``out_dtype`` last.
    """
    m, k = values.shape
    v4 = values.reshape(m, k // 4, 4)
    idx0, idx1, nib = encode_mask_groups(mask.bool().reshape(m, k // 4, 4))
    s0 = v4.gather(-1, idx0.unsqueeze(-1))
    s1 = v4.gather(-1, idx1.unsqueeze(-1))
    packed = torch.cat((s0, s1), dim=-1).reshape(m, k // 2)
    meta_dtype = _meta_dtype_for(out_dtype)
    meta = reorder_meta(pack_nibbles(nib, meta_dtype))
    return cast_store(packed, out_dtype), meta


# ---------------------------------------------------------------------------
# Counter-based uniform stream used by the CUDA kernels' seeded MVUE mode
# ---------------------------------------------------------------------------
_PH_M0 = np.uint64(0xD2511F53)
_PH_M1 = np.uint64(0xCD9E8D57)
_PH_W0 = np.uint32(0x9E3779B9)
_PH_W1 = np.uint32(0xBB67AE85)


def philox4x32_10(c0, c1, c2, c3, k0, k1, rounds: int = 10):
    """Philox-4x32 (Salmon et al., SC'11), vectorised over numpy uint32 arrays; 10 rounds for the exact MVUE
    mode, 7 for the fast one.  This is the project's own stream definition: the reference
    draws from Triton's ``tl.rand4x(..., n_rounds=5)``
    (sparse/_semi_structured_conversions.py:535-551), which is deliberately not
    reproduced stream-for-stream."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint32).copy() for c in np.broadcast_arrays(c0, c1, c2, c3))
    k0 = np.uint32(k0)
    k1 = np.uint32(k1)
    mask32 = np.uint64(0xFFFFFFFF)
    with np.errstate(over="ignore"):
        for _ in range(rounds):
            p0 = _PH_M0 * c0.astype(np.uint64)
            p1 = _PH_M1 * c2.astype(np.uint64)
            hi0 = (p0 >> np.uint64(32)).astype(np.uint32)
            lo0 = (p0 & mask32).astype(np.uint32)
            hi1 = (p1 >> np.uint64(32)).astype(np.uint32)
            lo1 = (p1 & mask32).astype(np.uint32)
            c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
            k0 = np.uint32((int(k0) + int(_PH_W0)) & 0xFFFFFFFF)
            k1 = np.uint32((int(k1) + int(_PH_W1)) & 0xFFFFFFFF)
    return c0, c1, c2, c3


def u32_to_uniform(x: np.ndarray) -> np.ndarray:
    """Top 24 bits scaled by 2^-24: uniform on [0, 1) with 2^-24 spacing."""
    return (x >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)


def u32_to_uniform23(x: np.ndarray) -> np.ndarray:
    """Low 23 bits as the mantissa of a float in [1, 2), minus one: uniform on [0, 1) with 2^-23 spacing (the
    conversion of the kernels' fast MVUE mode)."""
    bits = (x & np.uint32(0x007FFFFF)) | np.uint32(0x3F800000)
    return bits.view(np.float32) - np.float32(1.0)


def mvue_uniforms(m: int, k: int, seed: int, offset: int, rounds: int = 10, fast: bool = False
                  ) -> Tuple[np.ndarray, np.ndarray]:
    """The (u0, u1) pair of every group of 4 of a logical (m, k) matrix.  ``fast``: the stream of the kernels'
    fast mode (Philox4x32-7 and the 23-bit conversion), otherwise Philox4x32-``rounds`` and 24 bits.

    Group ``g`` of row ``r`` has linear index ``gi = r*(k/4) + g`` whatever the
    storage order.  One Philox block serves two groups: counter =
    (lo32(gi>>1), hi32(gi>>1), lo32(offset), hi32(offset)), key = (lo32(seed),
    hi32(seed)); the even group takes words 0,1 and the odd group words 2,3.
    """
    if fast:
        rounds = 7
    conv = u32_to_uniform23 if fast else u32_to_uniform
    gi = np.arange(m * (k // 4), dtype=np.uint64)
    pair = gi >> np.uint64(1)
    x0, x1, x2, x3 = philox4x32_10(
        (pair & np.uint64(0xFFFFFFFF)).astype(np.uint32), (pair >> np.uint64(32)).astype(np.uint32),
        np.uint32(offset & 0xFFFFFFFF), np.uint32((offset >> 32) & 0xFFFFFFFF),
        seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, rounds=rounds)
    odd = (gi & np.uint64(1)).astype(bool)
    u0 = conv(np.ascontiguousarray(np.where(odd, x2, x0))).reshape(m, k // 4)
    u1 = conv(np.ascontiguousarray(np.where(odd, x3, x1))).reshape(m, k // 4)
    return u0, u1


# ---------------------------------------------------------------------------
# A.4  MVUE24 (approximate)
# ---------------------------------------------------------------------------
def mvue24_groups(x4: np.ndarray, u0: np.ndarray, u1: np.ndarray):
    """sparse/utils.py:6-59, all float32, one rounding per operation, left-to-right sums.

    ``x4``: float32 (..., 4); ``u0``/``u1``: float32 (...).  Returns
    (values float32 (..., 4) = x_i / p_i for every i, mask bool (..., 4)).
    """
    f = np.float32
    x = [np.ascontiguousarray(x4[..., i], dtype=f) for i in range(4)]
    u0 = u0.astype(f)
    u1 = u1.astype(f)
    with np.errstate(all="ignore"):
        a = [np.abs(xi) + MVUE_EPS for xi in x]
        s = ((a[0] + a[1]) + a[2]) + a[3]
        t = [ai / s for ai in a]
        sm = [s - ai for ai in a]
        kk = [ti / si for ti, si in zip(t, sm)]
        ks = ((kk[0] + kk[1]) + kk[2]) + kk[3]
        p = [t[i] + a[i] * (ks - kk[i]) for i in range(4)]

        m0 = u0 <= t[0]
        m1 = (u0 <= (t[0] + t[1])) & ~m0
        m2 = (u0 <= ((t[0] + t[1]) + t[2])) & ~m1 & ~m0
        m3 = ~m2 & ~m1 & ~m0
        m = [m0, m1, m2, m3]

        d = [(~m[i]).astype(f) * a[i] for i in range(4)]
        ds = ((d[0] + d[1]) + d[2]) + d[3]
        tt = u1 * ds
        e0 = tt <= d[0]
        e1 = (tt <= (d[0] + d[1])) & ~e0
        e2 = (tt <= ((d[0] + d[1]) + d[2])) & ~e1 & ~e0
        e3 = ~e2 & ~e1 & ~e0
        e = [e0, e1, e2, e3]
        vals = np.stack([x[i] / p[i] for i in range(4)], axis=-1)
        mask = np.stack([m[i] | e[i] for i in range(4)], axis=-1)
    return vals.astype(f), mask


def mvue24_groups_f64(x4: np.ndarray, u0: np.ndarray, u1: np.ndarray):
    """The same estimator (sparse/utils.py:6-59) evaluated in float64: the yardstick for the kernels' fast
    arithmetic, whose float32 operations are ordered differently from the reference's.  Returns
    (values float64 (..., 4) = x_i / p_i, mask bool (..., 4))."""
    d = np.float64
    x = [np.ascontiguousarray(x4[..., i]).astype(d) for i in range(4)]
    u0 = u0.astype(d)
    u1 = u1.astype(d)
    with np.errstate(all="ignore"):
        a = [np.abs(xi) + d(MVUE_EPS) for xi in x]
        s = a[0] + a[1] + a[2] + a[3]
        t = [ai / s for ai in a]
        kk = [t[i] / (s - a[i]) for i in range(4)]
        ks = kk[0] + kk[1] + kk[2] + kk[3]
        p = [t[i] + a[i] * (ks - kk[i]) for i in range(4)]
        m0 = u0 <= t[0]
        m1 = (u0 <= t[0] + t[1]) & ~m0
        m2 = (u0 <= t[0] + t[1] + t[2]) & ~m1 & ~m0
        m = [m0, m1, m2, ~m2 & ~m1 & ~m0]
        dd = [np.where(m[i], 0.0, a[i]) for i in range(4)]
        tt = u1 * (dd[0] + dd[1] + dd[2] + dd[3])
        e0 = tt <= dd[0]
        e1 = (tt <= dd[0] + dd[1]) & ~e0
        e2 = (tt <= dd[0] + dd[1] + dd[2]) & ~e1 & ~e0
        e = [e0, e1, e2, ~e2 & ~e1 & ~e0]
        vals = np.stack([x[i] / p[i] for i in range(4)], axis=-1)
        mask = np.stack([m[i] | e[i] for i in range(4)], axis=-1)
    return vals, mask


def mvue24_dense_f64(x: torch.Tensor, seed: int, offset: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Float64 evaluation of the estimator on the uniforms of the kernels' fast mode for (seed, offset):
    (values x_i / p_i at every position, keep mask), both shaped like ``x``."""
    m, k = x.shape
    u0, u1 = mvue_uniforms(m, k, seed, offset, fast=True)
    vals, mask = mvue24_groups_f64(x.double().reshape(m, k // 4, 4).numpy(), u0, u1)
    return torch.from_numpy(vals).reshape(m, k), torch.from_numpy(mask).reshape(m, k)


def mvue24_probabilities(x4: np.ndarray) -> np.ndarray:
    """Inclusion probabilities p_i of sparse/utils.py:31-34 (float32 (..., 4)): the estimator stores
    x_i / p_i with probability p_i, which is what makes it unbiased."""
    f = np.float32
    a = [np.abs(x4[..., i].astype(f)) + MVUE_EPS for i in range(4)]
    s = ((a[0] + a[1]) + a[2]) + a[3]
    t = [ai / s for ai in a]
    kk = [ti / (s - ai) for ti, ai in zip(t, a)]
    ks = ((kk[0] + kk[1]) + kk[2]) + kk[3]
    return np.stack([t[i] + a[i] * (ks - kk[i]) for i in range(4)], axis=-1).astype(f)


def _uniform_pairs_from_tensor(U: torch.Tensor):
    """Test-mode convention: group g of row r uses U[r, 4g] and U[r, 4g+1]."""
    m, k = U.shape
    u = U.float().reshape(m, k // 4, 4).numpy()
    return np.ascontiguousarray(u[..., 0]), np.ascontiguousarray(u[..., 1])


def _mvue(x: torch.Tensor, U: Optional[torch.Tensor], seed: int, offset: int, rounds: int = 10):
    m, k = x.shape
    if U is not None:
        u0, u1 = _uniform_pairs_from_tensor(U)
    else:
        u0, u1 = mvue_uniforms(m, k, seed, offset, rounds)
    x4 = x.float().reshape(m, k // 4, 4).numpy()
    vals, mask = mvue24_groups(x4, u0, u1)
    return torch.from_numpy(vals).reshape(m, k), torch.from_numpy(mask).reshape(m, k)


def mvue24_dense(x: torch.Tensor, U: Optional[torch.Tensor] = None, seed: int = 0, offset: int = 0,
                 rounds: int = 10) -> torch.Tensor:
    """sparse/triton_ops.py:10-81: dense-shaped MVUE, zeros where dropped, stored in x's dtype.
    ``rounds`` = 7 gives the stream of the kernels' fast mode (with this function's exact arithmetic: the
    yardstick the fast arithmetic is measured against)."""
    vals, mask = _mvue(x, U, seed, offset, rounds)
    return torch.where(mask, cast_store(vals, x.dtype), torch.zeros((), dtype=x.dtype))


# ---------------------------------------------------------------------------
# dense -> 2:4 conversion in its three pruning modes
# ---------------------------------------------------------------------------
def prune_compress(dense: torch.Tensor, out_dtype: torch.dtype = torch.float16, *,
                   mask: Optional[torch.Tensor] = None, mvue: bool = False,
                   U: Optional[torch.Tensor] = None, seed: int = 0, offset: int = 0,
                   out_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """sparse/_semi_structured_conversions.py:431-661 / :664-1069 with
    PRUNE = 'mask' | 'mvue' | 'mse' (launcher :1072-1132).

    Works on the logical (m, k) matrix; the storage order of ``dense`` does not
    matter (the reference's row / col layouts only change the traversal).
    Returns (packed (m, k/2) contiguous, meta reordered).
    """
    if mask is not None and mvue:
        raise RuntimeError("Error using MVUE24 with mask is not supported! ")  # semi_structured.py:207-210
    # float8 quantisation (no counterpart in the reference): the value that would be stored is multiplied by
    # ``out_scale`` in float32 (one rounding) before the cast; the pruning decision is taken on the unscaled input
    q = (lambda v: v) if out_scale is None else (lambda v: v.float() * torch.tensor(out_scale, dtype=torch.float32))
    if mask is not None:
        return compress_with_mask(q(dense), mask, out_dtype)
    if mvue:
        vals, mk = _mvue(dense, U, seed, offset)
        return compress_with_mask(q(vals), mk, out_dtype)
    return compress_with_mask(q(dense), magnitude_mask24(dense), out_dtype)


def to_dense(packed: torch.Tensor, meta: torch.Tensor) -> torch.Tensor:
    """sparse/_semi_structured_conversions.py:217-328: inverse of the conversion."""
    m, kh = packed.shape
    k = kh * 2
    logical = unreorder_meta(meta.contiguous()).to(torch.int64)
    per = 4 if meta.dtype == torch.int16 else 8
    logical = logical & ((1 << (4 * per)) - 1)
    nib = torch.stack([(logical >> (4 * j)) & 0xF for j in range(per)], dim=-1).reshape(m, k // 4)
    idx0 = nib & 3
    idx1 = (nib >> 2) & 3
    p = packed.reshape(m, k // 4, 2)
    raw = p.view(torch.uint8) if packed.dtype in _F8 else p
    dense = torch.zeros(m, k // 4, 4, dtype=raw.dtype)
    dense.scatter_(-1, idx0.unsqueeze(-1), raw[..., 0:1])
    dense.scatter_(-1, idx1.unsqueeze(-1), raw[..., 1:2])
    dense = dense.reshape(m, k)
    return dense.view(packed.dtype) if packed.dtype in _F8 else dense


# ---------------------------------------------------------------------------
# dense-shaped prune ops
# ---------------------------------------------------------------------------
def sparse24(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """sparse/triton_ops.py:84-154: (x where kept else +0, mask as 1/0 in x's dtype)."""
    mk = magnitude_mask24(x)
    zero = torch.zeros((), dtype=x.dtype)
    return torch.where(mk, x, zero), mk.to(x.dtype)


def soft_threshold24(x: torch.Tensor, scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """sparse/utils.py:72-90 + sparse/triton_ops.py:157-227.

    theta = second-smallest magnitude of the group; kept values move toward
    zero by theta with one rounding in x's dtype.  ``scale`` (the S-STE
    per-tensor factor, README.md:233-260 of the reference) multiplies the
    result with one further rounding in x's dtype when given.
    """
    m, k = x.shape
    xf = x.float().reshape(m, k // 4, 4)
    a = xf.abs()
    a0, a1, a2, a3 = a.unbind(-1)
    mk = torch.stack(mask_from_magnitudes(a0, a1, a2, a3), dim=-1)
    thr = torch.minimum(torch.maximum(torch.minimum(a0, a1), torch.minimum(a2, a3)),
                        torch.minimum(torch.maximum(a0, a1), torch.maximum(a2, a3))).unsqueeze(-1)
    s = torch.where(xf > 0, xf - thr, xf + thr).to(x.dtype)  # fp32 op then one rounding == native op
    if scale is not None:
        s = (s.float() * torch.tensor(scale, dtype=torch.float32)).to(x.dtype)
    zero = torch.zeros((), dtype=x.dtype)
    return torch.where(mk, s, zero).reshape(m, k), mk.reshape(m, k).to(x.dtype)


# ---------------------------------------------------------------------------
# A.6  transposable 4x4 mask select
# ---------------------------------------------------------------------------
_PAIRS = ((0, 1), (0, 2), (0, 3), (1, 2), (1, 3), (2, 3))


def transposable_patterns() -> np.ndarray:
    """The 90 4x4 0/1 matrices whose rows and columns all sum to 2, in descending
    lexicographic order of the row-major 16-bit string — the order of the table
    in sparse/transposable_semi_structured.py:105-196.  Shape (90, 16) uint8."""
    pats = []
    for rows in itertools.product(_PAIRS, repeat=4):
        cnt = [0, 0, 0, 0]
        for a, b in rows:
            cnt[a] += 1
            cnt[b] += 1
        if cnt == [2, 2, 2, 2]:
            bits = []
            for a, b in rows:
                r = [0, 0, 0, 0]
                r[a] = r[b] = 1
                bits += r
            pats.append(tuple(bits))
    pats.sort(reverse=True)
    return np.array(pats, dtype=np.uint8)


def pattern_row_pairs() -> np.ndarray:
    """(90, 4, 2): for pattern p and row i the two kept columns (a < b)."""
    P = transposable_patterns().reshape(90, 4, 4)
    out = np.zeros((90, 4, 2), dtype=np.int64)
    for p in range(90):
        for i in range(4):
            out[p, i] = np.nonzero(P[p, i])[0]
    return out


def transposable_mask(x: torch.Tensor, abs: bool = True) -> torch.Tensor:
    """sparse/transposable_semi_structured.py:27-47: per 4x4 block, the first of the 90
    patterns (table order) that maximises the sum of the 8 selected (|w| if abs) entries.

    Score arithmetic (the reference's ``tl.dot`` has no reproducible summation order, so
    it is fixed here): float32, row sums first, then (row0+row1) + (row2+row3):
        s_i = v[i][a_i] + v[i][b_i];  score = (s_0 + s_1) + (s_2 + s_3).
    Whenever these sums are exact (e.g. fp16 weights whose block sum is below 1) this
    equals the exact-arithmetic argmax.
    """
    m, k = x.shape
    v = x.float()
    if abs:
        v = v.abs()
    blk = v.reshape(m // 4, 4, k // 4, 4).permute(0, 2, 1, 3).contiguous().numpy()  # (bm, bk, 4, 4)
    rp = pattern_row_pairs()
    best = np.full(blk.shape[:2], -np.inf, dtype=np.float32)
    arg = np.zeros(blk.shape[:2], dtype=np.int64)
    f = np.float32
    for p in range(90):
        s = [blk[:, :, i, rp[p, i, 0]].astype(f) + blk[:, :, i, rp[p, i, 1]].astype(f) for i in range(4)]
        sc = (s[0] + s[1]) + (s[2] + s[3])
        upd = sc > best
        best = np.where(upd, sc, best)
        arg = np.where(upd, p, arg)
    P = torch.from_numpy(transposable_patterns().reshape(90, 4, 4).astype(np.bool_))
    mk = P[torch.from_numpy(arg)]  # (bm, bk, 4, 4)
    return mk.permute(0, 2, 1, 3).reshape(m, k).contiguous()


def transposable_sparse(x: torch.Tensor, abs: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """``TransposableSparse.forward``: (x where mask else +0, bool mask)."""
    mk = transposable_mask(x, abs)
    return torch.where(mk, x, torch.zeros((), dtype=x.dtype)), mk


# ---------------------------------------------------------------------------
# A.7  masked decay
# ---------------------------------------------------------------------------
def masked_add(grad: torch.Tensor, p: torch.Tensor, mask: torch.Tensor, alpha: float) -> torch.Tensor:
    """sparse/decay.py:7-37: grad + (p * alpha) where mask == 0, else grad unchanged.

    float32 grad and p (the training recipe casts the gradient to float first,
    README.md:208-213 of the reference); alpha is an fp32 scalar; two roundings
    (multiply, then add), never a fused multiply-add.  Returns the new grad."""
    if grad.dtype != torch.float32 or p.dtype != torch.float32:
        raise RuntimeError("masked_add oracle: float32 grad and p only")
    prod = (p.numpy() * np.float32(alpha)).astype(np.float32)
    out = torch.from_numpy((grad.numpy() + prod).astype(np.float32))
    return torch.where(mask.bool(), grad, out)


# ---------------------------------------------------------------------------
# A.8  GEMM reference: fp32 dense matmul of the masked weight
# ---------------------------------------------------------------------------
def spmm_reference(packed: torch.Tensor, meta: torch.Tensor, dense_b: torch.Tensor) -> torch.Tensor:
    """D (Ms x N) = A_dense (Ms x K) @ B (K x N) in fp32, A rebuilt from (packed, meta).
    Stands for sparse/csrc/mySparseSemiStructuredLinear_cuda.cu:34-233 (fp32 accumulate)."""
    a = to_dense(packed.contiguous(), meta.contiguous()).float()
    return a @ dense_b.float()


# ---------------------------------------------------------------------------
# The reference's timed CPU path (used as the benchmark's CPU arm)
# ---------------------------------------------------------------------------
def transposable_mask_matmul(x: torch.Tensor) -> torch.Tensor:
    """The reference's CPU formulation of the mask select (sparse/legacy.py:271-354): one fp32
    matrix product of the flattened |4x4 blocks| with the 90 x 16 pattern table, then argmax.
    Multi-threaded through torch; used as the timed CPU arm.  Its summation order is the BLAS
    library's, so it equals ``transposable_mask`` only when the sums are exact."""
    m, k = x.shape
    blk = x.float().abs().reshape(m // 4, 4, k // 4, 4).permute(0, 2, 1, 3).reshape(-1, 16)
    P = torch.from_numpy(transposable_patterns().astype(np.float32))
    arg = (blk @ P.t()).argmax(dim=1)
    mk = P.bool()[arg].reshape(m // 4, k // 4, 4, 4)
    return mk.permute(0, 2, 1, 3).reshape(m, k).contiguous()


def cpu_select_and_dual_compress(w: torch.Tensor, out_dtype: torch.dtype = torch.float16, matmul_scores: bool = False):
    """Transposable mask select followed by compression of W and of W^T with that mask:
    the CPU form of one mask refresh of the training layer (README.md:148-155 of the reference).
    ``matmul_scores`` picks the reference's matmul formulation of the select (faster, timed arm)."""
    mk = transposable_mask_matmul(w) if matmul_scores else transposable_mask(w)
    pw, mw = compress_with_mask(w, mk, out_dtype)
    pt, mt = compress_with_mask(w.t().contiguous(), mk.t().contiguous(), out_dtype)
    return mk, pw, mw, pt, mt
