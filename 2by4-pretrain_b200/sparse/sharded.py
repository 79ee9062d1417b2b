"""Sharding of the single-op paths over the ranks of one node.

Every group of four is independent, so the conversions shard by row blocks with no exchange; the
sparse GEMM shards by blocks of output features (rows of W), each rank holding its block of W
compressed as a matrix of its own (own row count in the metadata placement formula, which uses the
number of rows of the logical matrix: sparse/_semi_structured_conversions.py:639-661 of the reference).
A collective appears only where the caller wants the full Y on every rank (``all_gather_columns``).

Nothing here reads another rank's memory: operands are local, the gather is NCCL's (gloo on CPU).
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist

# Row-block heights must keep whole metadata interleave groups (32 rows for int16 metadata, 16 for
# int32), whole 4x4 blocks of the transposable mask and whole 128-row tensor-core blocks.
ROW_ALIGN = 128


def row_block(m: int, rank: int, world: int, align: int = ROW_ALIGN) -> Tuple[int, int]:
    """Rows [r0, r1) of an m-row matrix owned by ``rank``: blocks of ``align`` rows dealt out as evenly
    as possible, earlier ranks taking the remainder.  A rank may own nothing when m < world * align."""
    if m % align != 0:
        raise RuntimeError(f"row count {m} is not a multiple of the shard alignment {align}")
    if not 0 <= rank < world:
        raise RuntimeError(f"rank {rank} outside world of {world}")
    blocks = m // align
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return b0 * align, b1 * align


def shard_rows(t: torch.Tensor, rank: Optional[int] = None, world: Optional[int] = None,
               align: int = ROW_ALIGN) -> torch.Tensor:
    """This rank's row block of a 2-D tensor (a view)."""
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    r0, r1 = row_block(t.shape[0], rank, world, align)
    return t[r0:r1]


class ColumnParallelSparseWeight:
    """This rank's block of output features of W (out_features x in_features) under a transposable
    2:4 mask, compressed for the forward GEMM (W_s) and for the backward GEMM (W_s^T).

    The mask of a row block of W equals the row block of the mask of W (4x4 blocks never straddle a
    block boundary), so every rank selects on its own rows only.
    """

    def __init__(self, weight: torch.Tensor, rank: Optional[int] = None, world: Optional[int] = None,
                 dtype: torch.dtype = torch.float16):
        from .transposable_semi_structured import select_and_compress
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.out_features, self.in_features = weight.shape
        self.r0, self.r1 = row_block(self.out_features, self.rank, self.world)
        self.dtype = dtype
        self.mask = None
        self.compressed = None
        if self.r1 > self.r0:
            local = weight[self.r0:self.r1].contiguous()
            self.mask, (pw, mw), (pt, mt) = select_and_compress(local, mask=None, dtype=dtype)
            self.compressed = (pw, mw, pt, mt)

    def forward_local(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, features_major: bool = False) -> torch.Tensor:
        """Y[:, r0:r1] = x @ W_s[r0:r1].T (+ bias[r0:r1]); x is replicated (T x in_features).  With
        ``features_major`` the block is computed as (r1 - r0, T) contiguous and returned as its transposed view: the
        layout ``all_gather_columns`` can gather with one collective and no copy."""
        from . import spmm as _spmm
        if self.compressed is None:
            return x.new_empty((x.shape[0], 0), dtype=self.dtype)
        pw, mw, _, _ = self.compressed
        b = None if bias is None else bias[self.r0:self.r1].to(self.dtype).contiguous()
        if not features_major:
            return _spmm.sparse_linear(x, pw, mw, bias=b)
        keep = _spmm.RETURN_TRANSPOSED_VIEW
        _spmm.RETURN_TRANSPOSED_VIEW = True
        try:
            return _spmm.sparse_linear(x, pw, mw, bias=b)
        finally:
            _spmm.RETURN_TRANSPOSED_VIEW = keep

    def grad_input_partial(self, grad_local: torch.Tensor) -> torch.Tensor:
        """This rank's term of dX = sum over ranks of dY[:, r0:r1] @ W_s[r0:r1]; the caller reduces."""
        from .spmm import sparse_linear
        _, _, pt, mt = self.compressed
        return sparse_linear(grad_local, pt, mt)


def all_gather_columns(y_local: torch.Tensor, out_features: int, world: Optional[int] = None,
                       group=None) -> torch.Tensor:
    """Assemble Y (T x out_features) from the ranks' column blocks.  Blocks differ in width when the
    128-row blocks do not divide evenly, so every rank pads to the widest block, gathers once, and
    copies the valid columns out."""
    world = dist.get_world_size(group) if world is None else world
    widths = [r1 - r0 for r0, r1 in (row_block(out_features, r, world) for r in range(world))]
    wmax = max(widths)
    t = y_local.shape[0]
    if min(widths) == wmax and y_local.dim() == 2 and y_local.t().is_contiguous():
        # equal blocks, each stored features-major (w, T): every rank's rows are one contiguous piece of the
        # (out_features, T) result, so one all-gather into that tensor does it; Y is its transposed view
        yt = y_local.new_empty((out_features, t))
        dist.all_gather_into_tensor(yt, y_local.t(), group=group)
        return yt.t()
    padded = y_local
    if y_local.shape[1] != wmax:
        padded = y_local.new_zeros((t, wmax))
        padded[:, :y_local.shape[1]] = y_local
    gathered = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(gathered, padded.contiguous(), group=group)
    y = y_local.new_empty((t, out_features))
    c = 0
    for r in range(world):
        y[:, c:c + widths[r]] = gathered[r][:, :widths[r]]
        c += widths[r]
    return y
