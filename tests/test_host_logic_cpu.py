"""CPU tests of host-side logic that needs no kernel: the device guard every wrapper runs before it hands raw
pointers to the library, the dense autograd layers kept for API compatibility, and the bookkeeping of the
tensor-core metadata cache."""
import types

import pytest
import torch
import torch.nn.functional as F


class _FakeTensor:
    """Stands in for a CUDA tensor: the guard only reads ``is_cuda`` and ``device.index``."""

    def __init__(self, index, is_cuda=True):
        self.is_cuda = is_cuda
        self.device = types.SimpleNamespace(index=index, type="cuda" if is_cuda else "cpu")


def test_device_guard_rejects_tensors_of_another_gpu(monkeypatch):
    from sparse import _ext
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    _ext.require_cuda(_FakeTensor(0), None, _FakeTensor(0))           # all on the current device: fine
    with pytest.raises(RuntimeError, match="current CUDA device is cuda:0"):
        _ext.require_cuda(_FakeTensor(0), _FakeTensor(1))             # spread over two devices
    with pytest.raises(RuntimeError, match="current CUDA device is cuda:0"):
        _ext.require_cuda(_FakeTensor(1))                             # one device, but not the current one
    with pytest.raises(RuntimeError, match="Only CUDA tensors"):
        _ext.require_cuda(_FakeTensor(None, is_cuda=False))
    with pytest.raises(RuntimeError, match="Only CUDA tensors"):
        _ext.require_cuda(torch.zeros(4))


def test_public_ops_refuse_cpu_tensors_instead_of_falling_back():
    import sparse
    x = torch.randn(32, 64)
    for call in (lambda: sparse.sparse24_triton(x), lambda: sparse.soft_threshold24_triton(x),
                 lambda: sparse.MVUE24_approx_triton(x), lambda: sparse.mask_select(x),
                 lambda: sparse.to_sparse_semi_structured(x)):
        with pytest.raises((RuntimeError, AssertionError)):
            call()


@pytest.mark.parametrize("bias", [True, False])
def test_my_linear_equals_torch_linear(bias):
    import sparse
    torch.manual_seed(0)
    layer = sparse.MyLinear(24, 40, bias=bias)
    x = torch.randn(3, 5, 24, requires_grad=True)
    y = layer(x)
    y.square().sum().backward()
    x2 = x.detach().clone().requires_grad_(True)
    w2 = layer.weight.detach().clone().requires_grad_(True)
    b2 = layer.bias.detach().clone().requires_grad_(True) if bias else None
    y2 = F.linear(x2, w2, b2)
    y2.square().sum().backward()
    assert torch.allclose(y, y2, atol=1e-6)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5) and torch.allclose(layer.weight.grad, w2.grad, atol=1e-5)
    if bias:
        assert torch.allclose(layer.bias.grad, b2.grad, atol=1e-5)


def test_dense_layers_are_distinct_functions_with_the_reference_names():
    from sparse import sparse_ops
    assert sparse_ops.my_linear is not sparse_ops.sparse_linear
    assert sparse_ops.my_linear.__name__ == "my_linear" and sparse_ops.sparse_linear.__name__ == "sparse_linear"
    assert issubclass(sparse_ops.my_linear, torch.autograd.Function)


def test_tensor_core_metadata_cache_notices_in_place_writes():
    from sparse import spmm
    meta = torch.zeros(128, 8, dtype=torch.int16)
    copy = torch.zeros(16, dtype=torch.uint8)
    spmm.register_tc_metadata(meta, copy)
    hit = spmm._tc_meta_cache[id(meta)]
    assert hit[0]() is meta and hit[1] is copy and hit[2] == spmm._stamp(meta)
    meta.add_(1)                                # an in-place write through torch bumps the version counter
    assert spmm._tc_meta_cache[id(meta)][2] != spmm._stamp(meta)
    spmm.invalidate_meta(meta)
    assert id(meta) not in spmm._tc_meta_cache


def test_masked_add_storage_order_view():
    """The flat view over a tensor's elements in storage order: identity for contiguous tensors, the underlying
    buffer for transposed / permuted ones, None when the storage has gaps."""
    from sparse.decay import _storage_order
    a = torch.arange(24.).reshape(4, 6)
    assert torch.equal(_storage_order(a), a.reshape(-1))
    assert torch.equal(_storage_order(a.t()), a.reshape(-1))            # same storage, same order
    b = torch.arange(120.).reshape(2, 3, 4, 5).permute(2, 0, 3, 1)
    assert torch.equal(_storage_order(b), torch.arange(120.))
    assert _storage_order(a[:, ::2]) is None                            # gaps
    assert _storage_order(a[1:3, :]).numel() == 12                      # a contiguous slab keeps its offset
    assert torch.equal(_storage_order(a[1:3, :]), a.reshape(-1)[6:18])
    assert _storage_order(a.expand(2, 4, 6)) is None                    # overlapping (stride 0)


def test_copy_engine_average_shards_partition_every_range():
    """The shards of a range, one per rank, are disjoint, in order, cover the range exactly and start on multiples of
    eight elements from its beginning (16-byte pieces for 16-bit values)."""
    from sparse.peer import CopyEngineAverage
    for world in (2, 3, 4, 8):
        avg = CopyEngineAverage.__new__(CopyEngineAverage)
        avg.world = world
        for a, b in ((0, 8), (16, 16 + 85_000_004), (4, 4 + 7), (0, 38_633_472), (8, 8 + 63)):
            pos = a
            for p in range(world):
                lo, hi = avg._shard(a, b, p)
                assert lo == pos and hi >= lo and (lo - a) % 8 == 0 or lo == b
                pos = hi
            assert pos == b
