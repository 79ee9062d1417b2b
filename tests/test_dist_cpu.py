"""Two-rank gloo tests (CPU) of the host-side multi-rank logic: the data-parallel step keeps the
replicas identical, every rank draws its own MVUE seeds and its own benchmark matrices."""
import os
import random
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

def _free_port():
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "2by4-pretrain_b200")


def _worker(rank, world, port, out):
    sys.path.insert(0, PKG)
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import train_gpt2
        random.seed(1234 + rank)
        first_seed = random.randint(0, 2 ** 31 - 1)
        model = train_gpt2.build("dense", torch.device("cpu"), layers=1, d=64, heads=2, seq=16, vocab=128)
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        gen = torch.Generator().manual_seed(10 + rank)
        for _ in range(2):
            tok = torch.randint(0, 128, (2, 17), generator=gen)
            loss = ddp(tok[:, :-1], tok[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad()
        flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
        gathered = [torch.zeros_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        seeds = [None] * world
        dist.all_gather_object(seeds, (first_seed, float(tok.sum())))
        if rank == 0:
            out.put((bool(all(torch.equal(gathered[0], g) for g in gathered)), seeds))
    except Exception as exc:  # surface the failure at once instead of letting the parent time out
        out.put(("error", repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_data_parallel_step_keeps_replicas_identical_and_seeds_distinct():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, seeds = q.get(timeout=240)
    assert same != "error", seeds
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same, "replicas diverged after the all-reduced steps"
    assert seeds[0][0] != seeds[1][0], "ranks must draw different MVUE seeds"
    assert seeds[0][1] != seeds[1][1], "ranks must see different token batches"


def test_bench_matrices_differ_per_rank():
    sys.path.insert(0, ROOT)
    import bench
    a = bench.make_weights(1, "cpu", seed0=2 + 0 * bench.BATCH)[0]
    b = bench.make_weights(1, "cpu", seed0=2 + 1 * bench.BATCH)[0]
    assert a.shape == (4096, 4096) and a.dtype == torch.float16 and not torch.equal(a, b)
    assert abs(float(a.float().std()) - 0.02) < 1e-3


def test_row_blocks_partition_the_rows():
    sys.path.insert(0, PKG)
    from sparse.sharded import row_block
    for m, world in ((3072, 8), (768, 8), (2304, 4), (128, 2), (1280, 3)):
        blocks = [row_block(m, r, world) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == m
        for (a0, a1), (b0, b1) in zip(blocks, blocks[1:]):
            assert a1 == b0 and a0 <= a1 and b0 <= b1
        assert all(b0 % 128 == 0 and b1 % 128 == 0 for b0, b1 in blocks)
        widths = [b1 - b0 for b0, b1 in blocks]
        assert max(widths) - min(widths) <= 128
    with pytest.raises(RuntimeError):
        row_block(100, 0, 2)
    with pytest.raises(RuntimeError):
        row_block(256, 2, 2)


def _gather_worker(rank, world, port, out):
    sys.path.insert(0, PKG)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sparse.sharded import all_gather_columns, row_block, shard_rows
        n_out, t = 384, 5                      # three 128-row blocks over two ranks: widths 256 and 128
        full = torch.arange(t * n_out, dtype=torch.float32).reshape(t, n_out)
        r0, r1 = row_block(n_out, rank, world)
        w = torch.arange(n_out * 8, dtype=torch.float32).reshape(n_out, 8)
        assert torch.equal(shard_rows(w), w[r0:r1])
        y = all_gather_columns(full[:, r0:r1].contiguous(), n_out)
        ok = bool(torch.equal(y, full))
        # equal blocks stored features-major (w, T): the single-collective path, result is a transposed view
        n2 = 512
        full2 = torch.arange(t * n2, dtype=torch.float32).reshape(t, n2)
        a, b = row_block(n2, rank, world)
        local = full2[:, a:b].t().contiguous().t()          # (T, w) view of a contiguous (w, T) block
        y2 = all_gather_columns(local, n2)
        ok = ok and bool(torch.equal(y2, full2)) and y2.t().is_contiguous()
        if rank == 0:
            out.put(ok)
    except Exception as exc:
        out.put(("error", repr(exc)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_column_blocks_gather_back_to_the_full_output():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res is True, res
