"""Two-rank gloo tests (CPU) of the host-side multi-rank logic: the data-parallel step keeps the
replicas identical, every rank draws its own MVUE seeds and its own benchmark matrices."""
import os
import random
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

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
    port = 29500 + (os.getpid() % 2000)
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
