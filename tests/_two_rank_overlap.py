"""Two-rank helper of test_gpu_spmm.py (run under torch.distributed.run): the graph-replayed trainer with the
gradient all-reduce split into block groups released from inside the backward graph must give the very losses of
the single all-reduce after the graph.  Dense linears and the framework's own layer norm / embedding (the library's
trainer kernels add their column sums with atomics, in no fixed order): every kernel of that step is deterministic,
and with two ranks an average has one summation order.  A last pair of runs repeats the comparison with the library's
trainer kernels, to a tolerance."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "2by4-pretrain_b200"))
import train_gpt2  # noqa: E402

local = int(os.environ.get("LOCAL_RANK", "0"))
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
train_gpt2.FUSED_OPS = False
losses = {}
for groups in (1, 4):
    r = train_gpt2.run_graphs(steps=5, warmup=2, mode="dense", batch=2, seq=256, layers=4, return_losses=True,
                              comm_groups=groups)
    losses[groups] = r["losses"]
ok = losses[1] == losses[4] and all(abs(v) < 20 for v in losses[1])
# the same model with the head's share of the tied gradient inside autograd (one exchange group for the whole tail)
r = train_gpt2.run_graphs(steps=5, warmup=2, mode="dense", batch=2, seq=256, layers=4, return_losses=True, comm_groups=4,
                          split_head=False)
ok = ok and all(abs(a - b) < 2e-2 for a, b in zip(r["losses"], losses[4]))     # bf16 head share: not bit-identical
# and with every group exchanged as bf16
r = train_gpt2.run_graphs(steps=5, warmup=2, mode="dense", batch=2, seq=256, layers=4, return_losses=True, comm_groups=4,
                          reduce_dtype=torch.bfloat16)
ok = ok and all(abs(a - b) < 2e-2 for a, b in zip(r["losses"], losses[4]))
# the same average from peer-to-peer copies on the DMA engines (sparse.peer) instead of NCCL's all-reduce kernels: with
# two ranks both compute (a + b) / 2, bit for bit
r = train_gpt2.run_graphs(steps=5, warmup=2, mode="dense", batch=2, seq=256, layers=4, return_losses=True, comm_groups=4,
                          exchange="copy")
ok = ok and r["losses"] == losses[4]
# the library's trainer kernels (atomics: last-bit differences between runs), one group against four
train_gpt2.FUSED_OPS = True
fused = {}
for groups in (1, 4):
    r = train_gpt2.run_graphs(steps=5, warmup=2, mode="dense", batch=2, seq=256, layers=4, return_losses=True,
                              comm_groups=groups)
    fused[groups] = r["losses"]
ok = ok and all(abs(a - b) < 1e-3 for a, b in zip(fused[1], fused[4]))
ok = ok and all(abs(a - b) < 2e-2 for a, b in zip(fused[4], losses[4]))
if dist.get_rank() == 0:
    print("OVERLAP_OK" if ok else f"OVERLAP_MISMATCH {losses} {fused}")
dist.destroy_process_group()
sys.exit(0 if ok else 1)
