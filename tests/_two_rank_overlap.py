"""Two-rank helper of test_gpu_spmm.py (run under torch.distributed.run): the graph-replayed trainer with the
gradient all-reduce split into block groups released from inside the backward graph must give the very losses of
the single all-reduce after the graph.  Dense linears: every kernel of that step is deterministic, and with two
ranks an average has one summation order."""
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
losses = {}
for groups in (1, 4):
    r = train_gpt2.run_graphs(steps=5, warmup=2, mode="dense", batch=2, seq=256, layers=4, return_losses=True,
                              comm_groups=groups)
    losses[groups] = r["losses"]
ok = losses[1] == losses[4] and all(abs(v) < 20 for v in losses[1])
if dist.get_rank() == 0:
    print("OVERLAP_OK" if ok else f"OVERLAP_MISMATCH {losses}")
dist.destroy_process_group()
sys.exit(0 if ok else 1)
