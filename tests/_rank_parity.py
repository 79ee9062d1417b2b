"""Helper of test_gpu_spmm.py: trains the small sparse GPT-2-shaped model for a few steps with the graph-replayed
trainer and prints the per-step losses of the whole job.  Run once as a single process with batch 2 B and once under
torch.distributed.run on two ranks with batch B: both see the same sequences (one global token stream), so the two
loss curves must track each other up to the MVUE draws and the all-reduce's summation order."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "2by4-pretrain_b200"))
import train_gpt2  # noqa: E402

batch = int(sys.argv[1])
mode = sys.argv[2] if len(sys.argv) > 2 else "sparse"
world = int(os.environ.get("WORLD_SIZE", "1"))
local = int(os.environ.get("LOCAL_RANK", "0"))
torch.cuda.set_device(local)
if world > 1:
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
r = train_gpt2.run_graphs(steps=30, warmup=0, mode=mode, batch=batch, seq=128, vocab=512, layers=2, d=256, heads=4, lr=3e-3,
                          freq=10, return_losses=True, comm_groups=2, data="affine", global_stream=True)
if int(os.environ.get("RANK", "0")) == 0:
    print("LOSSES " + json.dumps(r["losses"]))
if world > 1:
    dist.destroy_process_group()
