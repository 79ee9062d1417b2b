#!/usr/bin/env python
"""Benchmark of the 2:4 sparse-training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Default workload ``select_dual_compress``: one mask refresh of a
training layer — transposable 4x4 mask select plus 2:4 compression of W and W^T — on 4096 x 4096
fp16 weights ~N(0, 0.02), seeded per matrix.  One step is the mask refresh of a 48-layer model: 48 such
matrices (distinct buffers, 4 GB of traffic per step, far larger than the 126 MB L2, so no flush is needed)
converted by ONE launch of the batched entry point ``sp24_select_dual_compress_batch`` (what
``sparse.refresh_sparse_layers`` calls once per optimizer step).

  value      algorithmic GB/s with inputs resident in HBM (CUDA events on the launching stream)
  e2e        the same metric through the public Python API from pinned HOST buffers: H2D copy of W,
             kernel, D2H copy of mask + both compressed copies, all inside the timed region
  roofline   HBM: algorithmic bytes per launch / average launch time, against the measured copy
             bandwidth in MEASURED_PEAKS.json (fallback 6650 GB/s)
  cpu_baseline  the CPU restatement of the reference's path (oracle/), timed on the host cores

With N > 1 (torchrun) every rank processes its own batch of matrices (independent objects, no
collective in the data path); time is the max over ranks.  ``--impl reference`` times the CPU arm
alone, on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "2by4-pretrain_b200"))

import torch  # noqa: E402

M = K = 4096
BATCH = 48          # matrices per step = per launch of the batched kernel (its descriptor array holds 48)
E2E_BATCH = 8       # matrices per step of the host-buffer leg (PCIe-bound: 9 ms per step)
BYTES_PER_ELEM = 2 + 1 + 2 * (2 / 2 + 1 / 8)  # read fp16 W, write bool mask, write 2 x (fp16 values/2 + 4 bits/4 elems)
ALG_BYTES_PER_MATRIX = M * K * BYTES_PER_ELEM
METRIC = "prune/compress HBM GB/s (transposable select + dual 2:4 compress)"
WORKLOAD = f"cfg2: transposable select + dual 2:4 compress, {M}x{K} fp16 N(0,0.02) seed 2+i"


def ncu_traffic_per_launch():
    """DRAM bytes (read + write) of one launch of the benchmark kernel, taken from the committed ncu summary of that
    kernel (the line ``dram_bytes_per_matrix_4096x4096: N`` of the profile text) times the matrices per launch;
    None when the summary carries no such line."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "ts_dual*"))):
        try:
            m = re.search(r"dram_bytes_per_matrix_4096x4096:\s*([0-9.eE+]+)", open(path).read())
        except OSError:
            m = None
        if m:
            return float(m.group(1)) * BATCH
    return None


def measured_tensor_peak():
    """Dense bf16 GEMM peak (TFLOP/s) measured on this pool (burst figure: a kernel timed alone), else the fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML every 2 ms while the timed region runs
    (read-only queries; falls back to one nvidia-smi query when NVML is not importable)."""

    def __init__(self, index):
        self.index = index
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.thread = None
        self.nvml = None

    def _loop(self):
        nv, h = self.nvml, self.handle
        bits = {}
        for name, attr in (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown"),
                           ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown"),
                           ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown"),
                           ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap")):
            v = getattr(nv, attr, None) or getattr(nv, attr.replace("ClocksEventReason", "ClocksThrottleReason"), None)
            if v is not None:
                bits[name] = v
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                if get_reasons is not None:
                    r = get_reasons(h)
                    for name, bit in bits.items():
                        if r & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            idx = self.index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                try:
                    idx = int(vis.split(",")[self.index])
                except Exception:
                    idx = self.index
            self.handle = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM))
            self.nvml = nv
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:
            self.nvml = None

    def stop(self):
        if self.nvml is None:
            try:
                out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=10).stdout
                a, b = [float(x) for x in out.strip().split(",")]
                return {"sm_mhz": a, "sm_max_mhz": b, "samples": 1, "reasons": [], "source": "nvidia-smi after the run"}
            except Exception:
                return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["clock query unavailable"]}
        self._stop.set()
        self.thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.sm), "reasons": sorted(self.reasons), "source": "NVML, 2 ms period"}


def make_weights(n, device, seed0=2):
    ws = []
    for i in range(n):
        g = torch.Generator().manual_seed(seed0 + i)
        ws.append((torch.randn(M, K, generator=g) * 0.02).half())
    return ws


def make_device_batch(n, dev, seed0):
    """n weight matrices drawn on the device, their output buffers and the descriptor array of the batched call
    (mask + W + W^T copies, reference metadata order only).  Returns (descriptors, tensors to keep alive)."""
    from sparse import _ext
    ws, outs = [], []
    descs = (_ext.DualDesc * n)()
    for i in range(n):
        g = torch.Generator(device=dev).manual_seed(seed0 + i)
        w = (torch.randn(M, K, device=dev, generator=g) * 0.02).half()
        mask = torch.empty(M, K, dtype=torch.bool, device=dev)
        bw = torch.empty(M * K * 9 // 16, dtype=torch.float16, device=dev)
        bt = torch.empty(M * K * 9 // 16, dtype=torch.float16, device=dev)
        ws.append(w)
        outs.append((mask, bw, bt))
        d = descs[i]
        d.w, d.m, d.k, d.ld_w = w.data_ptr(), M, K, K
        d.mask, d.ld_mask = mask.data_ptr(), K
        d.packed_w, d.ld_packed_w, d.meta_w = bw.data_ptr(), K // 2, bw.data_ptr() + M * K
        d.packed_t, d.ld_packed_t, d.meta_t = bt.data_ptr(), K, bt.data_ptr() + M * K
        d.tc_w = d.tc_t = None
    return descs, (ws, outs)


def cpu_arm(seconds_budget=12.0, max_reps=6):
    """Times the CPU restatement of the path (mask select in the reference's matmul form + both
    compressions) on full 4096 x 4096 matrices; returns (GB/s, cores, description)."""
    from oracle import sp24_oracle as O
    w = make_weights(1, "cpu")[0]
    O.cpu_select_and_dual_compress(w[:512], matmul_scores=True)  # warm-up (thread pools, page faults)
    times = []
    t_end = time.perf_counter() + seconds_budget
    while len(times) < max_reps and (not times or time.perf_counter() < t_end):
        t0 = time.perf_counter()
        O.cpu_select_and_dual_compress(w, matmul_scores=True)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return ALG_BYTES_PER_MATRIX / med / 1e9, torch.get_num_threads(), \
        f"{len(times)} x one full {M}x{K} fp16 matrix (median), torch CPU threads={torch.get_num_threads()}", med


def run_reference(args, rank):
    if rank != 0:
        return
    try:  # torchrun pins OMP_NUM_THREADS=1; the CPU arm may use every host core
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:
        pass
    per_step = []
    from oracle import sp24_oracle as O
    w = make_weights(1, "cpu")[0]
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        O.cpu_select_and_dual_compress(w, matmul_scores=True)
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            per_step.append(dt)
    total = sum(per_step)
    val = ALG_BYTES_PER_MATRIX * len(per_step) / total / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / len(per_step) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "alg_bytes_per_elem": BYTES_PER_ELEM,
                   "step": "one matrix per step (bounded sample of the GPU arm's 48-matrix batch)"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{len(per_step)} steps x one {M}x{K} matrix; CPU restatement of the reference "
                                   "path (matmul-form mask select + pure-torch compress)"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the per-kernel side measurements")
    ap.add_argument("--case", default=None,
                    help="profiling aid: run ONE named kernel case (1 warm-up + 3 launches, inputs > L2) and exit; "
                         "prints no benchmark line")
    args = ap.parse_args()
    if args.case:
        run_case(args.case)
        return
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() != "INFO":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=dev)

    import sparse
    from sparse import _ext

    lib = _ext.lib()
    # device-resident inputs: 48 distinct matrices drawn on the device (seed 2 + matrix index, rank-disjoint)
    descs, keep_alive = make_device_batch(BATCH, dev, 2 + rank * BATCH)
    ws_cpu = make_weights(E2E_BATCH, "cpu", seed0=2 + rank * E2E_BATCH)      # host copies for the end-to-end leg
    stream = torch.cuda.current_stream()

    def step_device():
        # one launch: select + dual compress of all 48 matrices
        rc = lib.sp24_select_dual_compress_batch(descs, BATCH, _ext.F16, _ext.F16, 1, stream.cuda_stream)
        if rc:
            _ext.check(rc, "sp24_select_dual_compress_batch")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        step_device()
    ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    launches = args.steps * world
    total_bytes = ALG_BYTES_PER_MATRIX * BATCH * args.steps * world
    value = total_bytes / (ms * 1e-3) / 1e9
    per_launch_s = ms * 1e-3 / args.steps   # one GPU's launches: the roofline is per kernel launch, not per job
    achieved = ALG_BYTES_PER_MATRIX * BATCH / per_launch_s / 1e9
    del keep_alive, descs
    torch.cuda.empty_cache()

    # end-to-end through the public API with host buffers
    pinned = [w.pin_memory() for w in ws_cpu]
    host_out = [(torch.empty(M, K, dtype=torch.bool).pin_memory(),
                 torch.empty(M, K // 2, dtype=torch.float16).pin_memory(), torch.empty(M, K // 16, dtype=torch.int16).pin_memory(),
                 torch.empty(M // 2, K, dtype=torch.float16).pin_memory(), torch.empty(K, M // 16, dtype=torch.int16).pin_memory())
                for _ in range(E2E_BATCH)]

    # Three streams: uploads, the kernels, downloads.  PCIe is full duplex, so matrix i+1 goes up while matrix i is
    # compressed and matrix i-1 comes down; events order the three stages of every matrix.
    up, down = torch.cuda.Stream(), torch.cuda.Stream()

    def step_e2e():
        keep = []   # device tensors stay referenced until the step's last copy has been ordered behind them
        for wh, ho in zip(pinned, host_out):
            with torch.cuda.stream(up):
                wd = wh.to(dev, non_blocking=True)
                ev_up = torch.cuda.Event()
                ev_up.record(up)
            stream.wait_event(ev_up)
            mask, (pw, mw), (pt, mt) = sparse.select_and_compress(wd)
            ev_done = torch.cuda.Event()
            ev_done.record(stream)
            with torch.cuda.stream(down):
                down.wait_event(ev_done)
                ho[0].copy_(mask, non_blocking=True)
                ho[1].copy_(pw, non_blocking=True)
                ho[2].copy_(mw, non_blocking=True)
                ho[3].copy_(pt.t(), non_blocking=True)
                ho[4].copy_(mt, non_blocking=True)
            keep.append((wd, mask, pw, mw, pt, mt))
        ev_last = torch.cuda.Event()
        ev_last.record(down)
        stream.wait_event(ev_last)      # the timing events sit on the main stream: make it cover the downloads
        torch.cuda.current_stream().synchronize()
        del keep

    e2e_steps = max(2, min(args.steps, 5))
    step_e2e()
    barrier()
    ev0.record(stream)
    for _ in range(e2e_steps):
        step_e2e()
    ev1.record(stream)
    barrier()
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e_val = ALG_BYTES_PER_MATRIX * E2E_BATCH * e2e_steps * world / (e2e_ms * 1e-3) / 1e9
    h2d = E2E_BATCH * M * K * 2
    d2h = E2E_BATCH * (M * K + 2 * (M * K + M * K // 8))

    extra = None
    spmm_extra = None
    if rank == 0 and world == 1 and not args.no_extra:
        extra = side_measurements(dev)
        spmm_extra = spmm_measurements(dev)

    sharded = None
    if world > 1 and not args.no_extra:
        sharded = sharded_spmm_measurements(dev, rank, world)

    gpt2 = None
    if not args.no_extra:
        gpt2 = gpt2_measurements(world)

    if rank == 0:
        peak, peak_kind = measured_peak()
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "batch_per_step_per_gpu": BATCH, "launches_per_step": 1, "alg_bytes_per_elem": BYTES_PER_ELEM,
                       "l2": "inputs+outputs per step = 4.0 GB > 126 MB L2, no flush",
                       "parallelism": f"independent matrices x{world}"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": ncu_traffic_per_launch(), "peak_kind": peak_kind, "kernel": "ts_dual_batch_kernel",
                         "alg_bytes_per_launch": ALG_BYTES_PER_MATRIX * BATCH},
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "matrices_per_step": E2E_BATCH,
                    "streams": "pinned host buffers; uploads, kernels and downloads on three streams, ordered per matrix by events"},
            "gpu_launches": launches, "clocks": clocks,
        }
        if not args.no_cpu and world == 1:
            v, cores, sample, _ = cpu_arm()
            line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
            if not args.no_extra:
                line["cpu_side"] = cpu_side_measurements()
        if extra:
            line["kernels"] = extra
        if sharded:
            line["spmm_cfg4_column_parallel"] = sharded
        if spmm_extra:
            line["spmm_cfg4"] = spmm_extra
        if gpt2:
            line["gpt2_124m"] = gpt2
        # the three quantities of the metric side by side (the first is `value`)
        summary = {"prune_compress_GBps": value, "prune_compress_frac_of_hbm_peak": achieved / peak}
        if spmm_extra and "fp16" in spmm_extra:
            summary["spmm_fwd_bwd_TFLOPs_dense_equiv_fp16"] = spmm_extra["fp16"]["sparse_fwd_bwd_TFLOPs_dense_equiv"]
            summary["spmm_fwd_bwd_speedup_vs_dense_fp16"] = spmm_extra["fp16"]["speedup_vs_dense"]
        if gpt2 and "sparse_tokens_per_s" in gpt2:
            summary["gpt2_124m_tokens_per_s"] = gpt2["sparse_tokens_per_s"]
            summary["gpt2_124m_sparse_over_dense"] = gpt2["sparse_over_dense"]
        line["north_star_summary"] = summary
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_case(name):
    """One kernel on a case a little larger than L2 (a few hundred MB on the device), for ncu captures."""
    import sparse
    from sparse._semi_structured_conversions import prune_compress
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if name == "dual":
        w = (torch.randn(8192, 8192, device=dev) * 0.02).half()
        fn = lambda: sparse.select_and_compress(w)
    elif name == "dual_batch":        # the benchmark kernel on a sixth of its batch: 8 matrices of 4096 x 4096 in one launch
        from sparse import _ext
        descs, keep_alive = make_device_batch(8, dev, 2)
        lib = _ext.lib()

        def fn():
            _ext.check(lib.sp24_select_dual_compress_batch(descs, 8, _ext.F16, _ext.F16, 1, _ext.stream()), "batch")
    elif name == "select":
        w = (torch.randn(8192, 8192, device=dev) * 0.02).half()
        fn = lambda: sparse.mask_select(w)
    elif name == "dual_given_mask":   # the refresh between mask selections: mask read, both compressions written
        w = (torch.randn(8192, 8192, device=dev) * 0.02).half()
        _, mk = sparse.mask_select(w)
        fn = lambda: sparse.select_and_compress(w, mask=mk)
    elif name in ("mvue_row", "mse_row", "mvue_col", "mse_col", "mvue_fast_row", "mvue_fast_col"):
        m, k = 16384, 4096
        g = (torch.randn(m, k, device=dev) * 1e-3).bfloat16()
        mode = 3 if name.startswith("mvue_fast") else (2 if name.startswith("mvue") else 0)
        if name.endswith("col"):
            g = g.t()
            packed = torch.empty(m // 2, k, dtype=torch.bfloat16, device=dev).t()
            meta = torch.empty(k, m // 16, dtype=torch.int16, device=dev)
        else:
            packed = torch.empty(m, k // 2, dtype=torch.bfloat16, device=dev)
            meta = torch.empty(m, k // 16, dtype=torch.int16, device=dev)
        fn = lambda: prune_compress(g, packed, meta, mode=mode, seed=1)
    elif name in ("spmm_fwd", "spmm_dx", "spmm_dw", "spmm_dw_acc"):
        T, K, N = 16384, 768, 3072
        dt = torch.float16
        x = torch.randn(T, K, device=dev).to(dt)
        dy = (torch.randn(T, N, device=dev) * 1e-2).to(dt)
        w = torch.randn(N, K, device=dev) * 0.02
        mask, (pw, mw), (pt, mt) = sparse.select_and_compress(w, dtype=dt)
        ws = sparse.SparseSemiStructuredTensor(None, original_shape=w.shape, sparse_tensor_cutlass=pw, meta_tensor_cutlass=mw, dtype=dt)
        wt = sparse.SparseSemiStructuredTensor(None, original_shape=w.t().shape, sparse_tensor_cutlass=pt, meta_tensor_cutlass=mt, dtype=dt)
        dys = sparse.to_sparse_semi_structured(dy.t(), MVUE24=True, dtype=dt)
        if name == "spmm_fwd":
            fn = lambda: torch.mm(x, ws.t())
        elif name == "spmm_dx":
            fn = lambda: torch.mm(dy, wt.t())
        elif name == "spmm_dw":
            fn = lambda: torch.mm(dys, x)
        else:   # the form the training layer uses: fp32 gradient buffer, split-K, vector reductions
            from sparse.spmm import sparse_mm_accumulate_
            gw = torch.zeros(N, K, dtype=torch.float32, device=dev)
            fn = lambda: sparse_mm_accumulate_(gw, dys.sparse_tensor_cutlass, dys.meta_tensor_cutlass, x)
    elif name == "soft":
        g = (torch.randn(16384, 4096, device=dev) * 1e-3).bfloat16()
        fn = lambda: sparse.soft_threshold24_triton(g)
    elif name == "masked_add":
        p = torch.randn(8192, 4096, device=dev)
        gr = torch.randn(8192, 4096, device=dev)
        mk = torch.rand(8192, 4096, device=dev) < 0.5
        fn = lambda: sparse.masked_add_(gr, p, mk, alpha=2e-4)
    elif name in ("ce_fused", "add_ln_fwd", "add_ln_bwd", "gelu_bwd"):
        # the trainer's streaming kernels at the GPT-2-124M shapes (8192 tokens; 50304 classes, d = 768, 4 d = 3072)
        from sparse import train_ops
        rows = 8192
        if name == "ce_fused":
            logits = (torch.randn(rows, 50304, device=dev) * 2).bfloat16().requires_grad_(True)
            tgt = torch.randint(0, 50304, (rows,), device=dev)
            fn = lambda: train_ops.cross_entropy(logits, tgt)
        elif name == "gelu_bwd":
            xs = [torch.randn(rows, 3072, device=dev).bfloat16().requires_grad_(True) for _ in range(3)]
            dy = torch.randn(rows, 3072, device=dev).bfloat16()
            it = iter(range(1 << 30))
            fn = lambda: train_ops.gelu(xs[next(it) % 3]).backward(dy)
        else:
            ln = train_ops.LayerNorm(768).to(dev)
            xs = [torch.randn(rows, 768, device=dev).requires_grad_(True) for _ in range(6)]
            ds = [torch.randn(rows, 768, device=dev).bfloat16().requires_grad_(True) for _ in range(6)]
            dres, dy = torch.randn(rows, 768, device=dev), torch.randn(rows, 768, device=dev).bfloat16()
            it = iter(range(1 << 30))

            def fn():
                i = next(it) % 6
                with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                    res, y = train_ops.add_layer_norm(xs[i], ds[i], ln)
                if name == "add_ln_bwd":
                    torch.autograd.backward([res, y], [dres, dy])
    else:
        raise SystemExit(f"unknown case {name}")
    for _ in range(4):
        fn()
    torch.cuda.synchronize()
    print(f"case {name}: done")


def side_measurements(dev):
    """Per-kernel GB/s of the other conversion kernels (outside the headline timing): each timed over
    a rotating set of buffers larger than L2, CUDA events, 3 warm-up + 10 timed passes."""
    import sparse
    from sparse import _ext
    from sparse._semi_structured_conversions import prune_compress
    peak, _ = measured_peak()
    res = {}

    def timeit(fn, nbuf, reps=10):
        for i in range(3):
            fn(i % nbuf)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(i % nbuf)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / reps

    m, k = 8192, 4096
    n = m * k
    nb = 4
    G = [(torch.randn(m, k, device=dev) * 1e-3).bfloat16() for _ in range(nb)]
    packed = [torch.empty(m, k // 2, dtype=torch.bfloat16, device=dev) for _ in range(nb)]
    meta = [torch.empty(m, k // 16, dtype=torch.int16, device=dev) for _ in range(nb)]

    def rec(name, secs, nbytes):
        res[name] = {"ms": secs * 1e3, "GB/s": nbytes / secs / 1e9, "frac_of_hbm_peak": nbytes / secs / 1e9 / peak}

    rec("cfg3 mvue compress row bf16 8192x4096 (exact arithmetic)",
        timeit(lambda i: prune_compress(G[i], packed[i], meta[i], mode=2, seed=1, offset=i), nb), n * (2 + 1 + 0.125))
    rec("cfg3 mvue compress row bf16 8192x4096 (fast arithmetic, the training path)",
        timeit(lambda i: prune_compress(G[i], packed[i], meta[i], mode=3, seed=1, offset=i), nb), n * (2 + 1 + 0.125))
    rec("cfg3 magnitude compress row bf16 8192x4096",
        timeit(lambda i: prune_compress(G[i], packed[i], meta[i], mode=0), nb), n * (2 + 1 + 0.125))
    Gt = [g.t() for g in G]  # column-major view of a (4096, 8192) logical matrix
    packed_t = [torch.empty(m // 2, k, dtype=torch.bfloat16, device=dev).t() for _ in range(nb)]
    meta_t = [torch.empty(k, m // 16, dtype=torch.int16, device=dev) for _ in range(nb)]
    rec("mvue compress col-major bf16 (dY^T form) 4096x8192 (exact arithmetic)",
        timeit(lambda i: prune_compress(Gt[i], packed_t[i], meta_t[i], mode=2, seed=1, offset=i), nb), n * (2 + 1 + 0.125))
    rec("mvue compress col-major bf16 (dY^T form) 4096x8192 (fast arithmetic, the training path)",
        timeit(lambda i: prune_compress(Gt[i], packed_t[i], meta_t[i], mode=3, seed=1, offset=i), nb), n * (2 + 1 + 0.125))
    rec("cfg3 soft_threshold24 bf16 8192x4096", timeit(lambda i: sparse.soft_threshold24_triton(G[i]), nb), n * 6)
    rec("sparse24 bf16 8192x4096", timeit(lambda i: sparse.sparse24_triton(G[i]), nb), n * 6)
    rec("mvue24 dense bf16 8192x4096 (exact arithmetic)",
        timeit(lambda i: sparse.MVUE24_approx_triton(G[i], seed=3, offset=i, exact=True), nb), n * 4)
    rec("mvue24 dense bf16 8192x4096 (fast arithmetic)",
        timeit(lambda i: sparse.MVUE24_approx_triton(G[i], seed=3, offset=i, exact=False), nb), n * 4)
    del packed, meta, packed_t, meta_t
    Wf = [torch.randn(4096, 4096, device=dev) * 0.02 for _ in range(nb)]
    rec("transposable select fp32 4096x4096 (sparse+mask)", timeit(lambda i: sparse.mask_select(Wf[i]), nb), 4096 * 4096 * 9)
    # fp32 master weights -> fp16 compressed copies, through the C ABI with caller-allocated outputs (as a trainer
    # with a fixed memory plan would call it; the Python wrapper adds five allocations per call)
    lib = _ext.lib()
    mm = kk = 4096
    d_mask = [torch.empty(mm, kk, dtype=torch.bool, device=dev) for _ in range(nb)]
    d_bw = [torch.empty(mm * kk * 9 // 16, dtype=torch.float16, device=dev) for _ in range(nb)]
    d_bt = [torch.empty(mm * kk * 9 // 16, dtype=torch.float16, device=dev) for _ in range(nb)]

    def dual_f32(i):
        rc = lib.sp24_select_dual_compress(Wf[i].data_ptr(), _ext.F32, mm, kk, kk, 1, d_mask[i].data_ptr(), kk,
                                           d_bw[i].data_ptr(), _ext.F16, kk // 2, d_bw[i].data_ptr() + mm * kk,
                                           d_bt[i].data_ptr(), kk, d_bt[i].data_ptr() + mm * kk, _ext.stream())
        _ext.check(rc, "sp24_select_dual_compress")

    rec("select+dual compress fp32->fp16 4096x4096", timeit(dual_f32, nb), 4096 * 4096 * (4 + 1 + 2.25))
    del d_mask, d_bw, d_bt
    p = [torch.randn(m, k, device=dev) * 0.02 for _ in range(2)]
    gr = [torch.randn(m, k, device=dev) * 1e-3 for _ in range(2)]
    mk = [torch.rand(m, k, device=dev) < 0.5 for _ in range(2)]
    rec("cfg3 masked_add_ fp32 8192x4096", timeit(lambda i: sparse.masked_add_(gr[i], p[i], mk[i], alpha=2e-4), 2), n * 13)
    return res


def gpt2_measurements(world):
    """cfg5: GPT-2-124M-shaped model, 8 x 1024 synthetic tokens per GPU and step, data-parallel over the
    ranks of this job (graph-replayed step, grouped NCCL all-reduce of the flat gradient; the eager figure uses
    DistributedDataParallel).  Tokens/s of the sparse recipe (SparseLinearTranspose in every block, masked decay,
    AdamW) and of the same model with dense linears."""
    sys.path.insert(0, os.path.join(ROOT, "2by4-pretrain_b200"))
    import train_gpt2
    out = {}
    try:
        sp = train_gpt2.run_graphs(steps=50, warmup=3, mode="sparse")
        de = train_gpt2.run_graphs(steps=20, warmup=3, mode="dense")
        sp_eager = train_gpt2.run(steps=10, warmup=3, mode="sparse")
        bf16_exchange = {}
        if world > 1:   # the option that halves the exchanged bytes (the optimizer kernel reads the bf16 average)
            sp16 = train_gpt2.run_graphs(steps=30, warmup=3, mode="sparse", reduce_dtype=torch.bfloat16)
            bf16_exchange = {"sparse_tokens_per_s_bf16_gradient_exchange": sp16["tokens_per_s"],
                             "sparse_ms_per_step_bf16_gradient_exchange": sp16["ms_per_step"]}
        out = {"sparse_tokens_per_s": sp["tokens_per_s"], "sparse_ms_per_step": sp["ms_per_step"],
               "dense_tokens_per_s": de["tokens_per_s"], "dense_ms_per_step": de["ms_per_step"],
               "sparse_over_dense": sp["tokens_per_s"] / de["tokens_per_s"], "tokens_per_step": sp["tokens_per_step"],
               "loss_finite": sp["loss_finite"], "n_gpus": world,
               "sparse_eager_ddp_tokens_per_s": sp_eager["tokens_per_s"],
               "sparse_eager_ddp_host_enqueue_ms_per_step": sp_eager["host_enqueue_ms_per_step"],
               **bf16_exchange,
               "note": "step replayed from CUDA graphs (forward+backward; the flat fp32 gradient all-reduced by NCCL in "
                       "groups released by event nodes inside the backward graph: the output head's share of the tied "
                       "embedding gradient first, then four groups of blocks, the embeddings last, beside the masked "
                       "decay + AdamW of the other parameters); 50 timed sparse steps, mean, including the mask "
                       "refresh every 40 steps; eager = Python-launched step with DistributedDataParallel"}
    except Exception as exc:  # the headline line must still be printed
        out = {"error": repr(exc)[:300]}
    return out


def sharded_spmm_measurements(dev, rank, world):
    """cfg4 forward GEMM split by blocks of output features over the ranks (X replicated, every rank holds its
    rows of W compressed as its own matrix): whole-job dense-equivalent TFLOP/s without and with the
    all-gather of Y, device time, max over ranks."""
    import torch.distributed as dist
    from sparse.sharded import ColumnParallelSparseWeight, all_gather_columns
    T, K, N = 16384, 768, 3072
    g = torch.Generator(device="cpu").manual_seed(8)
    w = (torch.randn(N, K, generator=g) * 0.02).to(dev)
    xs = [torch.randn(T, K, device=dev).half() for _ in range(3)]
    sh = ColumnParallelSparseWeight(w, rank=rank, world=world)

    def timed(fn, reps=10):
        for i in range(3):
            fn(i)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_local = timed(lambda i: sh.forward_local(xs[i % 3]))
    ms_gather = timed(lambda i: all_gather_columns(sh.forward_local(xs[i % 3], features_major=True), N, world))
    flops = 2.0 * T * K * N
    return {"rows_of_W_per_rank": sh.r1 - sh.r0, "fwd_ms": ms_local, "fwd_TFLOPs_dense_equiv": flops / ms_local / 1e9,
            "fwd_plus_allgather_ms": ms_gather, "fwd_plus_allgather_TFLOPs_dense_equiv": flops / ms_gather / 1e9,
            "n_gpus": world, "scaling": "strong (one GEMM split over the ranks)"}


def cpu_side_measurements():
    """The other operations of the path on the host cores (CPU restatements of the reference's own CPU
    formulations), one warm-up and the median of three runs each; sizes reduced where stated."""
    from oracle import sp24_oracle as O
    res = {"threads": torch.get_num_threads()}

    def med(fn, reps=3):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return statistics.median(ts)

    g = torch.Generator().manual_seed(3)
    m, k = 2048, 4096                                   # a quarter of cfg3's rows
    G = (torch.randn(m, k, generator=g) * 1e-3).bfloat16()
    n = m * k
    t = med(lambda: O.prune_compress(G, torch.bfloat16))
    res["magnitude compress bf16 2048x4096"] = {"ms": t * 1e3, "GB/s": n * 3.125 / t / 1e9}
    packed, meta = O.prune_compress(G, torch.bfloat16)[:2]
    t = med(lambda: O.to_dense(packed, meta))
    res["to_dense bf16 2048x4096"] = {"ms": t * 1e3, "GB/s": n * 3.125 / t / 1e9}
    t = med(lambda: O.soft_threshold24(G))
    res["soft_threshold24 bf16 2048x4096"] = {"ms": t * 1e3, "GB/s": n * 6 / t / 1e9}
    t = med(lambda: O.mvue24_dense(G[:512], seed=1, offset=0), reps=1)
    res["mvue24 dense bf16 512x4096"] = {"ms": t * 1e3, "GB/s": 512 * k * 4 / t / 1e9}
    p = torch.randn(m, k, generator=g) * 0.02
    gr = torch.randn(m, k, generator=g) * 1e-3
    mk = torch.rand(m, k, generator=g) < 0.5
    t = med(lambda: O.masked_add(gr.clone(), p, mk, 2e-4))
    res["masked_add fp32 2048x4096 (includes one clone of grad)"] = {"ms": t * 1e3, "GB/s": n * 13 / t / 1e9}
    # cfg4 forward GEMM as a dense fp32 matmul of the masked weight, one eighth of the tokens
    T, K, N = 2048, 768, 3072
    x = torch.randn(T, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.02
    wm = torch.where(O.magnitude_mask24(w), w, torch.zeros(()))
    t = med(lambda: x @ wm.t())
    res["dense fp32 masked matmul 2048x768x3072"] = {"ms": t * 1e3, "TFLOP/s": 2.0 * T * K * N / t / 1e12}
    return res


def spmm_measurements(dev):
    """cfg4: one GPT-2 MLP projection, X 16384x768, W 3072x768 under a transposable 2:4 mask.
    Times the three sparse GEMMs of a training step (forward, dX, dW with the MVUE compression of dY^T
    included) against torch.mm (cuBLAS) dense GEMMs of the same shapes.  TFLOP/s are dense-equivalent
    (2*T*N*K per GEMM).  L2 is flushed by rotating over several operand sets."""
    import sparse
    T, K, N = 16384, 768, 3072
    flops = 2.0 * T * N * K
    res = {}
    tensor_peak, tensor_peak_kind = measured_tensor_peak()
    for dtype, tag in ((torch.float16, "fp16"), (torch.bfloat16, "bf16")):
        nb = 3
        xs = [torch.randn(T, K, device=dev).to(dtype) for _ in range(nb)]
        dys = [(torch.randn(T, N, device=dev) * 1e-2).to(dtype) for _ in range(nb)]
        w = torch.randn(N, K, device=dev) * 0.02
        mask, (pw, mw), (pt, mt) = sparse.select_and_compress(w, dtype=dtype)
        ws = sparse.SparseSemiStructuredTensor(None, original_shape=w.shape, sparse_tensor_cutlass=pw,
                                               meta_tensor_cutlass=mw, dtype=dtype)
        wt = sparse.SparseSemiStructuredTensor(None, original_shape=w.t().shape, sparse_tensor_cutlass=pt,
                                               meta_tensor_cutlass=mt, dtype=dtype)
        wd = torch.where(mask, w, torch.zeros((), device=dev)).to(dtype)

        def timeit(fn, reps=12):
            for i in range(3):
                fn(i % nb)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(reps):
                fn(i % nb)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e-3 / reps

        t_fwd = timeit(lambda i: torch.mm(xs[i], ws.t()))
        from sparse import spmm as _spmm
        _spmm.RETURN_TRANSPOSED_VIEW = True
        t_fwd_view = timeit(lambda i: torch.mm(xs[i], ws.t()))
        t_dx_view = timeit(lambda i: torch.mm(dys[i], wt.t()))
        _spmm.RETURN_TRANSPOSED_VIEW = False
        t_dx = timeit(lambda i: torch.mm(dys[i], wt.t()))
        t_dw = timeit(lambda i: torch.mm(sparse.to_sparse_semi_structured(dys[i].t(), MVUE24=True, dtype=dtype), xs[i]))
        t_dw_gemm_only = None
        pre = [sparse.to_sparse_semi_structured(dys[i].t(), MVUE24=True, dtype=dtype) for i in range(nb)]
        for i in range(nb):
            torch.mm(pre[i], xs[i])
        t_dw_gemm_only = timeit(lambda i: torch.mm(pre[i], xs[i]))
        # split-K form with fp32 accumulation into a zeroed gradient buffer (what the training layer uses)
        gw = torch.zeros(N, K, dtype=torch.float32, device=dev)

        def dw_splitk(i, compress=True):
            sp = sparse.to_sparse_semi_structured(dys[i].t(), MVUE24=True, dtype=dtype) if compress else pre[i]
            gw.zero_()
            _spmm.sparse_mm_accumulate_(gw, sp.sparse_tensor_cutlass, sp.meta_tensor_cutlass, xs[i])

        t_dw_splitk = timeit(lambda i: dw_splitk(i))
        t_dw_splitk_gemm = timeit(lambda i: dw_splitk(i, False))
        d_fwd = timeit(lambda i: torch.mm(xs[i], wd.t()))
        d_dx = timeit(lambda i: torch.mm(dys[i], wd))
        d_dw = timeit(lambda i: torch.mm(dys[i].t(), xs[i]))
        sp_total, de_total = t_fwd + t_dx + min(t_dw, t_dw_splitk), d_fwd + d_dx + d_dw
        res[tag] = {
            "sparse_ms": {"fwd": t_fwd * 1e3, "dx": t_dx * 1e3, "dw_incl_mvue_compress": t_dw * 1e3,
                          "dw_gemm_only": t_dw_gemm_only * 1e3,
                          "dw_splitk_fp32_incl_mvue_compress": t_dw_splitk * 1e3,
                          "dw_splitk_fp32_gemm_and_memset_only": t_dw_splitk_gemm * 1e3,
                          "fwd_transposed_view_like_reference": t_fwd_view * 1e3,
                          "dx_transposed_view_like_reference": t_dx_view * 1e3},
            "dense_cublas_ms": {"fwd": d_fwd * 1e3, "dx": d_dx * 1e3, "dw": d_dw * 1e3},
            "sparse_fwd_bwd_TFLOPs_dense_equiv": 3 * flops / sp_total / 1e12,
            "dense_fwd_bwd_TFLOPs": 3 * flops / de_total / 1e12,
            "speedup_vs_dense": de_total / sp_total,
            # the layer's option weight_grad = "dense": sparse forward and input gradient, exact dense weight gradient
            # (no MVUE estimate); not the reference recipe, reported beside it
            "speedup_vs_dense_with_dense_weight_gradient": de_total / (t_fwd + t_dx + d_dw),
            "per_gemm_TFLOPs": {"fwd": flops / t_fwd / 1e12, "dx": flops / t_dx / 1e12,
                                "dw_gemm_only": flops / t_dw_gemm_only / 1e12,
                                "dw_splitk_fp32_gemm_and_memset_only": flops / t_dw_splitk_gemm / 1e12},
            # dense-equivalent rate over twice the dense tensor peak (2:4 sparse MMAs run at twice the dense rate)
            "roofline": {"bound": "tensor", "peak": 2 * tensor_peak, "peak_kind": tensor_peak_kind, "unit": "TFLOP/s",
                         "frac": {"fwd": flops / t_fwd / 1e12 / (2 * tensor_peak), "dx": flops / t_dx / 1e12 / (2 * tensor_peak),
                                  "dw_gemm": flops / t_dw_splitk_gemm / 1e12 / (2 * tensor_peak)}},
        }
        del xs, dys, pre
    # fp8 e4m3 with per-tensor scales: forward, input gradient through the K-major W^T, weight gradient with the MVUE
    # compression of dY^T to e4m3 included; fp32 outputs (scales applied by one multiply on the result)
    from sparse import fp8, _ext as _e
    x = torch.randn(T, K, device=dev)
    w = torch.randn(N, K, device=dev) * 0.02
    dy = (torch.randn(T, N, device=dev) * 1e-2).bfloat16()
    _, mask = sparse.mask_select(w)
    w8 = fp8.Fp8SparseWeight(w, mask)
    xq, sx = fp8.quantize(x)
    gq, sg = fp8.quantize(dy)
    xq_t = xq.t().contiguous()

    def t8(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / reps

    t_f = t8(lambda: fp8.fst_fp8_forward(xq, sx, w8))
    t_x = t8(lambda: fp8.fst_fp8_input_grad(gq, sg, w8))
    t_w = t8(lambda: fp8.fst_fp8_weight_grad(dy, sg, xq_t, sx, seed=1))
    pg, mg = fp8.compress_q8(dy.t(), mode=_e.PRUNE_MVUE_FAST, scale=sg, seed=1)
    t_wc = t8(lambda: fp8.compress_q8(dy.t(), mode=_e.PRUNE_MVUE_FAST, scale=sg, seed=1))
    res["fp8_e4m3"] = {"fwd_ms": t_f * 1e3, "dx_ms": t_x * 1e3, "dw_incl_mvue_compress_ms": t_w * 1e3,
                       "dw_mvue_compress_only_ms": t_wc * 1e3,
                       "fwd_TFLOPs_dense_equiv": flops / t_f / 1e12, "dx_TFLOPs_dense_equiv": flops / t_x / 1e12,
                       "dw_TFLOPs_dense_equiv": flops / t_w / 1e12,
                       "fwd_bwd_TFLOPs_dense_equiv": 3 * flops / (t_f + t_x + t_w) / 1e12,
                       "note": "fp32 outputs (201 MB for fwd, 50 MB for dX), dequantisation scales applied in the GEMM epilogue"}
    from sparse.spmm import check_status
    check_status()
    return res


if __name__ == "__main__":
    main()
