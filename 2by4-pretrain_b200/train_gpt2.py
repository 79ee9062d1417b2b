"""Data-parallel 2:4 sparse pre-training of a GPT-2-124M-shaped model on synthetic tokens.

    python 2by4-pretrain_b200/train_gpt2.py --steps 20                      # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        2by4-pretrain_b200/train_gpt2.py --steps 20                         # 8 GPUs, NCCL

The model is written from the hyper-parameters alone (12 layers, d_model 768, 12 heads, MLP 3072,
sequence 1024, vocabulary 50304, normal(0, 0.02) init); every ``nn.Linear`` inside the blocks is a
``SparseLinearTranspose``.  The step follows the reference's recipe (README.md:125-226 of the reference):
forward / backward with three sparse GEMMs per layer, then masked decay
``masked_add_(p.grad, p.data, p.mask, alpha)`` on every sparse weight and ``p.cnt = 0``, then AdamW.
Gradients are averaged by ``DistributedDataParallel`` (bucketed NCCL all-reduce overlapped with backward).
Masks need no communication: the weights are identical on all ranks after the reduce, so every rank
recomputes the same transposable mask.  MVUE seeds come from Python's ``random``, seeded per rank.

``--graphs`` replays the step from CUDA graphs instead of launching ~2000 kernels from Python: one graph for
forward + backward on a mask-refresh step, one for the other steps, one for masked decay + AdamW (one fused
kernel launch per parameter segment).  Parameters, gradients and moments live in flat fp32 buffers; the gradient
buffer is all-reduced by a few NCCL calls issued from the host on a second stream (no collective is captured): one
per group of transformer blocks, each released by an event-record node inside the backward graph, so that all
but the last group's exchange overlaps the rest of the backward pass.  The MVUE seeds recorded in a graph stay fixed, so the kernels add a device counter, bumped
inside the graph, to their Philox offset: every replay draws fresh uniforms.
"""
import argparse
import math
import os
import random
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


# True: layer norm and cross entropy run on the library's streaming kernels (sparse.train_ops) instead of the
# framework's float32 layer norm + cast, gamma / beta gradient kernel and float32 log-softmax over the logits.
FUSED_OPS = True


def _layer_norm(d):
    if FUSED_OPS:
        from sparse.train_ops import LayerNorm
        return LayerNorm(d)
    return nn.LayerNorm(d)


def _add_norm(x, delta, norm):
    """(x + delta, norm(x + delta)): the residual connection and the following norm."""
    if FUSED_OPS:
        from sparse.train_ops import add_layer_norm
        return add_layer_norm(x, delta, norm)
    x = x + delta
    return x, norm(x)


def _gelu(x):
    if FUSED_OPS:
        from sparse.train_ops import gelu
        return gelu(x)
    return F.gelu(x, approximate="tanh")


class Block(nn.Module):
    # True: fc + GELU + proj through sparse.fst_mlp (GELU and its gradient in the GEMM epilogues).  Off by default:
    # at d_model 768 the two GEMMs that would carry the extra epilogue work have K = 768, six K steps per tile, and
    # their epilogue is already as long as the tile's tensor-core time; the separate GELU passes are faster.
    fused_mlp = False

    def __init__(self, d, heads, linear):
        super().__init__()
        self.heads = heads
        self.ln1 = _layer_norm(d)
        self.attn_qkv = linear(d, 3 * d)
        self.attn_proj = linear(d, d)
        self.ln2 = _layer_norm(d)
        self.fc = linear(d, 4 * d)
        self.proj = linear(4 * d, d)

    def forward(self, x, delta=None):
        """``x``: the residual stream, ``delta``: the previous block's MLP output, not yet added to it (None in front
        of the first block).  Returns the same pair for the next block: every residual add runs inside the kernel of
        the norm that follows it."""
        b, t, d = x.shape
        if delta is None:
            h = self.ln1(x)
        else:
            x, h = _add_norm(x, delta, self.ln1)
        q, k, v = self.attn_qkv(h).split(d, dim=2)
        q, k, v = (z.view(b, t, self.heads, d // self.heads).transpose(1, 2) for z in (q, k, v))
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x, h = _add_norm(x, self.attn_proj(y.transpose(1, 2).reshape(b, t, d)), self.ln2)
        if self.fused_mlp:
            import sparse
            return x, sparse.fst_mlp(h, self.fc, self.proj)
        return x, self.proj(_gelu(self.fc(h)))


class _tied_head(torch.autograd.Function):
    """logits = x W^T for the output head that shares W with the token embedding, with the head's share of dW written
    (bf16, overwritten every step) into a buffer of its own instead of flowing into W.grad through autograd.  The head's
    share is the first gradient a backward pass produces and the embedding's share the last; summed by autograd they
    become available only at the very end, which keeps the largest tensor of the model out of every overlapped
    gradient exchange.  ``on_ready`` is called once the buffer has been written."""

    @staticmethod
    def forward(ctx, x, weight, head_grad, on_ready):
        xb, wb = x.to(head_grad.dtype), weight.to(head_grad.dtype)
        ctx.save_for_backward(xb, wb)
        ctx.head_grad, ctx.on_ready, ctx.x_dtype = head_grad, on_ready, x.dtype
        return xb @ wb.t()

    @staticmethod
    def backward(ctx, g):
        xb, wb = ctx.saved_tensors
        g2, x2 = g.reshape(-1, g.shape[-1]), xb.reshape(-1, xb.shape[-1])
        torch.mm(g2.t(), x2, out=ctx.head_grad)
        if ctx.on_ready is not None:
            ctx.on_ready()
        return (g2 @ wb).view_as(xb).to(ctx.x_dtype), None, None, None


class GPT2(nn.Module):
    def __init__(self, linear, layers=12, d=768, heads=12, seq=1024, vocab=50304):
        super().__init__()
        self.seq = seq
        self.wte = nn.Embedding(vocab, d)
        self.wpe = nn.Embedding(seq, d)
        self.blocks = nn.ModuleList(Block(d, heads, linear) for _ in range(layers))
        self.ln_f = _layer_norm(d)
        # block index -> callable run when the gradient with respect to that block's input exists, i.e. when the
        # backward pass has left the block (used to start gradient all-reduces early)
        self.input_grad_hooks = {}
        # set by a trainer that exchanges the head's share of the tied weight's gradient separately (see _tied_head)
        self.head_grad = None
        self.head_ready = None
        self.first_block_hook = None
        # True: the embedding gradients are added straight into existing float32 .grad buffers (flat-buffer trainers)
        self.accumulate_into_grad = False
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx, targets):
        b, t = idx.shape
        if FUSED_OPS and idx.is_cuda:
            from sparse.train_ops import embed_tokens
            x = embed_tokens(idx, self.wte.weight, self.wpe.weight, self.accumulate_into_grad)
        else:
            x = self.wte(idx) + self.wpe(torch.arange(t, device=idx.device))
        if self.first_block_hook is not None and x.requires_grad:
            x.register_hook(lambda g, f=self.first_block_hook: f())     # the backward pass has left block 0
        delta = None
        for i, blk in enumerate(self.blocks):
            if i in self.input_grad_hooks and x.requires_grad:
                x.register_hook(lambda g, f=self.input_grad_hooks[i]: f())
            x, delta = blk(x, delta)
        x, h = _add_norm(x, delta, self.ln_f)
        if self.head_grad is not None:
            logits = _tied_head.apply(h, self.wte.weight, self.head_grad, self.head_ready)
        else:
            logits = F.linear(h, self.wte.weight)  # tied output head
        if FUSED_OPS and logits.dtype in (torch.float16, torch.bfloat16):
            from sparse.train_ops import cross_entropy
            return cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1))
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))


def masked_decay_(model, alpha):
    """README.md:205-214 of the reference: decay pruned weights through the gradient, reset ``cnt``."""
    import sparse
    with torch.no_grad():
        for p in model.parameters():
            if hasattr(p, "mask") and p.mode == "sparse" and p.grad is not None:
                p.grad = p.grad.float()
                sparse.masked_add_(p.grad.data, p.data, p.mask, alpha=alpha)
                p.cnt = 0


def build(mode, device, layers=12, d=768, heads=12, seq=1024, vocab=50304, seed=11):
    import sparse
    torch.manual_seed(seed)  # same initial weights on every rank

    def linear(i, o):
        return sparse.SparseLinearTranspose(i, o, bias=True)

    model = GPT2(linear, layers, d, heads, seq, vocab).to(device)
    for p in model.parameters():
        if hasattr(p, "mask"):
            p.mode = mode
            p.mask = p.mask.to(device)
    return model


def run(steps, warmup, mode="sparse", batch=8, seq=1024, vocab=50304, layers=12, d=768, heads=12, alpha=2e-4,
        lr=6e-4, verbose=False):
    """Returns a dict with tokens/s (whole job) and ms per step, timed on the device, max over ranks."""
    import torch.distributed as dist
    import sparse
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    own_group = False
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
        own_group = True
    random.seed(1234 + rank)  # MVUE streams differ per rank
    model = build(mode, dev, layers, d, heads, seq, vocab)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True)
    decay, no_decay = [], []
    for n_, p in model.named_parameters():
        (no_decay if p.dim() < 2 or hasattr(p, "mask") else decay).append(p)
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=lr, betas=(0.9, 0.95), fused=True)
    gen = torch.Generator(device="cpu").manual_seed(10 + rank)
    losses = []

    def one_step():
        tok = torch.randint(0, vocab, (batch, seq + 1), generator=gen)
        tok = tok.pin_memory().to(dev, non_blocking=True)
        x, y = tok[:, :-1], tok[:, 1:]
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
            if mode == "sparse":
                sparse.refresh_sparse_layers(model)     # all layers' W / W^T copies in one launch
            loss = net(x, y)
        loss.backward()
        if mode == "sparse":
            masked_decay_(model, alpha)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(warmup):
        one_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t_cpu = time.perf_counter()
    for _ in range(steps):
        losses.append(one_step().detach())
    t_cpu = time.perf_counter() - t_cpu  # host time to enqueue the steps (no synchronisation inside)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    last = float(torch.stack(losses).float()[-1].item())
    res = {"tokens_per_s": batch * seq * world * steps / (ms * 1e-3), "ms_per_step": ms / steps, "world": world,
           "tokens_per_step": batch * seq * world, "last_loss": last, "mode": mode, "loss_finite": math.isfinite(last),
           "host_enqueue_ms_per_step": t_cpu * 1e3 / steps}
    if mode == "sparse":
        from sparse.spmm import check_status
        check_status()
    del opt, net, model
    torch.cuda.empty_cache()
    if own_group:
        dist.destroy_process_group()
    if verbose and rank == 0:
        print(res)
    return res


def synthetic_tokens(n, seq, vocab, gen, data="uniform"):
    """(n, seq + 1) token ids.  "uniform": independent draws (nothing to learn: the loss stays near ln(vocab));
    "affine": a random first token, then x[t + 1] = (5 x[t] + 7) mod vocab, a next-token rule a small model learns
    within tens of steps (for tests that compare loss curves)."""
    if data == "uniform":
        return torch.randint(0, vocab, (n, seq + 1), generator=gen)
    tok = torch.empty((n, seq + 1), dtype=torch.long)
    tok[:, 0] = torch.randint(0, vocab, (n,), generator=gen)
    for t in range(seq):
        tok[:, t + 1] = (tok[:, t] * 5 + 7) % vocab
    return tok


def run_graphs(steps, warmup, mode="sparse", batch=8, seq=1024, vocab=50304, layers=12, d=768, heads=12, alpha=2e-4,
               lr=6e-4, freq=40, verbose=False, return_losses=False, comm_groups=5, data="uniform", global_stream=False,
               split_head=True, reduce_dtype=torch.float32, exchange="nccl"):
    """The same step as ``run`` replayed from CUDA graphs.  Returns the same dict.

    With more than one rank and ``comm_groups`` > 1 the gradient all-reduce is split into that many groups of
    transformer blocks, last blocks first; each group's all-reduce starts on a second stream as soon as the
    backward pass (still running inside the graph) has left the group, signalled by an event-record node in the
    graph.  ``comm_groups`` = 1 is one all-reduce of the whole flat gradient after the graph.

    ``split_head``: the output head's share of the tied embedding's gradient goes to a bf16 buffer of its own, which is
    all-reduced as soon as the backward pass has produced it (its first product) and added to the embedding's gradient
    before the update; the embeddings' own (lookup) gradients, complete only when the backward pass ends, form the
    last group alone.  ``reduce_dtype`` = torch.bfloat16 exchanges every group as bf16 (cast, all-reduce; the optimizer
    kernel reads the averaged 16-bit gradient, no cast back): half the bytes on the wire.

    ``exchange``: "nccl" (all-reduce kernels, which hold SMs beside the backward pass) or "copy" (``sparse.peer``: the
    same average from peer-to-peer copies on the DMA engines plus small element-wise kernels; one node, float32).

    ``global_stream``: every rank draws the whole job's batch (world x batch sequences) from one common seed and keeps
    its own slice, so that N ranks x batch B see exactly the sequences of one rank x batch N B; with ``return_losses``
    the per-step losses are then averaged over the ranks."""
    import torch.distributed as dist
    import sparse
    from sparse._semi_structured_conversions import set_device_rng_offset
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    own_group = False
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
        own_group = True
    random.seed(1234 + rank)
    model = build(mode, dev, layers, d, heads, seq, vocab)
    for mod in model.modules():   # weight gradients are added into the flat buffer by the GEMM itself
        if hasattr(mod, "accumulate_into_grad"):
            mod.accumulate_into_grad = True
    params = [p for p in model.parameters()]
    sparse_params = [p for p in params if hasattr(p, "mask") and p.mode == "sparse"]
    for p in sparse_params:
        p.freq = freq
    # Flat fp32 buffers for parameters, gradients and AdamW moments, ordered in three segments: (a) weights with
    # weight decay, (b) sparse weights (no weight decay, masked decay instead), (c) everything else.  Every p.data /
    # p.grad is a view for the whole run; the update is one fused launch per segment, the all-reduce one call.
    sparse_ids = {id(p) for p in sparse_params}
    seg_decay = [p for p in params if p.dim() >= 2 and not hasattr(p, "mask")]
    seg_sparse = [p for p in params if id(p) in sparse_ids]
    seg_other = [p for p in params if p.dim() < 2 or (hasattr(p, "mask") and id(p) not in sparse_ids)]
    order = seg_decay + seg_sparse + seg_other
    pad = lambda n: (n + 3) // 4 * 4     # keep every tensor (and segment) 16-byte aligned
    total = sum(pad(p.numel()) for p in order)
    flat_p = torch.zeros(total, dtype=torch.float32, device=dev)
    flat = torch.zeros(total, dtype=torch.float32, device=dev)
    flat_m, flat_v = torch.zeros_like(flat), torch.zeros_like(flat)
    flat_mask = torch.ones(sum(pad(p.numel()) for p in seg_sparse), dtype=torch.bool, device=dev)
    off, bounds = 0, []
    for seg in (seg_decay, seg_sparse, seg_other):
        start = off
        for p in seg:
            n_ = p.numel()
            flat_p[off:off + n_].copy_(p.data.reshape(-1))
            p.data = flat_p[off:off + n_].view_as(p)
            p.grad = flat[off:off + n_].view_as(p)
            if seg is seg_sparse:
                m_off = off - start
                flat_mask[m_off:m_off + n_].copy_(p.mask.reshape(-1))
                p.mask = flat_mask[m_off:m_off + n_].view_as(p)     # the select kernel refreshes it in place
            off += pad(n_)
        bounds.append((start, off))
    head_grad = None
    if split_head:
        head_grad = torch.zeros(model.wte.weight.shape, dtype=torch.bfloat16, device=dev)
        model.head_grad = head_grad
    step_dev = torch.zeros(1, dtype=torch.float32, device=dev)
    rng_counter = torch.zeros(1, dtype=torch.int64, device=dev)
    set_device_rng_offset(rng_counter if mode == "sparse" else None)
    static_tok = torch.zeros((batch, seq + 1), dtype=torch.long, device=dev)
    gen = torch.Generator(device="cpu").manual_seed(10 if global_stream else 10 + rank)

    def set_phase(reselect):
        # what SparseLinearTranspose.forward looks at: cnt == 0 -> rebuild the compressed copies,
        # counter % freq == 0 -> reselect the mask first
        for p in sparse_params:
            p.cnt = 0
            p.counter = 0 if reselect else 1

    def fwd_bwd():
        flat.zero_()
        rng_counter.add_(1)
        x, y = static_tok[:, :-1], static_tok[:, 1:]
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
            if mode == "sparse":
                sparse.refresh_sparse_layers(model)     # all layers' W / W^T copies in one launch
            loss = model(x, y)
        loss.backward()
        return loss.detach()

    seg_args = list(zip(bounds, (0.1, 0.0, 0.0), (False, True, False)))     # embeddings, sparse weights, everything else
    # 16-bit exchange: every group is cast into this buffer, all-reduced there, and read from there by the update
    stage = torch.empty(total, dtype=reduce_dtype, device=dev) if (world > 1 and reduce_dtype != torch.float32) else None

    def update_segment(which, extra_grad=None):
        (a, b), wd, use_mask = seg_args[which]
        if b > a:
            # after a 16-bit exchange the averaged gradient sits in the 16-bit staging buffer: the update reads it there
            grads = flat if stage is None else stage
            sparse.adamw_masked_decay_(flat_p[a:b], grads[a:b], flat_m[a:b], flat_v[a:b], step=step_dev, lr=lr,
                                       betas=(0.9, 0.95), eps=1e-8, weight_decay=wd,
                                       mask=flat_mask if (use_mask and mode == "sparse") else None,
                                       alpha=alpha if use_mask else 0.0, extra_grad=extra_grad)

    def update_blocks():
        # everything but the embeddings: needs only the block groups' exchanges
        step_dev.add_(1)
        update_segment(1)
        update_segment(2)

    def update_embeddings():
        # the (already averaged) head share of the tied embedding's gradient joins the lookup share inside the update
        # kernel: the token embedding is the first tensor of this segment
        assert seg_decay and seg_decay[0] is model.wte.weight
        update_segment(0, head_grad)

    def update():
        update_blocks()
        update_embeddings()

    def next_tokens():
        if global_stream:
            tok = synthetic_tokens(batch * world, seq, vocab, gen, data)[rank * batch:(rank + 1) * batch].contiguous()
        else:
            tok = synthetic_tokens(batch, seq, vocab, gen, data)
        static_tok.copy_(tok.pin_memory(), non_blocking=True)

    # Gradient exchange.  Group 0 = the last blocks (+ the final layer norm), ..., the last group = the first blocks
    # and the embeddings, whose gradients are complete only when the backward pass ends.  A group's slices of the
    # flat buffer are contiguous inside each segment because parameters keep the model's order there.
    n_groups = max(1, min(comm_groups, layers + 1)) if world > 1 else 1
    emb_alone = split_head and n_groups > 1        # blocks in the first n_groups - 1 groups, embeddings in the last
    n_block_groups = n_groups - 1 if emb_alone else n_groups
    per = (layers + n_block_groups - 1) // n_block_groups
    group_of = {}
    for i, blk in enumerate(model.blocks):
        for p in blk.parameters():
            group_of[id(p)] = n_block_groups - 1 - min(i // per, n_block_groups - 1)
    for p in model.ln_f.parameters():
        group_of[id(p)] = 0
    slices = [[] for _ in range(n_groups)]
    o = 0
    for p in order:
        g_ = group_of.get(id(p), n_groups - 1)
        a, b = o, o + pad(p.numel())
        if slices[g_] and slices[g_][-1][1] == a:
            slices[g_][-1][1] = b
        else:
            slices[g_].append([a, b])
        o = b
    comm = torch.cuda.Stream() if (n_groups > 1 or (world > 1 and split_head)) else None
    n_ready = n_groups - 1      # groups released from inside the graph; the last one waits for the end of backward
    ready = [torch.cuda.Event(external=True) for _ in range(max(n_ready, 0))]
    head_ready = torch.cuda.Event(external=True) if (world > 1 and split_head) else None
    tail = torch.cuda.Event()
    blocks_done = torch.cuda.Event()     # recorded on the exchange stream before the last (embeddings-only) group
    if world > 1 and split_head:
        model.head_ready = head_ready.record
    if n_groups > 1:
        for g_ in range(n_block_groups):
            # the lowest block of group g_ is (n_block_groups - 1 - g_) * per; its gradients are all accumulated once the
            # backward pass has also left the block below it (for block 0: once the embedding sum's gradient exists,
            # which the hook on block 0's input reports)
            below = (n_block_groups - 1 - g_) * per - 1
            if below >= 0:
                model.input_grad_hooks[below] = ready[g_].record
            elif emb_alone:
                model.first_block_hook = ready[g_].record

    averager = None
    if world > 1 and exchange == "copy":
        from sparse.peer import CopyEngineAverage
        if stage is not None:
            raise RuntimeError("run_graphs: the copy-engine exchange works on the float32 gradient buffer")
        averager = CopyEngineAverage()
        averager.add_buffer("flat", flat)
        if head_grad is not None:
            averager.add_buffer("head", head_grad)

    def exchange(a, b):
        if averager is not None:
            averager.average("flat", a, b)
        elif stage is None:
            dist.all_reduce(flat[a:b], op=dist.ReduceOp.AVG)
        else:
            stage[a:b].copy_(flat[a:b])                        # cast; no cast back: the optimizer kernel reads 16 bits
            dist.all_reduce(stage[a:b], op=dist.ReduceOp.AVG)

    # verbose runs time every exchange of the last step on the exchange stream (when it started after the step's first
    # kernel, how long it took): trace[name] = [start event, end event]
    trace = {} if verbose else None
    step_start = torch.cuda.Event(enable_timing=True) if verbose else None

    def mark(name, which):
        if trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            trace.setdefault(name, [None, None])[which] = ev

    def reduce_grads(before_embeddings=None):
        """Issues the exchanges.  ``before_embeddings`` (a callable) is run on the main stream once every group but the
        last, embeddings-only one has been exchanged, i.e. beside that last exchange: the update of all other
        parameters hides the one exchange that cannot overlap the backward pass."""
        overlap_update = before_embeddings is not None and world > 1 and comm is not None and emb_alone
        if not overlap_update and before_embeddings is not None:
            if world > 1:
                reduce_grads()
            before_embeddings()
            return
        if world == 1:
            return
        main = torch.cuda.current_stream()
        if comm is None:
            exchange(0, total)
            if averager is not None:
                averager.finish()
            return
        tail.record(main)
        with torch.cuda.stream(comm):
            if head_ready is not None:
                comm.wait_event(head_ready)
                mark("head", 0)
                if averager is not None:
                    averager.average("head", 0, head_grad.numel())
                else:
                    dist.all_reduce(head_grad, op=dist.ReduceOp.AVG)
                mark("head", 1)
            for g_ in range(n_groups):
                if overlap_update and g_ == n_groups - 1:
                    blocks_done.record(comm)
                comm.wait_event(ready[g_] if g_ < n_ready else tail)
                mark(f"group {g_}", 0)
                for a, b in slices[g_]:
                    exchange(a, b)
                mark(f"group {g_}", 1)
            if averager is not None:
                averager.finish()
        if overlap_update:
            main.wait_event(blocks_done)
            before_embeddings()
        main.wait_stream(comm)

    # eager warm-up on a side stream (allocator, cuBLAS workspaces, optimizer state, kernel attributes)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(3):
            next_tokens()
            set_phase(i == 0)
            fwd_bwd()
            reduce_grads()
            update()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    pool = torch.cuda.graph_pool_handle()
    graphs = {}
    losses_static = {}
    for key in ((True, False) if mode == "sparse" else (False,)):
        set_phase(key)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=pool):
            losses_static[key] = fwd_bwd()
        graphs[key] = g
    g_upd, g_upd_emb = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_upd, pool=pool):
        update_blocks()
    with torch.cuda.graph(g_upd_emb, pool=pool):
        update_embeddings()

    def one_step(i):
        next_tokens()
        key = (mode == "sparse") and (i % freq == 0)
        if step_start is not None:
            step_start.record()
        graphs[key].replay()
        mark("forward + backward graph", 1)
        reduce_grads(g_upd.replay)
        g_upd_emb.replay()
        return losses_static[key]

    it = 0
    for _ in range(warmup):
        one_step(it)
        it += 1
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    losses = []
    e0.record()
    t_cpu = time.perf_counter()
    for _ in range(steps):
        losses.append(one_step(it).clone())
        it += 1
    t_cpu = time.perf_counter() - t_cpu
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    loss_t = torch.stack(losses).float().reshape(-1)
    if world > 1 and return_losses and global_stream:
        dist.all_reduce(loss_t, op=dist.ReduceOp.AVG)     # mean over the ranks' slices = the loss of the whole batch
    loss_list = [float(v) for v in loss_t.cpu()]
    res = {"tokens_per_s": batch * seq * world * steps / (ms * 1e-3), "ms_per_step": ms / steps, "world": world,
           "tokens_per_step": batch * seq * world, "last_loss": loss_list[-1], "mode": mode,
           "loss_finite": all(math.isfinite(v) for v in loss_list), "host_enqueue_ms_per_step": t_cpu * 1e3 / steps,
           "graphs": True}
    if return_losses:
        res["losses"] = loss_list
    if mode == "sparse":
        from sparse.spmm import check_status
        check_status()
    set_device_rng_offset(None)
    if averager is not None:        # peers unmap this rank's buffers before they are freed
        torch.cuda.synchronize()
        averager.close()
        dist.barrier()
    del graphs, g_upd, g_upd_emb, model, flat, flat_p, flat_m, flat_v
    torch.cuda.empty_cache()
    if own_group:
        dist.destroy_process_group()
    if verbose and rank == 0:
        print({k: v for k, v in res.items() if k != "losses"})
        for name, (ev0, ev1) in (trace or {}).items():
            if ev0 is None:
                print(f"  {name}: ends {step_start.elapsed_time(ev1):.2f} ms into the step")
            else:
                print(f"  exchange {name}: starts {step_start.elapsed_time(ev0):.2f} ms into the step, takes "
                      f"{ev0.elapsed_time(ev1):.2f} ms")
    return res


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--mode", default="sparse", choices=["sparse", "dense"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--graphs", action="store_true", help="replay the step from CUDA graphs")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "copy"],
                    help="with --graphs and several ranks: NCCL all-reduce kernels, or peer copies on the DMA engines")
    ap.add_argument("--bf16-exchange", action="store_true", help="with --graphs: exchange the gradients as bf16")
    a = ap.parse_args()
    t0 = time.time()
    if a.graphs:
        r = run_graphs(a.steps, a.warmup, a.mode, batch=a.batch, layers=a.layers, verbose=True, exchange=a.exchange,
                       reduce_dtype=torch.bfloat16 if a.bf16_exchange else torch.float32)
    else:
        r = run(a.steps, a.warmup, a.mode, batch=a.batch, layers=a.layers, verbose=True)
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"wall {time.time() - t0:.1f}s")
