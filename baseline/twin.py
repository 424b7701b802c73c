"""PyTorch + NCCL restatement of the reference's training call sequence (the "twin" baseline).

The reference is a Rust front-end over libtorch: every op is an ATen call and data parallelism is
one `ncclAllReduce(Avg)` per parameter after backward on the default stream, one `ncclBroadcast`
per buffer, then the optimizer (flodl/src/distributed/ddp.rs:133-167,
flodl/src/graph/distributed.rs:405-437). This module issues exactly those calls through PyTorch:
`F.linear`, `F.scaled_dot_product_attention`, `F.layer_norm`, `F.gelu`, `F.cross_entropy`,
`F.embedding`, `F.conv2d`, `F.batch_norm` under bf16 autocast, `torch._fused_adamw_` (what
`_fused_adamw_` resolves to) or the per-parameter SGD loop of sgd.rs:132-172. None of this
repository's kernels, models or engine are used here.
"""
from __future__ import annotations

import json
import math
import time

import torch
import torch.distributed as dist
import torch.nn as tnn
import torch.nn.functional as F


class Layer(tnn.Module):
    def __init__(s, H, heads, I, p):
        super().__init__()
        s.q, s.k, s.v, s.o = (tnn.Linear(H, H) for _ in range(4))
        s.ln1, s.ln2 = tnn.LayerNorm(H, eps=1e-12), tnn.LayerNorm(H, eps=1e-12)
        s.up, s.down = tnn.Linear(H, I), tnn.Linear(I, H)
        s.heads, s.p = heads, p

    def forward(s, x, mask):
        B, S, H = x.shape
        sp = lambda t: t.reshape(B, S, s.heads, H // s.heads).transpose(1, 2)
        ctx = F.scaled_dot_product_attention(sp(s.q(x)), sp(s.k(x)), sp(s.v(x)), attn_mask=mask, dropout_p=s.p if s.training else 0.0)
        a = F.dropout(s.o(ctx.transpose(1, 2).reshape(B, S, H)), s.p, s.training)
        h = s.ln1(a + x)
        f = F.dropout(s.down(F.gelu(s.up(h))), s.p, s.training)
        return s.ln2(f + h)


class BertMLM(tnn.Module):
    def __init__(s, V=30522, H=768, L=12, heads=12, I=3072, P=512, p=0.1):
        super().__init__()
        s.we, s.pe, s.te = tnn.Embedding(V, H, padding_idx=0), tnn.Embedding(P, H), tnn.Embedding(2, H)
        s.ln = tnn.LayerNorm(H, eps=1e-12)
        s.layers = tnn.ModuleList(Layer(H, heads, I, p) for _ in range(L))
        s.t_dense, s.t_ln = tnn.Linear(H, H), tnn.LayerNorm(H, eps=1e-12)
        s.dec_bias = tnn.Parameter(torch.zeros(V))
        s.p = p

    def forward(s, ids, pos, tt, am, labels):
        mask = ((1.0 - am.float()) * -1e4).reshape(am.shape[0], 1, 1, am.shape[1])
        x = F.dropout(s.ln(s.we(ids) + s.pe(pos) + s.te(tt)), s.p, s.training)
        mask = mask.to(x.dtype) if x.dtype != torch.float32 else mask
        for l in s.layers:
            x = l(x, mask.to(torch.bfloat16) if torch.is_autocast_enabled() else mask)
        x = s.t_ln(F.gelu(s.t_dense(x)))
        logits = F.linear(x, s.we.weight, s.dec_bias)
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1), ignore_index=-100)


def run(args):
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)
    if args.model != "bert-base":
        if rank == 0:
            print(json.dumps({"impl": "twin", "unavailable": f"the PyTorch restatement covers bert-base only; `--impl reference` runs {args.model} "
                                                              "on the reference's own shim"}))
        return
    B, S, V = (args.batch or 32), 128, 30522
    model = BertMLM().to(dev).train()
    params = [p for p in model.parameters()]
    if world > 1:
        for p in params:
            dist.broadcast(p.data, 0)
    opt = torch.optim.AdamW(params, lr=1e-4, weight_decay=0.01, fused=True)
    gen = torch.Generator().manual_seed(100 + rank)

    def batch():
        ids = torch.randint(0, V, (B, S), generator=gen)
        labels = torch.full((B, S), -100, dtype=torch.long)
        m = torch.rand(B, S, generator=gen) < 0.15
        labels[m] = ids[m]
        ids = ids.clone(); ids[m] = 103
        return [t.pin_memory() for t in (ids, torch.arange(S).expand(B, S).contiguous(), torch.zeros(B, S, dtype=torch.long),
                                          torch.ones(B, S, dtype=torch.long), labels)]

    pool = [batch() for _ in range(8)]
    dev_pool = [[t.to(dev) for t in b] for b in pool]

    def step(inputs):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(*inputs)
        loss.backward()
        if world > 1:
            for p in params:                      # one collective per parameter, after backward
                if p.grad is not None:
                    dist.all_reduce(p.grad, dist.ReduceOp.AVG)
        opt.step()
        return loss.detach()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gmax(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(max(args.warmup, 3)):
        step(dev_pool[i % 8])
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(dev_pool[i % 8])
    e1.record()
    sync()
    ms = gmax(e0.elapsed_time(e1)) / args.steps
    sync()
    t0 = time.perf_counter()
    for i in range(args.steps):
        loss = step([t.to(dev, non_blocking=True) for t in pool[i % 8]])
        last = float(loss.item())
    sync()
    ms_e2e = gmax((time.perf_counter() - t0) * 1e3) / args.steps
    if rank == 0:
        print(json.dumps({"impl": "twin", "metric": "DDP samples/sec (max over ranks)", "value": round(world * B / ms * 1e3, 2),
                          "unit": "samples/s", "n_gpus": world, "steps": args.steps, "ms_per_step": round(ms, 4),
                          "e2e": {"value": round(world * B / ms_e2e * 1e3, 2), "ms_per_step": round(ms_e2e, 4)},
                          "config": {"model": "bert-base-mlm", "per_gpu_batch": B, "seq_len": S, "path": "ATen ops + per-parameter ncclAllReduce + fused AdamW"},
                          "final_loss": round(last, 4)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
