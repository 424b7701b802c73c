"""Headline benchmark: data-parallel training throughput (samples/s) on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

Default model: BERT-base masked-LM (12 layers, hidden 768, 12 heads, FFN 3072, vocab 30522),
seq 128, batch 32 per GPU, bf16, AdamW, synchronous data parallelism (gradient all-reduce every
step), synthetic token ids with 15 % masked positions, random-init weights. `--model resnet20`
and `--model lm` run the other two training configurations. Rank 0 prints ONE JSON line.

`value` is device-timed (CUDA events around exactly K steps, max over ranks) with the step's
inputs already resident; `e2e.value` times the same K steps through the public API including, per
step, the pinned-host -> device copy of that step's inputs and a device -> host read of the loss.
`--impl reference` runs the reference's own C++ shim (`flodl-sys/shim.cpp`, compiled unmodified into
`baseline/_ref/libflodl_shim.so`) with the call sequence of its Rust host; `--impl twin` runs a
plain PyTorch + NCCL restatement of the same sequence as a second opinion.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "twin", "abi"])
    ap.add_argument("--model", default="bert-base", choices=["bert-base", "resnet20", "lm"])
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (0 = the configuration's default)")
    ap.add_argument("--no-graph", action="store_true", help="eager steps instead of one CUDA graph per step")
    ap.add_argument("--comm", default="symm", choices=["symm", "nccl"])
    ap.add_argument("--api", default="engine", choices=["engine", "trainer", "builder"],
                    help="which public API drives the step: engine = TrainEngine (whole-step CUDA graph, the default and the headline); "
                         "trainer = Trainer.setup_head + loss.backward() + graph.step() (the reference's synchronous path, bert-base); "
                         "builder = Trainer.builder(...).run().join() with the coordinator in the loop (the reference's asynchronous path, lm)")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) during the timed region."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), 0
        self._stop_ev = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {getattr(nv, k): k for k in dir(nv) if k.startswith("nvmlClocksEventReason") or k.startswith("nvmlClocksThrottleReason")}
            while not self._stop_ev.is_set():
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                for bit, name in names.items():
                    if isinstance(bit, int) and bit and mask & bit and bit & (bit - 1) == 0:
                        self.reasons.add(name.replace("nvmlClocksEventReason", "").replace("nvmlClocksThrottleReason", ""))
                time.sleep(0.01)
        except Exception as e:  # NVML missing: report that instead of numbers
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._stop_ev.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        rs = sorted(r for r in self.reasons if r not in ("None", "GpuIdle", "ApplicationsClocksSetting"))
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz or None, "reasons": rs, "samples": len(s)}


# ---------------------------------------------------------------------------------------- workloads
def make_bert(args, dev):
    import torch
    from flodl_b200 import nn
    from flodl_b200.hf.models.bert import BertConfig, BertForMaskedLM, build_extended_attention_mask
    cfg = BertConfig.bert_base_uncased()
    B, S = (args.batch or 32), 128
    head = BertForMaskedLM.on_device(cfg, dev)
    head.graph().set_training(True)
    # BERT's own initialisation (normal(0, initializer_range = 0.02) matrices and embeddings, zero biases, unit
    # LayerNorm gains), as the reference arm uses: the first loss is then ln(vocab) ~ 10.3
    with torch.no_grad():
        for name, p in head.graph().named_parameters():
            t = p.t if hasattr(p, "t") else p
            if t.dim() >= 2:
                t.normal_(0.0, 0.02)
            elif name.endswith("LayerNorm.weight"):
                t.fill_(1.0)
            else:
                t.zero_()

    def batch(gen):
        ids = torch.randint(0, cfg.vocab_size, (B, S), generator=gen)
        labels = torch.full((B, S), -100, dtype=torch.long)
        m = torch.rand(B, S, generator=gen) < 0.15
        labels[m] = ids[m]
        ids = ids.clone()
        ids[m] = 103  # [MASK]
        pos = torch.arange(S).expand(B, S).contiguous()
        tt = torch.zeros(B, S, dtype=torch.long)
        am = torch.ones(B, S, dtype=torch.long)
        return [ids, pos, tt, am, labels]

    def step_fn(ids, pos, tt, am, labels):
        return head.compute_loss([ids, pos, tt, build_extended_attention_mask(am)], labels)

    opt = lambda ps: nn.AdamW(ps, 1e-4, 0.01)
    desc = {"model": "bert-base-mlm (12x768, 12 heads, ffn 3072, vocab 30522)", "seq_len": S, "optimizer": "AdamW lr 1e-4 wd 0.01",
            "dropout": 0.1}
    return head.graph(), step_fn, batch, opt, B, desc, None


def make_lm(args, dev):
    import torch
    from flodl_b200 import nn
    from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
    cfg = DecoderLMConfig(vocab_size=32000, d_model=512, n_layers=6, n_heads=8, d_ff=2048, max_seq=256, dropout=0.0)
    B, S = (args.batch or 32), 256
    model = DecoderLM(cfg, dev)
    model.set_training(True)

    def batch(gen):
        ids = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen)
        return [ids[:, :-1].contiguous(), ids[:, 1:].contiguous()]

    def step_fn(x, y):
        return model.loss(x, y)

    opt = lambda ps: nn.AdamW(ps, 3e-4, 0.01)
    desc = {"model": "decoder-lm (6x512, 8 heads, ffn 2048, vocab 32000, pre-LN, GELU)", "seq_len": S, "optimizer": "AdamW lr 3e-4"}
    return model, step_fn, batch, opt, B, desc, None


def make_resnet(args, dev):
    import torch
    from flodl_b200 import nn
    from flodl_b200.models.resnet import resnet20
    B = args.batch or 128
    model = resnet20(10, dev)
    model.set_training(True)

    def batch(gen):
        return [torch.randn(B, 3, 32, 32, generator=gen), torch.randint(0, 10, (B,), generator=gen)]

    def step_fn(x, y):
        from flodl_b200.autograd import Variable
        return nn.cross_entropy_loss(model.forward(Variable.wrap(x.to(torch.bfloat16))), Variable.wrap(y))

    opt = lambda ps: nn.SGD(ps, 0.1, 0.9, 1e-4)
    desc = {"model": "resnet20-cifar (3 stages x 3 BasicBlocks, 16/32/64 ch, BatchNorm)", "seq_len": None, "optimizer": "SGD lr 0.1 m 0.9 wd 1e-4"}
    return model, step_fn, batch, opt, B, desc, 3340.0   # reference's published solo-GPU figure (derived), samples/s


AVG_EVERY = 8

MAKERS = {"bert-base": make_bert, "lm": make_lm, "resnet20": make_resnet}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from flodl_b200 import nn, ops
    from flodl_b200.parallel import comm
    from flodl_b200.parallel.engine import TrainEngine

    comm.init_process_group(timeout_s=180.0)
    world, rank = comm.world_size(), comm.rank()
    local = comm.local_rank()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    torch.manual_seed(1234)
    guard = nn.AutocastGuard(torch.bfloat16)
    model, step_fn, batch, opt, B, desc, published = MAKERS[args.model](args, dev)
    # the decoder LM runs the asynchronous-DDP recipe: local AdamW steps, parameters averaged
    # across replicas every AVG_EVERY steps (fused peer-memory kernel); the others all-reduce gradients
    local_sgd = args.model == "lm" and world > 1
    eng = TrainEngine(model, opt, comm_backend=args.comm, grad_sync=not local_sgd, param_staging=local_sgd and args.comm == "symm")
    gen = torch.Generator().manual_seed(100 + rank)
    pool = [[t.pin_memory() for t in batch(gen)] for _ in range(8)]
    dev_pool = [[t.to(dev) for t in b] for b in pool]
    h2d = sum(t.numel() * t.element_size() for t in pool[0])
    loss_host = torch.zeros(1).pin_memory()

    ops.FLAGS.count_launches = True
    use_graph = not args.no_graph
    if use_graph:
        ops.FLAGS.launches = 0
        eng.capture(step_fn, dev_pool[0], warmup=3)
        per_step = ops.FLAGS.launches // 4 + eng.sync.launch_count // 4 + 1   # 3 warm-ups + the captured step; + optimizer
        one = lambda inputs: eng.replay(inputs)
    else:
        ops.FLAGS.launches = 0
        eng.step(lambda: step_fn(*dev_pool[0]))
        per_step = ops.FLAGS.launches + eng.sync.launch_count + 1
        one = lambda inputs: eng.step(lambda: step_fn(*inputs))
    ops.FLAGS.count_launches = False
    if eng.symm_bufs is not None:
        per_step += 1                      # the per-step buffer broadcast
    extra = [0]
    done = [0]

    def run(inputs):
        loss = one(inputs)
        done[0] += 1
        if local_sgd and done[0] % AVG_EVERY == 0:
            eng.average_params()
            extra[0] += 1
        return loss

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gmax(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, dist.ReduceOp.MAX)
        return float(t.item())

    first_loss = float("nan")
    for i in range(max(args.warmup, 3)):
        l0 = run(dev_pool[i % len(dev_pool)])
        if i == 0:
            first_loss = float(l0.float().item())
    sync_all()
    eng.check()

    # ---- device-timed: inputs resident, CUDA events around exactly K steps -----------------------
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for i in range(args.steps):
        loss = run(dev_pool[i % len(dev_pool)])
    e1.record()
    sync_all()
    ms_dev = gmax(e0.elapsed_time(e1)) / args.steps

    # ---- end to end: pinned H2D of the step's inputs + D2H read of the loss, every step ----------
    sync_all()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        host = pool[i % len(pool)]
        loss = run(host if use_graph else [t.to(dev, non_blocking=True) for t in host])
        loss_host.copy_(loss.reshape(1).float(), non_blocking=False)
        last = float(loss_host[0])
    sync_all()
    ms_e2e = gmax((time.perf_counter() - t0) * 1e3) / args.steps
    clocks = sampler.stop()
    eng.check()

    # ---- replicas must still agree: compare a checksum of the flat parameter buffer across ranks --
    params_in_sync = None
    if world > 1:
        if local_sgd:
            eng.average_params()          # Local SGD replicas only agree right after an averaging round
        p = eng.flat.params
        sums = torch.stack([p.double().sum(), p.double().abs().sum(), p[:: max(1, p.numel() // 4096)].double().pow(2).sum()])
        allsums = [torch.empty_like(sums) for _ in range(world)]
        dist.all_gather(allsums, sums)
        params_in_sync = all(torch.equal(allsums[0], a) for a in allsums)

    if rank == 0:
        value = world * B / (ms_dev / 1e3)
        e2e = world * B / (ms_e2e / 1e3)
        out = {
            "metric": "DDP samples/sec (max over ranks)", "value": round(value, 2), "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_dev, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (round(value / published, 3) if published else None), "dtype": "bf16",
            "data": "synthetic (random token ids / images of the named shape, random-init weights)", "impl": "ours",
            "config": dict(desc, global_batch=world * B, per_gpu_batch=B, parallelism=f"dp{world}",
                           step="one CUDA graph per step" if use_graph else "eager",
                           grad_sync=("none" if world == 1 else f"parameter averaging every {AVG_EVERY} steps ({args.comm})" if local_sgd else args.comm),
                           l2="working set (weights + optimizer state + activations, > 1 GB) exceeds the 126 MB L2; no flush needed"),
            "clocks": clocks,
            "e2e": {"value": round(e2e, 2), "unit": "samples/s", "ms_per_step": round(ms_e2e, 4), "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(per_step * args.steps + (args.steps // AVG_EVERY if local_sgd else 0)),
            "first_loss": round(first_loss, 4), "final_loss": round(last, 4), "params_in_sync": params_in_sync,
            "collective": (None if world == 1 else ("this repository's kernels over " + ("NVLS multimem" if getattr(eng.symm_grads or eng.symm_params, "nvls", False)
                           else "peer loads/stores") if args.comm == "symm" else "NCCL")),
        }
        print(json.dumps(out), flush=True)
    guard.release()
    if world > 1:
        dist.barrier()
        comm.destroy_process_group()


def run_trainer_api(args):
    """The reference-shaped synchronous path (flodl/src/distributed/ddp.rs:900-923): `Trainer.setup_head`, then per batch
    forward, `loss.backward()`, `graph.step()`; gradients are exchanged by `DistributedState` (bucketed, overlapped with
    backward), nothing is captured into a CUDA graph."""
    import torch
    import torch.distributed as dist
    from flodl_b200 import nn
    from flodl_b200.parallel import comm
    from flodl_b200.parallel.ddp import Trainer
    comm.init_process_group(timeout_s=180.0)
    world, rank, local = comm.world_size(), comm.rank(), comm.local_rank()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    torch.manual_seed(1234)
    guard = nn.AutocastGuard(torch.bfloat16)
    graph, step_fn, batch, opt, B, desc, _ = make_bert(args, dev)
    Trainer.setup_with(graph, None, opt, None, scatter=False)
    gen = torch.Generator().manual_seed(100 + rank)
    pool = [[t.pin_memory() for t in batch(gen)] for _ in range(8)]

    def one(host):
        inputs = [t.to(dev, non_blocking=True) for t in host]
        if graph._ddp is not None:
            graph._ddp.begin_batch(B)
        loss = step_fn(*inputs)
        loss.backward()
        graph.step()
        return loss

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for i in range(max(args.warmup, 3)):
        one(pool[i % 8])
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = 0.0
    for i in range(args.steps):
        last = one(pool[i % 8])
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank == 0:
        print(json.dumps({"metric": "DDP samples/sec (max over ranks)", "api": "Trainer.setup_head + graph.step()", "impl": "ours", "value": round(world * B / (ms / 1e3), 2),
                          "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
                          "config": dict(desc, per_gpu_batch=B, parallelism=f"dp{world}", step="eager, inputs copied from pinned host memory every step"),
                          "final_loss": round(float(last.item()), 4)}), flush=True)
    guard.release()
    if world > 1:
        dist.barrier()
        comm.destroy_process_group()


def run_builder_api(args):
    """The reference-shaped asynchronous path (flodl/src/distributed/ddp_run/orchestrator.rs:1339-1359):
    `Trainer.builder(...).run().join()`: one worker per rank, the coordinator on rank 0, parameters averaged every
    AVG_EVERY batches (pinned cadence). Throughput comes from the coordinator's own epoch clock."""
    import torch
    from flodl_b200 import nn
    from flodl_b200.data import TensorDataSet
    from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
    from flodl_b200.parallel import comm
    from flodl_b200.parallel.ddp import Trainer
    from flodl_b200.parallel.ddp_run import ApplyPolicy, AverageBackend
    comm.init_process_group(timeout_s=180.0)
    world, rank = comm.world_size(), comm.rank()
    torch.cuda.set_device(comm.local_rank())
    B, S = (args.batch or 32), 256
    cfg = DecoderLMConfig(vocab_size=32000, d_model=512, n_layers=6, n_heads=8, d_ff=2048, max_seq=256, dropout=0.0)
    batches_per_epoch = max(AVG_EVERY, (args.steps // AVG_EVERY) * AVG_EVERY)
    n = batches_per_epoch * B * world
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (n, S + 1), generator=g)
    ds = TensorDataSet(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())

    def factory(d):
        torch.manual_seed(11)
        return DecoderLM(cfg, d)
    epochs = 3
    b = (Trainer.builder(factory, lambda ps: nn.AdamW(ps, 3e-4, 0.01), lambda m, batch: m.loss(batch[0], batch[1]))
         .dataset(ds).batch_size(B).num_epochs(epochs).lr_scale_ratio(0.0).policy(ApplyPolicy.Cadence).backend(AverageBackend.Nccl)
         .anchor(AVG_EVERY).max_anchor(AVG_EVERY).cuda_graph(True))
    with nn.AutocastGuard(torch.bfloat16):
        h = b.run()
        state = h.join()
    if rank == 0:
        ms = h.poll_metrics()
        best = min(m.epoch_ms for m in ms[1:]) if len(ms) > 1 else ms[0].epoch_ms      # the first epoch pays for set-up and capture
        print(json.dumps({"metric": "DDP samples/sec (coordinator epoch clock)", "api": "Trainer.builder(...).run().join()", "impl": "ours",
                          "value": round(n / (best / 1e3), 2), "unit": "samples/s", "n_gpus": world, "epochs": epochs,
                          "batches_per_epoch_per_rank": batches_per_epoch, "ms_per_step": round(best / batches_per_epoch, 4),
                          "config": {"model": "decoder-lm (6x512, 8 heads, ffn 2048, vocab 32000, pre-LN, GELU)", "seq_len": S, "per_gpu_batch": B,
                                     "grad_sync": f"parameter averaging every {AVG_EVERY} batches, coordinator in the loop"},
                          "errors": [str(e) for e in h.errors()], "final_loss": round(ms[-1].avg_loss, 4), "trained": state is not None}), flush=True)
    comm.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        # the reference's own C++ shim (compiled unmodified into baseline/_ref), driven through its C ABI;
        # nothing of this repository's package or kernels is imported on this path
        from baseline import reference_arm
        reference_arm.run(args, ClockSampler)
        return
    if args.impl == "abi":
        # the same host call sequence as the reference arm, over this repository's drop-in `flodl_*` C library
        from baseline import reference_arm
        shim = os.path.join(os.path.dirname(os.path.abspath(__file__)), "flodl_b200", "libflodl_b200_shim.so")
        reference_arm.run(args, ClockSampler, shim_path=shim)
        return
    if args.impl == "twin":
        from baseline import twin
        twin.run(args)
        return
    if args.api == "trainer":
        return run_trainer_api(args)
    if args.api == "builder":
        return run_builder_api(args)
    run_ours(args)


if __name__ == "__main__":
    main()
