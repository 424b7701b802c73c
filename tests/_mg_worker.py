"""Worker for the multi-GPU tests: launched with torch.distributed.run, one rank per GPU.
Checks the symmetric-memory collectives against fp64 host references and prints `MG_OK` on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flodl_b200.parallel import comm  # noqa: E402


def gather_all(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return out


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "collectives"
    comm.init_process_group()
    rank, world = comm.rank(), comm.world_size()
    dev = torch.device("cuda", comm.local_rank())
    torch.cuda.set_device(dev)
    torch.manual_seed(7 + rank)
    if mode == "collectives":
        n = 1 << 20
        buf = comm.SymmetricBuffer(n * 4 + 4096, timeout_s=5.0)
        # ---- two-shot all-reduce, fp32 and bf16, several sizes incl. odd vector counts
        for dtype in (torch.float32, torch.bfloat16):
            for numel in (8 * 3, 1024, 8 * 12345, n if dtype == torch.float32 else 2 * n):
                v = buf.view(dtype, 0, numel)
                x = (torch.randn(numel, device=dev) * 1e-3).to(dtype)
                v.copy_(x)
                ref = torch.stack([g.double() for g in gather_all(x)]).mean(0)
                torch.cuda.synchronize(); dist.barrier()
                buf.all_reduce(0, numel, dtype, blocks=8)
                torch.cuda.synchronize()
                buf.check()
                tol = 1e-6 if dtype == torch.float32 else 2e-5
                err = (v.double() - ref).abs().max().item()
                assert err < tol, (str(dtype), numel, err)
                # every rank must hold bit-identical results
                allv = gather_all(v.clone())
                assert all(torch.equal(allv[0], a) for a in allv)
        # ---- weighted (unbalanced shards)
        numel = 4096
        w = [float(i + 1) for i in range(world)]
        w = [a / sum(w) for a in w]
        v = buf.view(torch.float32, 0, numel)
        x = torch.randn(numel, device=dev)
        v.copy_(x)
        ref = sum(wi * g.double() for wi, g in zip(w, gather_all(x)))
        torch.cuda.synchronize(); dist.barrier()
        buf.all_reduce(0, numel, torch.float32, weights=w, blocks=4)
        torch.cuda.synchronize()
        assert (v.double() - ref).abs().max().item() < 1e-5
        # ---- one-shot with cast: bf16 in, fp32 out
        numel = 8 * 1000
        v = buf.view(torch.bfloat16, 0, numel)
        x = torch.randn(numel, device=dev).bfloat16()
        v.copy_(x)
        out = torch.empty(numel, device=dev)
        ref = torch.stack([g.double() for g in gather_all(x)]).mean(0)
        torch.cuda.synchronize(); dist.barrier()
        buf.all_reduce_into(0, numel, torch.bfloat16, out, blocks=4)
        torch.cuda.synchronize()
        buf.check()
        assert (out.double() - ref).abs().max().item() < 1e-5
        # ---- broadcast
        numel = 4 * 7777
        v = buf.view(torch.float32, 0, numel)
        x = torch.randn(numel, device=dev)
        v.copy_(x)
        root_vals = gather_all(x)[world - 1]
        torch.cuda.synchronize(); dist.barrier()
        buf.broadcast(0, numel * 4, root=world - 1, blocks=8)
        torch.cuda.synchronize()
        assert torch.equal(v, root_vals)
        # a message above 1 MB: with more than two ranks this takes the scatter + all-gather path
        numel = 4 * 250_003
        v = buf.view(torch.float32, 0, numel)
        x = torch.randn(numel, device=dev)
        v.copy_(x)
        root_vals = gather_all(x)[0]
        torch.cuda.synchronize(); dist.barrier()
        buf.broadcast(0, numel * 4, root=0, blocks=24)
        torch.cuda.synchronize()
        buf.check()
        assert torch.equal(v, root_vals)
        # ---- parameter averaging + lerp + divergence
        numel = 4 * 50001
        stage = comm.SymmetricBuffer(numel * 4, timeout_s=5.0)
        v = buf.view(torch.float32, 0, numel)
        x = torch.randn(numel, device=dev)
        v.copy_(x)
        p16 = torch.empty(numel, device=dev, dtype=torch.bfloat16)
        mean = torch.stack([g.double() for g in gather_all(x)]).mean(0)
        torch.cuda.synchronize(); dist.barrier()
        out2 = buf.comm.param_average(stage.comm, numel, None, 1.0, p16, 16)
        torch.cuda.synchronize()
        buf.check()
        assert (v.double() - mean).abs().max().item() < 1e-6
        assert (p16.float() - v).abs().max().item() < 2e-2
        d2 = ((mean - x.double()) ** 2).sum().item()
        n2 = (mean ** 2).sum().item()
        assert abs(out2[0].item() - d2) / d2 < 1e-3 and abs(out2[1].item() - n2) / n2 < 1e-3
        # ---- bounded wait: a barrier nobody else joins must time out with a status, not hang
        # (plain peer memory for this one: nothing that is meant to time out runs on a multicast binding)
        lone = comm.SymmetricBuffer(4096, timeout_s=0.3, nvls=False)
        torch.cuda.synchronize(); dist.barrier()
        if rank == 0:
            lone.barrier()
            torch.cuda.synchronize()
            assert lone.status() == 4, lone.status()
            z = torch.ones(4, device=dev).sum().item()      # the context is still usable
            assert z == 4.0
        dist.barrier()
        # the give-up was published to every peer: their next launch on this buffer returns at once
        if rank != 0:
            lone.barrier()
            torch.cuda.synchronize()
            assert lone.status() == 7, lone.status()
        dist.barrier()
        # recover() on every rank re-arms the buffer: the same barrier, joined by all, now passes
        lone.recover()
        lone.barrier()
        torch.cuda.synchronize()
        assert lone.status() == 0, lone.status()
        # ---- world sizes that are not powers of two use the same kernels (peer path)
        assert buf.nvls == (os.environ.get("FLODL_B200_NVLS", "1") != "0" and buf.C.multicast_supported(dev.index)), buf.nvls
    elif mode == "engine":
        from flodl_b200 import nn
        from flodl_b200.hf.models.bert import BertConfig, BertForMaskedLM, build_extended_attention_mask
        from flodl_b200.parallel.engine import TrainEngine
        torch.manual_seed(100 + rank)   # different init per rank: the engine must broadcast rank 0's
        cfg = BertConfig(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                         max_position_embeddings=128, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
        head = BertForMaskedLM.on_device(cfg, dev)
        head.graph().set_training(True)
        B, S = 4, 128
        g = torch.Generator().manual_seed(5 + rank)
        ids = torch.randint(0, 512, (B, S), generator=g).to(dev)
        labels = torch.full((B, S), -100, dtype=torch.long)
        labels[:, ::5] = ids.cpu()[:, ::5]
        labels = labels.to(dev)
        pos = torch.arange(S, device=dev).expand(B, S).contiguous()
        tt = torch.zeros(B, S, dtype=torch.long, device=dev)
        mask = build_extended_attention_mask(torch.ones(B, S, device=dev))
        with nn.AutocastGuard(torch.bfloat16):
            eng = TrainEngine(head.graph(), lambda ps: nn.AdamW(ps, 1e-3, 0.0), bucket_mb=0.25)
            p0 = gather_all(eng.flat.params.clone())
            assert all(torch.equal(p0[0], a) for a in p0), "parameters not synchronised after broadcast"
            eng.sync.enable_timing()
            for step in range(4):
                eng.step(lambda: head.compute_loss([ids, pos, tt, mask], labels))
                torch.cuda.synchronize()
                eng.check()
                gs = gather_all(eng.flat.grads.clone())
                assert all(torch.equal(gs[0], a) for a in gs), f"gradients differ across ranks at step {step}"
                ps = gather_all(eng.flat.params.clone())
                assert all(torch.equal(ps[0], a) for a in ps), f"parameters diverged at step {step}"
            assert len(eng.sync.buckets) > 1 and eng.sync.launch_count >= 4 * len(eng.sync.buckets)
            rep = eng.sync.bucket_report()
            assert [r["bucket"] for r in rep] == list(range(len(eng.sync.buckets))) and all(r["ms"] > 0 and r["launches"] == 4 for r in rep), rep
            assert sum(r["bytes"] for r in rep) == eng.flat.total * 4
    elif mode == "giveup":
        # A rank that is late by more than the collectives' time limit: the others must not apply
        # un-reduced gradients. The fused optimizer is predicated on the exchange's status word, so
        # parameters stay as they were on every rank; the next check raises; recover() re-arms.
        import time
        from flodl_b200 import nn
        from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
        from flodl_b200.parallel.engine import TrainEngine
        from flodl_b200.tensor import TensorError
        cfg = DecoderLMConfig(vocab_size=256, d_model=64, n_layers=2, n_heads=2, d_ff=128, max_seq=64, dropout=0.0)
        torch.manual_seed(3)
        model = DecoderLM(cfg, dev)
        model.set_training(True)
        g = torch.Generator().manual_seed(20 + rank)
        ids = torch.randint(0, 256, (4, 65), generator=g).to(dev)
        x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
        with nn.AutocastGuard(torch.bfloat16):
            eng = TrainEngine(model, lambda ps: nn.AdamW(ps, 1e-2, 0.0), bucket_mb=0.05, comm_timeout_s=0.4)
            assert eng.symm_grads is not None and not eng.symm_grads.nvls
            for _ in range(2):
                eng.step(lambda: model.loss(x, y))
            torch.cuda.synchronize(); eng.check(); dist.barrier()
            before = eng.flat.params.clone()
            if rank == world - 1:
                time.sleep(1.5)                       # the failure is made on the host: this rank is late
            raised = False
            try:
                eng.step(lambda: model.loss(x, y))
                torch.cuda.synchronize()
                eng.check()
            except TensorError:
                raised = True
            assert raised, "a collective that gave up must surface as an exception"
            torch.cuda.synchronize()
            assert torch.equal(eng.flat.params, before), "parameters changed although the gradient exchange gave up"
            eng.recover()
            eng.step(lambda: model.loss(x, y))
            torch.cuda.synchronize()
            eng.check()
            ps = gather_all(eng.flat.params.clone())
            assert all(torch.equal(ps[0], a) for a in ps), "replicas differ after recovery"
            assert not torch.equal(eng.flat.params, before)
    elif mode == "resnet_buffers":
        # BatchNorm statistics differ per rank (different data); after every step all ranks must
        # hold rank 0's running statistics, through the one-launch pull broadcast
        from flodl_b200 import nn
        from flodl_b200.autograd import Variable
        from flodl_b200.models.resnet import resnet20
        from flodl_b200.parallel.engine import TrainEngine
        torch.manual_seed(1)
        model = resnet20(10, dev)
        model.set_training(True)
        g = torch.Generator().manual_seed(50 + rank)
        x = torch.randn(16, 3, 32, 32, generator=g).to(dev).bfloat16()
        y = torch.randint(0, 10, (16,), generator=g).to(dev)
        with nn.AutocastGuard(torch.bfloat16):
            eng = TrainEngine(model, lambda ps: nn.SGD(ps, 0.05, 0.9, 1e-4))
            assert eng.symm_bufs is not None and eng._buf_bytes > 0
            for step in range(3):
                eng.step(lambda: nn.cross_entropy_loss(model.forward(Variable.wrap(x)), Variable.wrap(y)))
                torch.cuda.synchronize()
                eng.check()
                pack = torch.cat([b.reshape(-1) for b in eng._float_bufs])
                allb = gather_all(pack)
                assert all(torch.equal(allb[0], a) for a in allb), f"buffers differ across ranks at step {step}"
                assert pack.abs().sum().item() > 0
    elif mode == "graph_ddp":
        # the reference's user-facing path: Trainer.setup + model.forward(global batch) + model.step()
        from flodl_b200 import nn
        from flodl_b200.graph import FlowBuilder
        from flodl_b200.parallel.ddp import Trainer

        def build(seed):
            torch.manual_seed(seed)
            return (FlowBuilder.from_(nn.Linear.on_device(64, 128, dev)).through(nn.GELU()).through(nn.LayerNorm.on_device(128, dev))
                    .through(nn.Linear.on_device(128, 64, dev)).build())
        m = build(100 + rank)
        Trainer.setup(m, None, lambda ps: nn.Adam(ps, 1e-2))
        assert m.is_distributed() and m.world_size() == world
        ref = build(100)
        ropt = nn.Adam(ref.parameters(), 1e-2)
        gen = torch.Generator().manual_seed(9)
        X = torch.randn(5, 8 * world, 64, generator=gen).to(dev)
        Y = torch.randn(5, 8 * world, 64, generator=gen).to(dev)
        for step in range(5):
            out = m.forward(X[step])
            nn.mse_loss(out, Y[step][rank * 8:(rank + 1) * 8]).backward()
            m.step()
            nn.mse_loss(ref.forward(X[step]), Y[step]).backward()
            ropt.step()
            ropt.zero_grad()
        torch.cuda.synchronize()
        for (n1, p1), (_, p2) in zip(m.named_parameters(), ref.named_parameters()):
            err = (p1.t.detach() - p2.t.detach()).abs().max().item()
            assert err < 5e-3, (n1, err)       # bf16-free fp32 path: only reduction order differs
        ps = gather_all(m._ddp.flat.params.clone())
        assert all(torch.equal(ps[0], a) for a in ps)
    elif mode in ("async_fixed", "async_cadence", "async_cpu"):
        from flodl_b200 import nn
        from flodl_b200.data import TensorDataSet
        from flodl_b200.models.gpt import DecoderLM, DecoderLMConfig
        from flodl_b200.parallel.ddp import Trainer
        from flodl_b200.parallel.ddp_run import ApplyPolicy, AverageBackend
        cfg = DecoderLMConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=2, d_ff=256, max_seq=128, dropout=0.0)
        gen = torch.Generator().manual_seed(3)
        base = torch.randint(0, 512, (64,), generator=gen)
        ids = base.repeat(40 * 129 // 64 + 1)[:40 * 129].view(40, 129)      # a periodic stream: learnable quickly
        ds = TensorDataSet(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())

        def factory(d):
            torch.manual_seed(11)
            return DecoderLM(cfg, d)

        def train_fn(model, batch):
            return model.loss(batch[0], batch[1])
        b = (Trainer.builder(factory, lambda ps: nn.AdamW(ps, 2e-3, 0.0), train_fn).dataset(ds).batch_size(4).num_epochs(4)
             .lr_scale_ratio(0.0))
        if mode == "async_fixed":
            b = b.policy(ApplyPolicy.Cadence).backend(AverageBackend.Nccl).anchor(2).max_anchor(2)
        elif mode == "async_cadence":
            b = b.policy(ApplyPolicy.Cadence).backend(AverageBackend.Nccl)
        else:
            b = b.policy(ApplyPolicy.Async).backend(AverageBackend.Cpu)
        with nn.AutocastGuard(torch.bfloat16):
            h = b.run()
            state = h.join()
        assert state is not None and len(state.params) > 0 and not h.errors(), h.errors()
        if rank == 0:
            ms = h.poll_metrics()
            assert [m.epoch for m in ms] == [0, 1, 2, 3], [m.epoch for m in ms]
            assert ms[-1].avg_loss < 0.7 * ms[0].avg_loss, [m.avg_loss for m in ms]
        w = h._gpu_workers[0]
        if mode != "async_cpu":
            assert w.current_version() > 0, "no averaging round ran"
            assert w.engine.symm_stage is not None, "the fused averaging kernel was not in use"
            w.engine.check()
    dist.barrier()
    if rank == 0:
        print("MG_OK", mode, flush=True)
    comm.destroy_process_group()


if __name__ == "__main__":
    main()
