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
        lone = comm.SymmetricBuffer(4096, timeout_s=0.3)
        torch.cuda.synchronize(); dist.barrier()
        if rank == 0:
            lone.barrier()
            torch.cuda.synchronize()
            assert lone.status() == 4, lone.status()
            z = torch.ones(4, device=dev).sum().item()      # the context is still usable
            assert z == 4.0
        dist.barrier()
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
            for step in range(4):
                eng.step(lambda: head.compute_loss([ids, pos, tt, mask], labels))
                torch.cuda.synchronize()
                eng.check()
                gs = gather_all(eng.flat.grads.clone())
                assert all(torch.equal(gs[0], a) for a in gs), f"gradients differ across ranks at step {step}"
                ps = gather_all(eng.flat.params.clone())
                assert all(torch.equal(ps[0], a) for a in ps), f"parameters diverged at step {step}"
            assert len(eng.sync.buckets) > 1 and eng.sync.launch_count >= 4 * len(eng.sync.buckets)
    dist.barrier()
    if rank == 0:
        print("MG_OK", mode, flush=True)
    comm.destroy_process_group()


if __name__ == "__main__":
    main()
