"""Per-kernel micro-benchmarks: each hand-written sm_100a path of this library against the library
call it replaces (cuBLAS / cuDNN / ATen through PyTorch), on the shapes of the training configs.

    python bench_kernels.py                       # every row, markdown table + one JSON line per row
    python bench_kernels.py --only gemm,adam      # some rows
    python bench_kernels.py --only layernorm --small --iters 3 --warmup 1   # a short run to profile

Timing: CUDA events on the launching stream around ONE call, a 256 MB write between timed calls
(larger than the 126 MB L2, so every call starts cold), `--warmup` untimed calls first, median of
`--iters`. Fractions are against the measured peaks in `MEASURED_PEAKS.json` when that file is
present (copy bandwidth for memory-bound rows, burst cuBLAS bf16 for GEMM-shaped rows).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BF16 = torch.bfloat16
_FLUSH = None
NO_GRAPH = False      # --eager: time plain launches (what a profiler capture wants)


def peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        # kernels are timed one call at a time: the burst cuBLAS figure is the matching denominator
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_ms(fn, iters: int, warmup: int) -> float:
    """Median device time of `fn` in milliseconds, L2 flushed before every timed call. `fn` is captured
    into a CUDA graph when it can be, so the host's launch path (argument checks, tensor-map encoding,
    allocator) is outside the measurement for this library and for the baseline alike; a function
    that cannot be captured is timed eagerly."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    run = fn
    if not NO_GRAPH:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                fn()
            g.replay()
            torch.cuda.synchronize()
            run = g.replay
        except Exception:
            torch.cuda.synchronize()
            run = fn
    out = []
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def flat(*tensors):
    """Re-home parameter tensors into the library's flat buffers (fp32 master + bf16 shadow + gradient slots)."""
    from flodl_b200.parallel.flat import FlatParams
    return FlatParams(list(tensors))


class Row:
    def __init__(self, name, shape, ours_ms, base_ms, work, unit, peak, base_name):
        self.name, self.shape, self.ours_ms, self.base_ms, self.unit, self.base_name = name, shape, ours_ms, base_ms, unit, base_name
        self.ours = work / (ours_ms * 1e-3)
        self.base = work / (base_ms * 1e-3)
        self.frac = self.ours / peak

    def json(self, src):
        return {"kernel": self.name, "shape": self.shape, "ours_ms": round(self.ours_ms, 4), "baseline_ms": round(self.base_ms, 4),
                "baseline": self.base_name, "ours": round(self.ours, 1), "baseline_rate": round(self.base, 1), "unit": self.unit,
                "fraction_of_peak": round(self.frac, 3), "peak_source": src, "speedup": round(self.base_ms / self.ours_ms, 3)}


# ---- rows -------------------------------------------------------------------------------------------
def bench_gemm(args, hbm, tf):
    from flodl_b200 import ops
    shapes = [(4096, 768, 768), (4096, 3072, 768), (4096, 768, 3072), (4096, 30528, 768), (8192, 512, 512), (8192, 2048, 512),
              (8192, 32000, 512)]
    if args.small:
        shapes = [(4096, 3072, 768)]
    rows = []
    for M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=BF16, requires_grad=True)
        w = torch.randn(N, K, device="cuda") * 0.02
        b = torch.zeros(N, device="cuda")
        w.requires_grad_(True)
        b.requires_grad_(True)
        flat(w, b)
        wb, bb = w.detach().to(BF16).requires_grad_(True), b.detach().to(BF16).requires_grad_(True)
        xb = x.detach().clone().requires_grad_(True)
        fl = 2.0 * M * N * K / 1e12
        with torch.no_grad():
            o = time_ms(lambda: ops.linear(x, w, b), args.iters, args.warmup)
            r = time_ms(lambda: F.linear(xb, wb, bb), args.iters, args.warmup)
        rows.append(Row("gemm fwd (+bias)", f"{M}x{N}x{K}", o, r, fl, "TFLOP/s", tf, "cuBLASLt (F.linear)"))
        with torch.no_grad():
            o = time_ms(lambda: ops.linear(x, w, b, "gelu"), args.iters, args.warmup)
            r = time_ms(lambda: F.gelu(F.linear(xb, wb, bb)), args.iters, args.warmup)
        rows.append(Row("gemm fwd + bias + GELU", f"{M}x{N}x{K}", o, r, fl, "TFLOP/s", tf, "cuBLASLt + ATen gelu"))
        dy = torch.randn(M, N, device="cuda", dtype=BF16)

        def ours_fb():
            x.grad = None
            ops.linear(x, w, b).backward(dy)

        def ref_fb():
            xb.grad = wb.grad = bb.grad = None
            F.linear(xb, wb, bb).backward(dy)
        o, r = time_ms(ours_fb, args.iters, args.warmup), time_ms(ref_fb, args.iters, args.warmup)
        rows.append(Row("gemm fwd + dX + dW + db", f"{M}x{N}x{K}", o, r, 3 * fl, "TFLOP/s", tf, "cuBLASLt autograd"))
    return rows


def bench_attention(args, hbm, tf):
    from flodl_b200 import ops
    rows = []
    for (B, H, S, D, causal, name) in [(32, 12, 128, 64, False, "BERT"), (32, 8, 256, 64, True, "LM causal")]:
        qkv = torch.randn(B, S, 3, H, D, device="cuda", dtype=BF16, requires_grad=True)
        mask = torch.zeros(B, 1, 1, S, device="cuda") if not causal else None
        q2 = qkv.detach().clone().requires_grad_(True)
        fl = 4.0 * B * H * S * S * D / 1e12 * (0.5 if causal else 1.0)

        def ref(t):
            qh, kh, vh = (t[:, :, i].permute(0, 2, 1, 3) for i in range(3))
            return F.scaled_dot_product_attention(qh, kh, vh, attn_mask=None if mask is None else mask.to(BF16), is_causal=causal)
        with torch.no_grad():
            o = time_ms(lambda: ops.attention(qkv, mask=mask, causal=causal), args.iters, args.warmup)
            r = time_ms(lambda: ref(q2), args.iters, args.warmup)
        rows.append(Row(f"attention fwd ({name})", f"B{B} H{H} S{S} D{D}", o, r, fl, "TFLOP/s", tf, "ATen SDPA"))
        do = torch.randn(B, S, H, D, device="cuda", dtype=BF16)

        def ours_fb():
            qkv.grad = None
            ops.attention(qkv, mask=mask, causal=causal).backward(do)

        def ref_fb():
            q2.grad = None
            ref(q2).backward(do.permute(0, 2, 1, 3))
        o, r = time_ms(ours_fb, args.iters, args.warmup), time_ms(ref_fb, args.iters, args.warmup)
        rows.append(Row(f"attention fwd+bwd ({name})", f"B{B} H{H} S{S} D{D}", o, r, 3.5 * fl, "TFLOP/s", tf, "ATen SDPA autograd"))
    return rows


def bench_layernorm(args, hbm, tf):
    from flodl_b200 import ops
    rows = []
    shapes = [(4096, 768, 1e-12), (8192, 512, 1e-5)] if not args.small else [(65536, 768, 1e-12)]
    for R, C, eps in shapes:
        reps = 1 if args.small else 16          # stack rows so the tensors exceed L2
        x = torch.randn(R * reps, C, device="cuda", dtype=BF16, requires_grad=True)
        res = torch.randn(R * reps, C, device="cuda", dtype=BF16)
        g, b = torch.ones(C, device="cuda", requires_grad=True), torch.zeros(C, device="cuda", requires_grad=True)
        flat(g, b)
        gb, bb = g.detach().to(BF16).requires_grad_(True), b.detach().to(BF16).requires_grad_(True)
        x2 = x.detach().clone().requires_grad_(True)
        nbytes = x.numel() * 2
        with torch.no_grad():
            o = time_ms(lambda: ops.layer_norm(x, g, b, eps), args.iters, args.warmup)
            r = time_ms(lambda: F.layer_norm(x2, (C,), gb, bb, eps), args.iters, args.warmup)
        rows.append(Row("layernorm fwd", f"{R * reps}x{C}", o, r, 2 * nbytes / 1e9, "GB/s", hbm, "ATen native_layer_norm"))
        with torch.no_grad():
            o = time_ms(lambda: ops.layer_norm(x, g, b, eps, residual=res), args.iters, args.warmup)
            r = time_ms(lambda: F.layer_norm(x2 + res, (C,), gb, bb, eps), args.iters, args.warmup)
        rows.append(Row("layernorm(x + residual) fwd", f"{R * reps}x{C}", o, r, 3 * nbytes / 1e9, "GB/s", hbm, "ATen add + layer_norm"))
        dy = torch.randn_like(x)

        def ours_fb():
            x.grad = None
            ops.layer_norm(x, g, b, eps).backward(dy)

        def ref_fb():
            x2.grad = gb.grad = bb.grad = None
            F.layer_norm(x2, (C,), gb, bb, eps).backward(dy)
        o, r = time_ms(ours_fb, args.iters, args.warmup), time_ms(ref_fb, args.iters, args.warmup)
        rows.append(Row("layernorm fwd+bwd", f"{R * reps}x{C}", o, r, 5 * nbytes / 1e9, "GB/s", hbm, "ATen autograd"))
    return rows


def bench_gelu(args, hbm, tf):
    from flodl_b200 import ops
    rows = []
    R, C = (4096 * 8, 3072) if not args.small else (4096 * 4, 3072)
    x = torch.randn(R, C, device="cuda", dtype=BF16)
    for approx in ("none", "tanh"):
        with torch.no_grad():
            o = time_ms(lambda: ops.gelu(x, approx), args.iters, args.warmup)
            r = time_ms(lambda: F.gelu(x, approximate=approx), args.iters, args.warmup)
        rows.append(Row(f"gelu ({'erf' if approx == 'none' else 'tanh'})", f"{R}x{C}", o, r, 2 * x.numel() * 2 / 1e9, "GB/s", hbm, "ATen gelu"))
    return rows


def bench_cross_entropy(args, hbm, tf):
    from flodl_b200 import ops
    rows = []
    shapes = [(4096, 30522, 0.15), (8192, 32000, 1.0), (128, 10, 1.0)] if not args.small else [(4096, 30522, 0.15)]
    for R, V, active in shapes:
        logits = torch.randn(R, V, device="cuda", dtype=BF16, requires_grad=True)
        tgt = torch.randint(0, V, (R,), device="cuda")
        if active < 1.0:
            tgt[torch.rand(R, device="cuda") > active] = -100
        l2 = logits.detach().clone().requires_grad_(True)

        def ours():
            logits.grad = None
            ops.cross_entropy(logits, tgt).backward()

        def ref():
            l2.grad = None
            F.cross_entropy(l2.float(), tgt, ignore_index=-100).backward()
        o, r = time_ms(ours, args.iters, args.warmup), time_ms(ref, args.iters, args.warmup)
        rows.append(Row("softmax cross-entropy fwd+bwd", f"{R}x{V} ({int(active * 100)}% rows active)", o, r, 2 * R * V * 2 / 1e9, "GB/s", hbm,
                        "ATen cross_entropy (fp32 upcast) autograd"))
    return rows


def _param_lists(sizes):
    mine = [torch.randn(n, device="cuda").requires_grad_(True) for n in sizes]
    ref = [p.detach().clone().requires_grad_(True) for p in mine]
    return mine, ref


def bench_adam(args, hbm, tf):
    from flodl_b200 import nn
    rows = []
    for name, total in ([("BERT-base", 110_000_000), ("decoder LM", 52_000_000)] if not args.small else [("small", 32_000_000)]):
        sizes = [total // 200] * 200
        mine, ref = _param_lists(sizes)
        f = flat(*mine)
        opt = nn.AdamW(mine, 1e-4, 0.01)
        ropt = torch.optim.AdamW(ref, 1e-4, weight_decay=0.01, fused=True)
        f.grads.normal_()
        for p in ref:
            p.grad = torch.randn_like(p)
        o, r = time_ms(opt.step, args.iters, args.warmup), time_ms(ropt.step, args.iters, args.warmup)
        n = f.total
        # read p, g, m, v; write p, m, v, bf16 shadow
        rows.append(Row(f"AdamW step ({name}, flat buffer + bf16 shadow)", f"{n / 1e6:.0f} M params", o, r, (7 * 4 + 2) * n / 1e9, "GB/s", hbm,
                        "torch _fused_adamw_ (no bf16 copy)"))
    return rows


def bench_sgd(args, hbm, tf):
    from flodl_b200 import nn
    sizes = [432] + [16, 16] * 7 + [2304] * 6 + [4608, 32, 32] + [9216] * 5 + [32, 32] * 5 + [18432, 64, 64] + [36864] * 5 + [64, 64] * 5 + [640, 10]
    mine, ref = _param_lists(sizes)
    f = flat(*mine)
    opt = nn.SGD(mine, 0.1, 0.9, 1e-4)
    ropt = torch.optim.SGD(ref, 0.1, momentum=0.9, weight_decay=1e-4, foreach=False)
    fopt = torch.optim.SGD([p.detach().clone().requires_grad_(True) for p in ref], 0.1, momentum=0.9, weight_decay=1e-4, foreach=True)
    f.grads.normal_()
    for p in ref:
        p.grad = torch.randn_like(p)
    for g in fopt.param_groups:
        for p in g["params"]:
            p.grad = torch.randn_like(p)
    o, r = time_ms(opt.step, args.iters, args.warmup), time_ms(ropt.step, args.iters, args.warmup)
    r2 = time_ms(fopt.step, args.iters, args.warmup)
    n = sum(sizes)
    return [Row("SGD-momentum step (ResNet-20 parameter list)", f"{len(sizes)} tensors, {n / 1e6:.2f} M params", o, r, 1e-6, "steps/us", 1.0,
                "per-parameter loop (torch SGD foreach=False)"),
            Row("SGD-momentum step (ResNet-20 parameter list)", f"{len(sizes)} tensors, {n / 1e6:.2f} M params", o, r2, 1e-6, "steps/us", 1.0,
                "torch SGD foreach=True")]


def bench_batchnorm(args, hbm, tf):
    from flodl_b200 import ops
    rows = []
    shapes = [(128, 16, 32, False), (128, 32, 16, False), (128, 64, 8, False), (128, 16, 32, True), (128, 32, 16, True), (128, 64, 8, True)]
    if args.small:
        shapes = [(1024, 64, 32, False), (1024, 64, 32, True)]
    for N, C, HW, channels_last in shapes:
        reps = 1 if args.small else 32
        fmt = torch.channels_last if channels_last else torch.contiguous_format
        x = torch.randn(N * reps, C, HW, HW, device="cuda", dtype=BF16).contiguous(memory_format=fmt).requires_grad_(True)
        res = torch.randn_like(x)
        g, b = torch.ones(C, device="cuda", requires_grad=True), torch.zeros(C, device="cuda", requires_grad=True)
        rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
        x2 = x.detach().clone().requires_grad_(True)
        gb, bb = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
        dy = torch.randn_like(x)
        nbytes = x.numel() * 2

        def ours():
            x.grad = None
            ops.batch_norm(x, rm, rv, g, b, True, 0.1, 1e-5, relu=True, residual=res).backward(dy)

        def ref():
            x2.grad = gb.grad = bb.grad = None
            torch.relu(F.batch_norm(x2, rm, rv, gb, bb, True, 0.1, 1e-5) + res).backward(dy)
        o, r = time_ms(ours, args.iters, args.warmup), time_ms(ref, args.iters, args.warmup)
        # fwd: read x twice + residual, write y; bwd: read dy, x, y twice, write dx, dres
        rows.append(Row("batchnorm + add + relu fwd+bwd", f"[{N * reps},{C},{HW},{HW}]" + (" channels-last" if channels_last else ""), o, r, 12 * nbytes / 1e9, "GB/s", hbm,
                        "cuDNN batch_norm + ATen add + relu autograd"))
    return rows


def bench_gradnorm(args, hbm, tf):
    from flodl_b200 import _ext
    C = _ext.require()
    n = 110_000_000 if not args.small else 32_000_000
    sizes = [n // 200] * 200
    grads = torch.randn(sum(sizes), device="cuda")
    plist = [torch.zeros(s, device="cuda", requires_grad=True) for s in sizes]
    off = 0
    for p in plist:
        p.grad = grads[off:off + p.numel()].clone()
        off += p.numel()
    o = time_ms(lambda: C.grad_norm(grads, 1.0, 1.0), args.iters, args.warmup)
    r = time_ms(lambda: torch.nn.utils.clip_grad_norm_(plist, 1.0, foreach=True), args.iters, args.warmup)
    return [Row("global grad norm + clip coefficient", f"{grads.numel() / 1e6:.0f} M grads", o, r, grads.numel() * 4 / 1e9, "GB/s", hbm,
                "torch clip_grad_norm_ (foreach norm + mul)")]


def bench_conv(args, hbm, tf):
    """The three passes of the CIFAR-ResNet convolutions on channels-last bf16 tensors, native tcgen05
    kernels against cuDNN (through ATen) on the same tensors."""
    C = _ext_module()
    rows = []
    shapes = [(128, 16, 16, 32, 3, 1), (128, 16, 32, 32, 3, 2), (128, 32, 32, 16, 3, 1), (128, 32, 64, 16, 3, 2),
              (128, 64, 64, 8, 3, 1), (128, 16, 32, 32, 1, 2)]
    if args.small:
        shapes = [(128, 16, 16, 32, 3, 1)]
    cl = torch.channels_last
    for N, Ci, Co, HW, k, s in shapes:
        pad = k // 2
        x = torch.randn(N, Ci, HW, HW, device="cuda", dtype=BF16).contiguous(memory_format=cl)
        w = (torch.randn(Co, Ci, k, k, device="cuda") * 0.1).to(BF16).contiguous(memory_format=cl)
        Ho = (HW + 2 * pad - k) // s + 1
        fl = 2.0 * N * Co * Ho * Ho * Ci * k * k / 1e12
        dy = torch.randn(N, Co, Ho, Ho, device="cuda", dtype=BF16).contiguous(memory_format=cl)
        dw = torch.zeros(Co, Ci, k, k, device="cuda").contiguous(memory_format=cl)
        sums = torch.zeros(2, Co, device="cuda")
        shape = f"N{N} {Ci}->{Co} @{HW}^2 k{k} s{s}"

        def bwd(mask):
            return lambda: torch.ops.aten.convolution_backward(dy, x, w, None, [s, s], [pad, pad], [1, 1], False, [0, 0], 1, mask)
        o = time_ms(lambda: C.conv_fprop(x, w, s, pad, sums), args.iters, args.warmup)
        r = time_ms(lambda: F.conv2d(x, w, None, s, pad), args.iters, args.warmup)
        rows.append(Row("conv fprop (+BN sums)", shape, o, r, fl, "TFLOP/s", tf, "cuDNN fprop"))
        if C.conv_dgrad_supported(N, HW, HW, Ci, Co, k, s, pad):
            o = time_ms(lambda: C.conv_dgrad(dy, w, s, pad), args.iters, args.warmup)
            r = time_ms(bwd([True, False, False]), args.iters, args.warmup)
            rows.append(Row("conv dgrad", shape, o, r, fl, "TFLOP/s", tf, "cuDNN dgrad"))
        o = time_ms(lambda: C.conv_wgrad(x, dy, dw, s, pad), args.iters, args.warmup)
        r = time_ms(bwd([False, True, False]), args.iters, args.warmup)
        rows.append(Row("conv wgrad (fp32 accumulate in place)", shape, o, r, fl, "TFLOP/s", tf, "cuDNN wgrad"))
    return rows


def _ext_module():
    from flodl_b200 import _ext
    return _ext.require()


BENCHES = {"gemm": bench_gemm, "attention": bench_attention, "layernorm": bench_layernorm, "gelu": bench_gelu,
           "cross_entropy": bench_cross_entropy, "adam": bench_adam, "sgd": bench_sgd, "batchnorm": bench_batchnorm,
           "gradnorm": bench_gradnorm, "conv": bench_conv}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="comma-separated subset of: " + ", ".join(BENCHES))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--small", action="store_true", help="one modest shape per row (for profiler captures)")
    ap.add_argument("--out", default="", help="also write the markdown table here")
    ap.add_argument("--eager", action="store_true", help="time plain launches instead of CUDA-graph replays")
    args = ap.parse_args()
    global NO_GRAPH
    NO_GRAPH = args.eager or args.small
    from flodl_b200 import _ext, nn
    _ext.require()
    torch.manual_seed(0)
    hbm, tf, src = peaks()
    names = [n for n in args.only.split(",") if n] or list(BENCHES)
    guard = nn.AutocastGuard(BF16)
    lines = [f"| kernel | shape | ours ms | baseline ms | ours | baseline | speed-up | of {src} peak |", "|---|---|---|---|---|---|---|---|"]
    for n in names:
        for row in BENCHES[n](args, hbm, tf):
            print(json.dumps(row.json(src)), flush=True)
            peak = f"{row.frac:.2f}" if row.unit != "steps/us" else "-"
            lines.append(f"| {row.name} | {row.shape} | {row.ours_ms:.4f} | {row.base_ms:.4f} ({row.base_name}) | {row.ours:.1f} {row.unit} | "
                         f"{row.base:.1f} {row.unit} | {row.base_ms / row.ours_ms:.2f}x | {peak} |")
    guard.release()
    table = "\n".join(lines)
    print(table)
    if args.out:
        with open(args.out, "w") as f:
            f.write(f"peaks ({src}): HBM copy {hbm:.0f} GB/s, bf16 GEMM burst {tf:.0f} TFLOP/s\n\n" + table + "\n")


if __name__ == "__main__":
    main()
