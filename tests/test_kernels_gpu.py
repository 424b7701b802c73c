"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from flodl_b200 import _ext
    return _ext.require()


def _ref_gemm(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _gemm_case(C, M, N, K, a_mn, b_mn, config, out_dtype=torch.bfloat16, **kw):
    torch.manual_seed(M * 7 + N * 3 + K)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    out = torch.zeros(M, N, device=dev, dtype=out_dtype)
    C.clear_status(0)
    C.gemm(a, b, out, a_mn, b_mn, config=config, **kw)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0, f"kernel status {C.read_status(0)}"
    ref = _ref_gemm(a, b, a_mn, b_mn)
    return out.float(), ref


@pytest.mark.parametrize("config", [2, 1, 3, 0, 4])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_layouts(C, config, a_mn, b_mn):
    out, ref = _gemm_case(C, 512, 768, 256, a_mn, b_mn, config)
    err = (out - ref).abs().max().item()
    assert err <= 0.02 * ref.abs().max().item() + 0.05, f"max err {err}"


@pytest.mark.parametrize("config", [0, 1, 2, 3, 4, 5])
def test_gemm_ragged_edges(C, config):
    # M, N not multiples of the tile, K not a multiple of 64 (TMA zero-fills the tails)
    out, ref = _gemm_case(C, 300, 328, 200, False, False, config)
    err = (out - ref).abs().max().item()
    assert err <= 0.02 * ref.abs().max().item() + 0.05, f"max err {err}"


@pytest.mark.parametrize("config", [0, 2, 4, 5])
def test_gemm_many_tiles_per_cta(C, config):
    # more tiles than SMs: exercises the accumulator double buffering and barrier phases
    out, ref = _gemm_case(C, 4096, 3072, 768, False, False, config)
    err = (out - ref).abs().max().item()
    assert err <= 0.02 * ref.abs().max().item() + 0.05, f"max err {err}"


@pytest.mark.parametrize("config", [-1, 0, 1, 4, 5])
def test_gemm_bias_gelu_aux(C, config):
    M, N, K = 512, 768, 256
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device="cuda")
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    aux = torch.empty_like(out)
    C.gemm(a, b, out, bias=bias, epi=1, aux=aux, config=config)
    pre = a.float() @ b.float().t() + bias
    ref = torch.nn.functional.gelu(pre)
    assert (aux.float() - pre).abs().max().item() < 0.05
    assert (out.float() - ref).abs().max().item() < 0.05
    # backward epilogue: dY * gelu'(aux)
    g = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") / math.sqrt(K)).bfloat16()
    dpre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(g, w, dpre, epi=2, aux=aux, config=config)
    x = aux.float().requires_grad_(True)
    torch.nn.functional.gelu(x).backward(g.float() @ w.float().t())
    assert (dpre.float() - x.grad).abs().max().item() < 0.06


def test_gemm_fp32_out_accumulate_splitk_alpha(C):
    M, N, K = 256, 384, 1024
    torch.manual_seed(1)
    a = torch.randn(K, M, device="cuda").bfloat16()   # MN-major A: dW = dY^T X
    b = torch.randn(K, N, device="cuda").bfloat16()
    ref = a.float().t() @ b.float()
    base = torch.randn(M, N, device="cuda")
    out = base.clone()
    C.gemm(a, b, out, True, True, accumulate=True)
    assert (out - (base + ref)).abs().max().item() < 0.02 * ref.abs().max().item()
    out2 = base.clone()
    C.gemm(a, b, out2, True, True, accumulate=True, split_k=4)
    assert (out2 - (base + ref)).abs().max().item() < 0.02 * ref.abs().max().item()
    out4 = base.clone()
    C.gemm(a, b, out4, True, True, accumulate=True, split_k=2, config=4)     # 128x192 tiles, 128+64 epilogue split
    assert (out4 - (base + ref)).abs().max().item() < 0.02 * ref.abs().max().item()
    alpha = torch.tensor([0.25], device="cuda")
    out3 = torch.empty(M, N, device="cuda")
    C.gemm(a, b, out3, True, True, alpha=alpha)
    assert (out3 - 0.25 * ref).abs().max().item() < 0.02 * ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cols", [768, 512, 16 * 8, 1024])
def test_layernorm_fwd_bwd(C, dtype, cols):
    rows = 1000
    torch.manual_seed(2)
    x = torch.randn(rows, cols, device="cuda").to(dtype)
    r = torch.randn(rows, cols, device="cuda").to(dtype)
    g = torch.randn(cols, device="cuda")
    b = torch.randn(cols, device="cuda")
    y, pre, mean, rstd = C.layernorm_fwd(x, r, g, b, 1e-5, 0.0, 0, True)
    pre_ref = (x.float() + r.float()).to(dtype).float()
    ref = torch.nn.functional.layer_norm(pre_ref, (cols,), g, b, 1e-5)
    tol = 0.02 * ref.abs().max().item() if dtype == torch.bfloat16 else 1e-4
    assert (y.float() - ref).abs().max().item() < tol
    assert (pre.float() - pre_ref).abs().max().item() < 1e-6
    dy = torch.randn(rows, cols, device="cuda").to(dtype)
    dpre, _, dg, db = C.layernorm_bwd(dy, pre, mean, rstd, g, 0.0, 0, False, True, None, None)
    xr = pre_ref.clone().requires_grad_(True)
    gr = g.clone().requires_grad_(True)
    br = b.clone().requires_grad_(True)
    torch.nn.functional.layer_norm(xr, (cols,), gr, br, 1e-5).backward(dy.float())
    assert (dpre.float() - xr.grad).abs().max().item() < (0.02 * xr.grad.abs().max().item() + 0.02 if dtype == torch.bfloat16 else 1e-3)
    assert (dg - gr.grad).abs().max().item() < 5e-2 * max(1.0, gr.grad.abs().max().item()) * (1 if dtype == torch.bfloat16 else 0.01)
    assert (db - br.grad).abs().max().item() < 1e-2 * max(1.0, br.grad.abs().max().item())


def test_layernorm_dropout_mask_consistent(C):
    rows, cols, p = 512, 768, 0.1
    x = torch.ones(rows, cols, device="cuda", dtype=torch.bfloat16)
    r = torch.zeros_like(x)
    _, pre, mean, rstd = C.layernorm_fwd(x, r, None, None, 1e-5, p, 1234, True)
    keep = (pre.float() != 0)
    frac = keep.float().mean().item()
    assert abs(frac - (1 - p)) < 0.01
    assert torch.allclose(pre.float()[keep], torch.full_like(pre.float()[keep], 1 / (1 - p)), atol=1e-2)
    # the standalone dropout kernel and the LN backward regenerate the same mask
    d = C.dropout(x, p, 1234)
    assert torch.equal(d.float() != 0, keep)
    dy = torch.ones_like(x)
    dpre, dxd, _, _ = C.layernorm_bwd(dy, pre, mean, rstd, None, p, 1234, True, False, None, None)
    assert ((dxd.float() != 0) & ~keep).sum().item() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tanh", [False, True])
def test_gelu(C, dtype, tanh):
    x = torch.randn(4099 * 3, device="cuda").to(dtype)
    y = C.gelu_fwd(x, tanh)
    xr = x.float().requires_grad_(True)
    ref = torch.nn.functional.gelu(xr, approximate="tanh" if tanh else "none")
    tol = 0.02 if dtype == torch.bfloat16 else 1e-5
    assert (y.float() - ref).abs().max().item() < tol
    dy = torch.randn_like(x)
    dx = C.gelu_bwd(dy, x, tanh)
    ref.backward(dy.float())
    assert (dx.float() - xr.grad).abs().max().item() < (0.03 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,V,pad", [(256, 30522, 6), (128, 10, 0), (64, 32000, 0)])
def test_softmax_ce(C, dtype, rows, V, pad):
    torch.manual_seed(3)
    buf = torch.randn(rows, V + pad, device="cuda").to(dtype) * 3
    logits = buf[:, :V]
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[::3] = -100
    lr = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, tgt, ignore_index=-100)
    ref.backward()
    loss, dl, cinv = C.softmax_ce(logits, tgt, -100, True, False)
    assert abs(loss.item() - ref.item()) < (2e-2 if dtype == torch.bfloat16 else 1e-4)
    assert (dl.float() - lr.grad).abs().max().item() < (2e-3 if dtype == torch.bfloat16 else 1e-6)
    assert cinv[0].item() == (tgt != -100).sum().item()


def test_adam_matches_reference(C):
    n = 100003
    torch.manual_seed(4)
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr = p.clone()
    mr, vr = m.clone(), v.clone()
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.01
    for t in range(1, 4):
        hyper = torch.tensor([lr, 1 - b1 ** t, 1 - b2 ** t, wd], device="cuda")
        C.adam_step(p, g, m, v, p16, hyper, b1, b2, eps)
        pr *= 1 - lr * wd
        mr = b1 * mr + (1 - b1) * g
        vr = b2 * vr + (1 - b2) * g * g
        pr -= (lr / (1 - b1 ** t)) * mr / ((vr / (1 - b2 ** t)).sqrt() + eps)
    assert (p - pr).abs().max().item() < 1e-5
    assert (p16.float() - pr).abs().max().item() < 2e-2
    # bf16 gradients + device-side gradient scale
    gs = torch.tensor([0.5], device="cuda")
    p2, m2, v2 = pr.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    hyper = torch.tensor([lr, 1 - b1, 1 - b2, 0.0], device="cuda")
    C.adam_step(p2, g.bfloat16(), m2, v2, None, hyper, b1, b2, eps, gs)
    gq = g.bfloat16().float() * 0.5
    ref = pr - (lr / (1 - b1)) * ((1 - b1) * gq) / ((((1 - b2) * gq * gq) / (1 - b2)).sqrt() + eps)
    assert (p2 - ref).abs().max().item() < 1e-5


def test_sgd_matches_reference(C):
    n = 5001
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    buf = torch.zeros(n, device="cuda")
    pr, br = p.clone(), None
    lr, mu, wd = 0.1, 0.9, 1e-4
    for step in range(3):
        hyper = torch.tensor([lr, mu, wd, 1.0 if step == 0 else 0.0], device="cuda")
        C.sgd_step(p, g, buf, None, hyper)
        gg = g + wd * pr
        br = gg.clone() if br is None else mu * br + gg
        pr = pr - lr * br
    assert (p - pr).abs().max().item() < 1e-5


def test_grad_norm_and_clip(C):
    g = torch.randn(1_000_003, device="cuda")
    out = C.grad_norm(g, 1.0, 1.0)
    ref = g.double().norm().item()
    assert abs(out[0].item() - ref) / ref < 1e-5
    assert abs(out[1].item() - 1.0 / (ref + 1e-6)) < 1e-6
    out = C.grad_norm(g.bfloat16(), 0.0, 1.0)
    assert abs(out[0].item() - g.bfloat16().double().norm().item()) / ref < 1e-4
    assert out[1].item() == 1.0


def test_colsum_and_cast(C):
    x = torch.randn(4096, 770, device="cuda").bfloat16()
    out = torch.zeros(770, device="cuda")
    C.colsum(x, out)
    assert (out - x.float().sum(0)).abs().max().item() < 1e-2
    y = torch.empty(4096 * 770, device="cuda")
    C.cast_into(x.view(-1), y, 2.0)
    assert torch.equal(y, x.view(-1).float() * 2)


def _attn_ref(q, k, v, mask, scale, causal):
    # q, k, v: [B, S, H, D] fp32
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    s = (qh @ kh.transpose(-1, -2)) * scale
    if mask is not None:
        s = s + mask[:, None, None, :]
    if causal:
        S = q.shape[1]
        s = s.masked_fill(torch.ones(S, S, device=q.device).triu(1).bool(), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vh).permute(0, 2, 1, 3)


@pytest.mark.parametrize("B,H,S,causal,use_mask", [(2, 3, 128, False, True), (2, 2, 256, True, False), (1, 2, 256, False, True), (2, 2, 384, True, False), (1, 1, 200, False, False),
                                                        # one key block: the kernels that share an SM between four / two CTAs
                                                        (4, 12, 128, True, False), (3, 2, 77, False, True), (2, 4, 64, True, False), (32, 12, 128, False, True)])
def test_attention_fwd_bwd(C, B, H, S, causal, use_mask):
    torch.manual_seed(5)
    D = 64
    qkv = torch.randn(B, S, 3, H, D, device="cuda").bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    mask = None
    if use_mask:
        mask = torch.zeros(B, S, device="cuda")
        mask[:, S - 17:] = -1e4
    scale = 1.0 / math.sqrt(D)
    C.clear_status(0)
    o, lse = C.attn_fwd(q, k, v, mask, scale, causal)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref = _attn_ref(qf, kf, vf, mask, scale, causal)
    assert (o.float() - ref).abs().max().item() < 0.03, (o.float() - ref).abs().max().item()
    do = torch.randn(B, S, H, D, device="cuda").bfloat16()
    dqkv = C.attn_bwd(q, k, v, o, do, lse, mask, scale, causal)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0
    ref.backward(do.float())
    for i, g in enumerate((qf.grad, kf.grad, vf.grad)):
        err = (dqkv[:, :, i].float() - g).abs().max().item()
        assert err < 0.06 * max(1.0, g.abs().max().item()), (i, err, g.abs().max().item())


def test_attention_dropout_statistics(C):
    torch.manual_seed(6)
    B, H, S, D = 2, 2, 128, 64
    qkv = torch.zeros(B, S, 3, H, D, device="cuda").bfloat16()
    qkv[:, :, 2] = 1.0   # V = 1 -> each output = sum of kept probabilities / (1 - p)
    o, _ = C.attn_fwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], None, 0.125, False, 0.25, 77)
    m = o.float().mean().item()
    assert abs(m - 1.0) < 0.02
    assert o.float().std().item() > 0.01


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("relu,use_res", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("channels_last", [False, True])
def test_batchnorm_fused(C, dtype, relu, use_res, channels_last):
    torch.manual_seed(8)
    N, Ch, H = 16, 32, 8
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    x = torch.randn(N, Ch, H, H, device="cuda").to(dtype).contiguous(memory_format=fmt)
    res = torch.randn(N, Ch, H, H, device="cuda").to(dtype).contiguous(memory_format=fmt) if use_res else None
    g = torch.rand(Ch, device="cuda") + 0.5
    b = torch.randn(Ch, device="cuda")
    rm, rv = torch.zeros(Ch, device="cuda"), torch.ones(Ch, device="cuda")
    rm_ref, rv_ref = rm.clone(), rv.clone()
    y, mean, rstd = C.bn_fwd(x, res, g, b, rm, rv, 1e-5, 0.1, relu, True)
    xr = x.float().clone().requires_grad_(True)
    gr, br = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    rr = res.float().clone().requires_grad_(True) if use_res else None
    ref = torch.nn.functional.batch_norm(xr, rm_ref, rv_ref, gr, br, True, 0.1, 1e-5)
    if use_res:
        ref = ref + rr
    if relu:
        ref = torch.relu(ref)
    tol = 0.05 if dtype == torch.bfloat16 else 1e-4
    assert (y.float() - ref).abs().max().item() < tol
    assert (rm - rm_ref).abs().max().item() < 1e-4 and (rv - rv_ref).abs().max().item() < 1e-3
    assert y.is_contiguous(memory_format=fmt)
    dy = torch.randn_like(ref).to(dtype).contiguous(memory_format=fmt)
    dx, dres, dg, db = C.bn_bwd(dy, x, y, g, mean, rstd, relu, use_res, None, None)
    # reference backward with the kernel's own ReLU mask (ties at 0 in bf16 would otherwise differ)
    (ref * (y.float() > 0 if relu else 1)).backward(dy.float()) if False else ref.backward(dy.float())
    btol = 0.08 if dtype == torch.bfloat16 else 2e-3
    assert (dx.float() - xr.grad).abs().max().item() < btol
    assert (dg - gr.grad).abs().max().item() < btol * 10 and (db - br.grad).abs().max().item() < btol * 10
    if use_res:
        assert (dres.float() - rr.grad).abs().max().item() < btol


def test_batchnorm_channels_last_many_blocks_accumulates(C):
    # enough pixels for several hundred blocks: exercises the last-block fold, the counter reset
    # (two calls in a row) and accumulation into existing gradient slots
    torch.manual_seed(9)
    x = torch.randn(64, 16, 32, 32, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    g, b = torch.rand(16, device="cuda") + 0.5, torch.randn(16, device="cuda")
    rm, rv = torch.zeros(16, device="cuda"), torch.ones(16, device="cuda")
    for _ in range(2):
        y, mean, rstd = C.bn_fwd(x, None, g, b, rm, rv, 1e-5, 0.1, False, True)
    ref = torch.nn.functional.batch_norm(x.float(), None, None, g, b, True, 0.1, 1e-5)
    assert (y.float() - ref).abs().max().item() < 0.05
    assert (mean - x.float().mean(dim=(0, 2, 3))).abs().max().item() < 1e-3
    dy = torch.randn_like(x)
    dg_acc, db_acc = torch.ones(16, device="cuda"), torch.ones(16, device="cuda")
    dx, _, _, _ = C.bn_bwd(dy, x, y, g, mean, rstd, False, False, dg_acc, db_acc)
    xr = x.float().clone().requires_grad_(True)
    gr, br = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    torch.nn.functional.batch_norm(xr, None, None, gr, br, True, 0.1, 1e-5).backward(dy.float())
    assert (dx.float() - xr.grad).abs().max().item() < 0.08
    assert (dg_acc - 1 - gr.grad).abs().max().item() < 0.02 * gr.grad.abs().max().item() + 0.5
    assert (db_acc - 1 - br.grad).abs().max().item() < 0.02 * br.grad.abs().max().item() + 0.5


@pytest.mark.parametrize("N,Ci,Co,HW,k,stride", [(8, 16, 16, 32, 3, 1), (4, 16, 32, 32, 3, 2), (4, 32, 32, 16, 3, 1), (4, 32, 64, 16, 3, 2),
                                                 (6, 64, 64, 8, 3, 1), (4, 16, 32, 32, 1, 2), (2, 32, 8, 16, 3, 1), (150, 16, 16, 32, 3, 1), (2, 64, 16, 64, 3, 1), (3, 16, 32, 28, 3, 1), (2, 32, 64, 7, 3, 1), (300, 32, 32, 16, 3, 1)])
def test_conv_wgrad_tensor_core(C, N, Ci, Co, HW, k, stride):
    torch.manual_seed(11)
    pad = k // 2
    assert C.conv_wgrad_supported(N, HW, HW, Ci, Co, k, stride, pad)
    x = torch.randn(N, Ci, HW, HW, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    Ho = (HW + 2 * pad - k) // stride + 1
    dy = (torch.randn(N, Co, Ho, Ho, device="cuda") * 0.1).bfloat16().contiguous(memory_format=torch.channels_last)
    base = torch.randn(Co, Ci, k, k, device="cuda").contiguous(memory_format=torch.channels_last)
    dw = base.clone()
    assert dw.is_contiguous(memory_format=torch.channels_last)
    C.conv_wgrad(x, dy, dw, stride, pad)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0
    ref = torch.nn.grad.conv2d_weight(x.float(), (Co, Ci, k, k), dy.float(), stride=stride, padding=pad)
    err = (dw - base - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 0.02, f"max err {err} (ref max {ref.abs().max().item()})"
    # a second call accumulates again
    C.conv_wgrad(x, dy, dw, stride, pad)
    assert (dw - base - 2 * ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.04


def test_conv_wgrad_rejects_unsupported(C):
    assert not C.conv_wgrad_supported(4, 32, 32, 3, 16, 3, 1, 1)       # 3 input channels: rows are not 16-byte multiples
    assert not C.conv_wgrad_supported(4, 32, 32, 16, 16, 5, 1, 2)      # 5x5
    assert not C.conv_wgrad_supported(4, 28, 28, 16, 16, 3, 2, 1)      # strided, width not a power of two


@pytest.mark.parametrize("N,Ci,Co,HW,k,stride", [(8, 16, 16, 32, 3, 1), (4, 16, 32, 32, 3, 2), (4, 32, 32, 16, 3, 1), (4, 32, 64, 16, 3, 2),
                                                 (5, 64, 64, 8, 3, 1), (4, 16, 32, 32, 1, 2), (2, 32, 16, 16, 3, 1), (160, 16, 16, 32, 3, 1),
                                                 (2, 64, 48, 64, 3, 1), (3, 16, 32, 28, 3, 1), (2, 32, 32, 7, 3, 1), (12, 64, 64, 64, 3, 1)])
def test_conv_fprop_tensor_core(C, N, Ci, Co, HW, k, stride):
    torch.manual_seed(12)
    pad = k // 2
    assert C.conv_fprop_supported(N, HW, HW, Ci, Co, k, stride, pad)
    x = torch.randn(N, Ci, HW, HW, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(Co, Ci, k, k, device="cuda") * 0.1).bfloat16().contiguous(memory_format=torch.channels_last)
    stats = torch.zeros(2, Co, device="cuda")
    y = C.conv_fprop(x, w, stride, pad, stats)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0
    ref = F.conv2d(x.float(), w.float(), None, stride, pad)
    assert y.shape == ref.shape and y.is_contiguous(memory_format=torch.channels_last)
    err = (y.float() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 0.01, f"max err {err} (ref max {ref.abs().max().item()})"
    # the fused statistics are those of the rounded output
    yf = y.float()
    s1, s2 = yf.sum((0, 2, 3)), (yf * yf).sum((0, 2, 3))
    assert (stats[0] - s1).abs().max().item() <= 1e-3 * s1.abs().max().item() + 0.05
    assert (stats[1] - s2).abs().max().item() <= 1e-3 * s2.abs().max().item() + 0.05
    # without statistics
    y2 = C.conv_fprop(x, w, stride, pad)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("N,Ci,Co,HW,k", [(8, 16, 16, 32, 3), (4, 32, 32, 16, 3), (5, 64, 64, 8, 3), (4, 16, 32, 32, 1), (2, 32, 16, 16, 3),
                                          (2, 16, 64, 64, 3), (3, 32, 16, 28, 3), (2, 64, 32, 7, 3), (12, 64, 64, 64, 3)])
def test_conv_dgrad_tensor_core(C, N, Ci, Co, HW, k):
    torch.manual_seed(13)
    pad = k // 2
    assert C.conv_dgrad_supported(N, HW, HW, Ci, Co, k, 1, pad)
    dy = torch.randn(N, Co, HW, HW, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(Co, Ci, k, k, device="cuda") * 0.1).bfloat16().contiguous(memory_format=torch.channels_last)
    dx = C.conv_dgrad(dy, w, 1, pad)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0
    ref = torch.nn.grad.conv2d_input((N, Ci, HW, HW), w.float(), dy.float(), stride=1, padding=pad)
    assert dx.shape == ref.shape and dx.is_contiguous(memory_format=torch.channels_last)
    err = (dx.float() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 0.01, f"max err {err} (ref max {ref.abs().max().item()})"


def test_conv_fprop_dgrad_reject_unsupported(C):
    assert not C.conv_fprop_supported(4, 32, 32, 3, 16, 3, 1, 1)       # 3-channel stem
    assert not C.conv_fprop_supported(4, 28, 28, 16, 32, 3, 2, 1)      # strided, width not a power of two
    assert not C.conv_fprop_supported(4, 4, 4, 32, 64, 3, 2, 1)        # strided, fewer than 64 output pixels per image
    assert not C.conv_fprop_supported(4, 32, 32, 16, 16, 5, 1, 2)      # 5x5
    assert not C.conv_dgrad_supported(4, 32, 32, 16, 32, 3, 2, 1)      # strided data gradient



def test_bn_from_conv_sums_matches_stats_pass(C):
    torch.manual_seed(14)
    N, Ci, Co, HW = 16, 16, 32, 32
    x = torch.randn(N, Ci, HW, HW, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(Co, Ci, 3, 3, device="cuda") * 0.1).bfloat16().contiguous(memory_format=torch.channels_last)
    res = torch.randn(N, Co, HW, HW, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
    gamma, beta = torch.rand(Co, device="cuda") + 0.5, torch.randn(Co, device="cuda")
    sums = torch.zeros(2, Co, device="cuda")
    y = C.conv_fprop(x, w, 1, 1, sums)
    rm1, rv1 = torch.zeros(Co, device="cuda"), torch.ones(Co, device="cuda")
    rm2, rv2 = rm1.clone(), rv1.clone()
    o1, m1, r1 = C.bn_fwd(y, res, gamma, beta, rm1, rv1, 1e-5, 0.1, True, True)
    o2, m2, r2 = C.bn_fwd(y, res, gamma, beta, rm2, rv2, 1e-5, 0.1, True, True, sums)
    torch.cuda.synchronize()
    assert (m1 - m2).abs().max().item() < 1e-4
    assert ((r1 - r2).abs() / r1.abs()).max().item() < 1e-3
    assert (rm1 - rm2).abs().max().item() < 1e-4 and (rv1 - rv2).abs().max().item() < 1e-3
    assert (o1.float() - o2.float()).abs().max().item() <= 0.04


def test_eager_adam_on_unflattened_parameters_matches_torch(C):
    from flodl_b200 import nn
    torch.manual_seed(15)
    shapes = [(33, 17), (64,), (5, 4, 3)]
    ours = [nn.Parameter(torch.randn(*s, device="cuda"), f"p{i}") for i, s in enumerate(shapes)]
    ref = [p.t.detach().clone().requires_grad_(True) for p in ours]
    opt, ropt = nn.Adam(ours, 0.01), torch.optim.Adam(ref, lr=0.01)
    for step in range(3):
        for p, r in zip(ours, ref):
            g = torch.randn_like(r)
            p.t.grad = g.clone()
            r.grad = g.clone()
        opt.step()
        ropt.step()
    for p, r in zip(ours, ref):
        assert (p.t.detach() - r.detach()).abs().max().item() < 1e-5


@pytest.mark.parametrize("config", [0, 2])
def test_gemm_device_side_row_and_reduction_counts(C, config):
    """`m_dyn` / `k_dyn`: the kernel works on the device-side counts, buffers keep their static size."""
    torch.manual_seed(11)
    M, N, K, m_act = 1024, 512, 256, 300
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
    cnt = torch.tensor([m_act], device="cuda", dtype=torch.int32)
    C.clear_status(0)
    C.gemm(a, b, out, False, False, config=config, m_dyn=cnt)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0
    ref = a.float() @ b.float().t()
    assert (out[:m_act].float() - ref[:m_act]).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.05
    tile_m = 256 if config == 0 else 128
    first_untouched = (m_act + tile_m - 1) // tile_m * tile_m
    assert torch.all(out[first_untouched:] == 7.0), "tiles past the dynamic row count must not be written"
    # reduction length: dW[n, k] = sum_t dy[t, n] x[t, k] over the first k_act rows only (rows up to the
    # next multiple of 64 are zero, as the producers of such operands guarantee)
    T, k_act = 1024, 200
    dy = torch.randn(T, 384, device="cuda").bfloat16()
    x = torch.randn(T, 256, device="cuda").bfloat16()
    dy[k_act:256] = 0
    x[k_act:256] = 0
    dw = torch.zeros(384, 256, device="cuda")
    kc = torch.tensor([k_act], device="cuda", dtype=torch.int32)
    C.gemm(dy, x, dw, True, True, config=config, accumulate=True, k_dyn=kc)
    torch.cuda.synchronize()
    assert C.read_status(0) == 0
    ref = dy[:k_act].float().t() @ x[:k_act].float()
    assert (dw - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 0.05
    # a zero count leaves the output alone
    dw2 = torch.full((384, 256), 3.0, device="cuda")
    C.gemm(dy, x, dw2, True, True, config=config, accumulate=True, k_dyn=torch.zeros(1, device="cuda", dtype=torch.int32))
    torch.cuda.synchronize()
    assert torch.all(dw2 == 3.0)


def test_row_compaction_kernels(C):
    torch.manual_seed(5)
    rows, cols = 3000, 136
    tgt = torch.randint(0, 50, (rows,), device="cuda")
    tgt[torch.rand(rows, device="cuda") < 0.8] = -100
    idx, tc, counts = C.compact_targets(tgt, -100)
    n, n_pad = counts.tolist()
    act = (tgt != -100).nonzero().flatten()
    assert n == act.numel() and n_pad == min(rows, (n + 255) // 256 * 256)
    assert torch.equal(idx[:n].long(), act) and torch.equal(tc[:n], tgt[act]) and torch.all(tc[n:] == -100)
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    xc = torch.full_like(x, 9.0)
    C.gather_rows(x, idx, counts, xc)
    assert torch.equal(xc[:n], x[act]) and torch.all(xc[n:n_pad] == 0) and torch.all(xc[n_pad:] == 9.0)
    dx = torch.zeros_like(x)
    C.scatter_rows(xc, idx, counts, dx)
    ref = torch.zeros_like(x)
    ref[act] = x[act]
    assert torch.equal(dx, ref)
    # nothing active
    idx, tc, counts = C.compact_targets(torch.full((700,), -100, device="cuda"), -100)
    assert counts.tolist() == [0, 0]


def test_masked_lm_loss_on_labelled_rows_only_matches_full_projection():
    """The masked-LM head projects only the labelled rows; loss and every gradient must agree with the
    projection of all rows (ignored rows contribute nothing to either)."""
    from flodl_b200 import ops
    torch.manual_seed(9)
    rows, K, V = 2048, 256, 3000
    x0 = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w0 = (torch.randn(V, K, device="cuda") * 0.05)
    b0 = torch.randn(V, device="cuda") * 0.1
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[torch.rand(rows, device="cuda") < 0.85] = -100
    res = []
    for sparse in (False, True):
        x, w, b = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
        loss = ops.linear_cross_entropy(x, w, b, tgt, -100, sparse_targets=sparse)
        (loss * 1.5).backward()
        torch.cuda.synchronize()
        res.append((loss.item(), x.grad.float(), w.grad.float(), b.grad.float()))
    (l0, dx0, dw0, db0), (l1, dx1, dw1, db1) = res
    assert abs(l0 - l1) < 1e-4 * max(1.0, abs(l0)), (l0, l1)
    assert torch.equal(dx1[tgt == -100], torch.zeros_like(dx1[tgt == -100]))
    for a, b_, name in ((dx0, dx1, "dx"), (dw0, dw1, "dw"), (db0, db1, "db")):
        scale = a.abs().max().item() + 1e-12
        assert (a - b_).abs().max().item() <= 2e-2 * scale, (name, (a - b_).abs().max().item(), scale)
    # against fp32 PyTorch
    xr, wr, br = x0.float().requires_grad_(True), w0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    ref = F.cross_entropy(F.linear(xr, wr.bfloat16().float(), br), tgt, ignore_index=-100)
    (ref * 1.5).backward()
    assert abs(ref.item() - l1) < 5e-2      # bf16 logits against an fp32 projection
    assert (wr.grad - dw1).abs().max().item() <= 3e-2 * wr.grad.abs().max().item() + 1e-4


def test_bounds_checked_debug_build_records_instead_of_faulting():
    """The debug library (`FLODL_B200_BOUNDS_CHECK=1`, built beside the regular one) range-checks every
    index a kernel reads from device memory; see tests/_bounds_worker.py for the sweep."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, FLODL_B200_BOUNDS_CHECK="1")
    res = subprocess.run([sys.executable, os.path.join(here, "_bounds_worker.py")], capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0 and "BOUNDS_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
