"""CPU tests of the nn layer: shapes, values against plain PyTorch, optimizer math, schedulers,
clipping, loss functions, GradScaler."""
import math

import pytest
import torch
import torch.nn.functional as F

from flodl_b200 import nn
from flodl_b200.autograd import Variable, no_grad


def V(t, rg=False):
    return Variable(t, requires_grad=rg)


# ---- layers ---------------------------------------------------------------------------------------
def test_linear_shapes_init_and_forward():
    torch.manual_seed(0)
    lin = nn.Linear(8, 4)
    names = [p.name for p in lin.parameters()]
    assert names == ["weight", "bias"]
    w, b = (p.t for p in lin.parameters())
    assert list(w.shape) == [4, 8] and list(b.shape) == [4]
    bound = 1.0 / math.sqrt(8)          # kaiming_uniform(a=sqrt(5)) on [out,in] -> U(-1/sqrt(in), 1/sqrt(in))
    assert w.abs().max() <= bound + 1e-6 and b.abs().max() <= bound + 1e-6
    x = torch.randn(5, 8)
    y = lin.forward(V(x))
    torch.testing.assert_close(y.t, F.linear(x, w, b))
    nb = nn.Linear.no_bias(8, 4)
    assert len(nb.parameters()) == 1


def test_linear_backward_matches_torch():
    torch.manual_seed(1)
    lin = nn.Linear(6, 3)
    x = torch.randn(4, 6, requires_grad=True)
    y = lin.forward(V(x)).t.pow(2).sum()
    y.backward()
    w, b = (p.t for p in lin.parameters())
    x2 = x.detach().clone().requires_grad_(True)
    w2, b2 = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    F.linear(x2, w2, b2).pow(2).sum().backward()
    torch.testing.assert_close(w.grad, w2.grad)
    torch.testing.assert_close(b.grad, b2.grad)
    torch.testing.assert_close(x.grad, x2.grad)


def test_shared_weight_linear_dedups_parameters():
    a = nn.Linear(4, 4)
    b = nn.Linear.from_shared_weight(a.parameters()[0], None)
    m = nn.modules(a, b) if callable(getattr(nn, "modules", None)) else None
    ids = {p.key() for p in a.parameters()} | {p.key() for p in b.parameters()}
    assert len(ids) == 2           # weight (shared) + a's bias


def test_layernorm_matches_torch_and_eps_default():
    torch.manual_seed(2)
    ln = nn.LayerNorm(16)
    x = torch.randn(3, 16)
    w, b = (p.t for p in ln.parameters())
    torch.testing.assert_close(ln.forward(V(x)).t, F.layer_norm(x, (16,), w, b, 1e-5))
    ln12 = nn.LayerNorm.with_eps(16, 1e-12)
    torch.testing.assert_close(ln12.forward(V(x)).t, F.layer_norm(x, (16,), None, None, 1e-12))


def test_batchnorm_training_requires_two_samples_and_updates_running_stats():
    bn = nn.BatchNorm2d(3)
    bn.set_training(True)
    x = torch.randn(4, 3, 5, 5)
    y = bn.forward(V(x)).t
    assert y.shape == x.shape
    rm = [b for b in bn.buffers() if b.name == "running_mean"][0].get()
    torch.testing.assert_close(rm, 0.1 * x.mean(dim=(0, 2, 3)), atol=1e-6, rtol=1e-5)
    with pytest.raises(Exception):
        bn.forward(V(torch.randn(1, 3, 5, 5)))
    bn.set_training(False)
    assert bn.forward(V(torch.randn(1, 3, 5, 5))).t.shape == (1, 3, 5, 5)


def test_conv2d_builder_and_shapes():
    conv = nn.Conv2d.configure(3, 8, 3).with_stride(2).with_padding(1).without_bias().done()
    assert len(conv.parameters()) == 1
    y = conv.forward(V(torch.randn(2, 3, 16, 16)))
    assert list(y.t.shape) == [2, 8, 8, 8]


def test_embedding_padding_idx_gets_no_gradient():
    emb = nn.Embedding.with_padding_idx(10, 4, 0)
    idx = torch.tensor([[0, 1, 2], [0, 0, 3]])
    out = emb.forward(V(idx))
    out.t.sum().backward()
    g = emb.parameters()[0].t.grad
    assert g[0].abs().sum() == 0 and g[1].abs().sum() > 0


def test_multihead_attention_matches_decomposed_reference():
    torch.manual_seed(3)
    mha = nn.MultiheadAttention(16, 4)
    mha.set_training(False)
    x = torch.randn(2, 5, 16)
    y = mha.forward(V(x)).t
    ps = {p.name: p.t for p in mha.parameters()}
    assert len(ps) == 8
    assert y.shape == x.shape and torch.isfinite(y).all()


def test_dropout_eval_is_identity_and_train_scales():
    d = nn.Dropout(0.5)
    d.set_training(False)
    x = torch.ones(1000)
    assert torch.equal(d.forward(V(x)).t, x)
    d.set_training(True)
    y = d.forward(V(x)).t
    assert set(y.unique().tolist()) <= {0.0, 2.0}


def test_gru_lstm_shapes():
    g = nn.GRU(4, 8)
    out = g.forward(V(torch.randn(3, 7, 4)))
    assert out.t.shape[-1] == 8
    l = nn.LSTM(4, 8, 2)
    out = l.forward(V(torch.randn(3, 7, 4)))
    assert out.t.shape[-1] == 8


@pytest.mark.parametrize("name,ref", [
    ("ReLU", torch.relu), ("Sigmoid", torch.sigmoid), ("Tanh", torch.tanh), ("SiLU", F.silu), ("Mish", F.mish),
    ("SELU", F.selu), ("Hardswish", F.hardswish), ("Hardsigmoid", F.hardsigmoid), ("Softplus", F.softplus),
    ("Identity", lambda x: x),
])
def test_activations_match_torch(name, ref):
    x = torch.linspace(-3, 3, 41)
    torch.testing.assert_close(getattr(nn, name)().forward(V(x)).t, ref(x))


def test_gelu_exact_and_tanh():
    x = torch.linspace(-3, 3, 41)
    torch.testing.assert_close(nn.GELU().forward(V(x)).t, F.gelu(x))
    torch.testing.assert_close(nn.GELU.tanh().forward(V(x)).t, F.gelu(x, approximate="tanh"))


# ---- losses ---------------------------------------------------------------------------------------
def test_losses_match_torch():
    torch.manual_seed(4)
    p, t = torch.randn(6, 5), torch.randn(6, 5)
    torch.testing.assert_close(nn.mse_loss(V(p), V(t)).t, F.mse_loss(p, t))
    torch.testing.assert_close(nn.l1_loss(V(p), V(t)).t, F.l1_loss(p, t))
    torch.testing.assert_close(nn.smooth_l1_loss(V(p), V(t)).t, F.smooth_l1_loss(p, t))
    y = torch.tensor([0, 1, 4, -100, 2, 3])
    torch.testing.assert_close(nn.cross_entropy_loss(V(p), V(y)).t, F.cross_entropy(p, y, ignore_index=-100))
    prob = torch.sigmoid(p)
    tgt = (t > 0).float()
    torch.testing.assert_close(nn.bce_loss(V(prob), V(tgt)).t, F.binary_cross_entropy(prob, tgt))
    torch.testing.assert_close(nn.bce_with_logits_loss(V(p), V(tgt)).t, F.binary_cross_entropy_with_logits(p, tgt))
    lp = F.log_softmax(p, -1)
    torch.testing.assert_close(nn.nll_loss(V(lp), V(y.clamp(min=0))).t, F.nll_loss(lp, y.clamp(min=0)))


def test_cross_entropy_rejects_non_2d_prediction():
    with pytest.raises(Exception):
        nn.cross_entropy_loss(V(torch.randn(2, 3, 4)), V(torch.zeros(2, 3, dtype=torch.long)))


# ---- optimizers -----------------------------------------------------------------------------------
def _pair(shape=(5, 3)):
    torch.manual_seed(5)
    w = torch.randn(*shape)
    mine = nn.Parameter(w.clone(), "w")
    ref = w.clone().requires_grad_(True)
    return mine, ref


def _run(opt_mine, opt_ref, mine, ref, steps=5):
    for s in range(steps):
        g = torch.randn_like(ref) * (s + 1)
        mine.t.grad = g.clone()
        ref.grad = g.clone()
        opt_mine.step()
        opt_ref.step()
    return mine.t.detach(), ref.detach()


def test_adam_matches_torch():
    mine, ref = _pair()
    a, b = _run(nn.Adam([mine], 1e-2), torch.optim.Adam([ref], 1e-2), mine, ref)
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)


def test_adamw_matches_torch():
    mine, ref = _pair()
    a, b = _run(nn.AdamW([mine], 1e-2, 0.1), torch.optim.AdamW([ref], 1e-2, weight_decay=0.1), mine, ref)
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)


def test_sgd_momentum_weight_decay_matches_torch():
    mine, ref = _pair()
    a, b = _run(nn.SGD([mine], 0.1, 0.9, 1e-2), torch.optim.SGD([ref], 0.1, momentum=0.9, weight_decay=1e-2), mine, ref)
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)


def test_rmsprop_adagrad_match_torch():
    mine, ref = _pair()
    a, b = _run(nn.RMSprop([mine], 1e-2), torch.optim.RMSprop([ref], 1e-2), mine, ref)
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)
    mine, ref = _pair()
    a, b = _run(nn.Adagrad([mine], 1e-2), torch.optim.Adagrad([ref], 1e-2), mine, ref)
    torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)


def test_radam_nadam_match_torch():
    mine, ref = _pair()
    a, b = _run(nn.RAdam([mine], 1e-2), torch.optim.RAdam([ref], 1e-2), mine, ref, steps=8)
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-4)
    # NAdam here has no momentum-decay schedule (unlike torch.optim.NAdam): check the closed form
    mine, _ = _pair()
    opt = nn.NAdam([mine], 1e-2)
    w = mine.t.detach().clone().double()
    m = torch.zeros_like(w)
    v = torch.zeros_like(w)
    b1, b2, eps, lr = 0.9, 0.999, 1e-8, 1e-2
    for t in range(1, 6):
        g = torch.randn_like(mine.t)
        mine.t.grad = g.clone()
        opt.step()
        gd = g.double()
        m = b1 * m + (1 - b1) * gd
        v = b2 * v + (1 - b2) * gd * gd
        m_hat = m * b1 / (1 - b1 ** (t + 1)) + gd * (1 - b1) / (1 - b1 ** t)
        w = w - lr * m_hat / ((v / (1 - b2 ** t)).sqrt() + eps)
    torch.testing.assert_close(mine.t.detach().double(), w, atol=1e-5, rtol=1e-4)


def test_optimizer_skips_params_without_grad_and_zero_grad_sets_none():
    a, b = nn.Parameter(torch.ones(3), "a"), nn.Parameter(torch.ones(3), "b")
    opt = nn.Adam([a, b], 0.1)
    a.t.grad = torch.ones(3)
    opt.step()
    assert torch.equal(b.t.detach(), torch.ones(3)) and not torch.equal(a.t.detach(), torch.ones(3))
    opt.zero_grad()
    assert a.t.grad is None


def test_param_groups_and_lr_controls():
    a, b = nn.Parameter(torch.ones(2), "a"), nn.Parameter(torch.ones(2), "b")
    opt = nn.SGD.with_groups(momentum=0.0).group([a], 0.1).group([b], 1.0).build()
    a.t.grad, b.t.grad = torch.ones(2), torch.ones(2)
    opt.step()
    torch.testing.assert_close(a.t.detach(), torch.full((2,), 0.9))
    torch.testing.assert_close(b.t.detach(), torch.zeros(2))
    opt.set_group_lr(0, 0.5)
    opt.scale_lr(2.0)
    a.t.grad, b.t.grad = torch.ones(2), torch.ones(2)
    opt.step()
    torch.testing.assert_close(a.t.detach(), torch.full((2,), -0.1))
    torch.testing.assert_close(b.t.detach(), torch.full((2,), -2.0))


def test_adam_state_roundtrip():
    mine, ref = _pair()
    opt = nn.Adam([mine], 1e-2)
    for _ in range(3):
        mine.t.grad = torch.randn_like(mine.t)
        opt.step()
    blob = opt.state_bytes()
    w_before = mine.t.detach().clone()
    g = torch.randn_like(mine.t)
    mine.t.grad = g.clone()
    opt.step()
    after_a = mine.t.detach().clone()
    # fresh optimizer + restored state must take the same step
    fresh = nn.Parameter(w_before.clone(), "w")
    opt2 = nn.Adam([fresh], 1e-2)
    import io
    opt2.load_state(io.BytesIO(blob))
    fresh.t.grad = g.clone()
    opt2.step()
    torch.testing.assert_close(fresh.t.detach(), after_a, atol=1e-7, rtol=1e-6)


# ---- schedulers -----------------------------------------------------------------------------------
def test_schedulers():
    s = nn.StepDecay(1.0, 10, 0.5)
    assert s.lr(0) == 1.0 and s.lr(10) == 0.5 and s.lr(25) == 0.25
    c = nn.CosineScheduler(1.0, 0.0, 100)
    assert abs(c.lr(0) - 1.0) < 1e-9 and abs(c.lr(50) - 0.5) < 1e-9 and abs(c.lr(100)) < 1e-9
    w = nn.WarmupScheduler(nn.StepDecay(1.0, 1000, 0.5), 1.0, 10)
    assert w.lr(0) < w.lr(5) < w.lr(10) and abs(w.lr(10) - 1.0) < 1e-9
    e = nn.ExponentialLR(1.0, 0.9)
    assert abs(e.lr(3) - 0.9 ** 3) < 1e-12
    m = nn.MultiStepLR(1.0, [5, 8], 0.1)
    assert m.lr(4) == 1.0 and abs(m.lr(5) - 0.1) < 1e-12 and abs(m.lr(9) - 0.01) < 1e-12
    o = nn.OneCycleLR(1.0, 100)
    assert o.lr(0) < o.lr(30) and o.lr(99) < o.lr(30)
    cy = nn.CyclicLR(0.1, 1.0, 10)
    assert abs(cy.lr(0) - 0.1) < 1e-9 and abs(cy.lr(10) - 1.0) < 1e-9 and abs(cy.lr(20) - 0.1) < 1e-9


def test_plateau_scheduler_reduces_after_patience():
    p = nn.PlateauScheduler(1.0, 2, 0.5, 0.1)
    for v in (1.0, 1.0, 1.0, 1.0):
        p.observe(v)
    assert p.lr(0) < 1.0


# ---- clipping / amp -------------------------------------------------------------------------------
def test_clip_grad_norm_returns_preclip_norm_and_scales():
    a, b = nn.Parameter(torch.zeros(3), "a"), nn.Parameter(torch.zeros(4), "b")
    a.t.grad, b.t.grad = torch.full((3,), 3.0), torch.full((4,), 4.0)
    total = math.sqrt(9 * 3 + 16 * 4)
    n = nn.clip_grad_norm([a, b], 1.0)
    assert abs(n - total) < 1e-4
    new = math.sqrt(float(a.t.grad.pow(2).sum() + b.t.grad.pow(2).sum()))
    assert abs(new - 1.0) < 1e-3
    n2 = nn.clip_grad_norm([a, b], 10.0)       # below the limit: untouched
    assert abs(n2 - new) < 1e-5
    a.t.grad = torch.tensor([5.0, -5.0, 0.5])
    nn.clip_grad_value([a], 1.0)
    assert a.t.grad.abs().max() <= 1.0


def test_grad_scaler_backoff_and_growth():
    p = nn.Parameter(torch.ones(2), "p")
    opt = nn.SGD([p], 0.1)
    sc = nn.GradScaler(init_scale=4.0, growth=2.0, backoff=0.5, interval=2)
    p.t.grad = torch.tensor([float("inf"), 1.0])
    assert sc.step([p], opt.step) is False
    sc.update()
    assert sc.scale_factor() == 2.0 and torch.equal(p.t.detach(), torch.ones(2))
    for _ in range(2):
        p.t.grad = torch.tensor([2.0, 2.0])
        assert sc.step([p], opt.step) is True
        sc.update()
    assert sc.scale_factor() == 4.0


def test_init_functions_statistics():
    torch.manual_seed(6)
    t = nn.xavier_uniform([64, 32], 32, 64)
    bound = math.sqrt(6.0 / (64 + 32))
    assert t.abs().max() <= bound + 1e-6
    k = nn.kaiming_normal([256, 128], 128)
    assert abs(float(k.std()) - math.sqrt(2.0 / 128)) < 0.02
    o = nn.orthogonal([16, 16])
    torch.testing.assert_close(o @ o.T, torch.eye(16), atol=1e-4, rtol=1e-4)
    tn = nn.trunc_normal([1000], 0.0, 1.0, -2.0, 2.0)
    assert tn.min() >= -2.0 and tn.max() <= 2.0


def test_no_grad_context():
    x = V(torch.ones(3), rg=True)
    with no_grad():
        y = x.mul_scalar(2.0)
    assert not y.t.requires_grad
