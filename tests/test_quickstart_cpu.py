"""The quick-start MLP on CPU, fp32, seed 0: Linear(2,16) -> GELU -> LayerNorm(16) -> residual
Linear(16,16) via `.also` -> Linear(16,2); x ~ N(0,1) [32,2], target [sin x0, cos x1]; MSE, Adam
lr 0.01, clip_grad_norm 1.0, 200 steps. Checked against the same model written in plain PyTorch."""
import torch

from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import FlowBuilder


def build():
    torch.manual_seed(0)
    return (FlowBuilder.from_(nn.Linear(2, 16)).through(nn.GELU()).through(nn.LayerNorm(16)).also(nn.Linear(16, 16))
            .through(nn.Linear(16, 2)).build())


def data():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(32, 2, generator=g)
    return x, torch.stack([torch.sin(x[:, 0]), torch.cos(x[:, 1])], dim=1)


def test_mlp_trains_and_matches_plain_pytorch():
    model = build()
    x, y = data()
    # the same weights in a torch.nn model
    w = [p.t.detach().clone() for p in model.parameters()]
    names = [n for n, _ in model.named_parameters()]
    assert names == ["linear_1/weight", "linear_1/bias", "layernorm_3/weight", "layernorm_3/bias", "linear_4/weight",
                     "linear_4/bias", "linear_6/weight", "linear_6/bias"], names
    ref = [t.clone().requires_grad_(True) for t in w]
    ropt = torch.optim.Adam(ref, lr=0.01)

    def ref_forward(x):
        h = torch.nn.functional.gelu(torch.nn.functional.linear(x, ref[0], ref[1]))
        h = torch.nn.functional.layer_norm(h, (16,), ref[2], ref[3], 1e-5)
        h = h + torch.nn.functional.linear(h, ref[4], ref[5])
        return torch.nn.functional.linear(h, ref[6], ref[7])

    opt = nn.Adam(model.parameters(), 0.01)
    model.set_training(True)
    losses, ref_losses = [], []
    for _ in range(200):
        loss = nn.mse_loss(model.forward(Variable.wrap(x)), Variable.wrap(y))
        loss.backward()
        nn.clip_grad_norm(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
        rl = torch.nn.functional.mse_loss(ref_forward(x), y)
        ropt.zero_grad()
        rl.backward()
        torch.nn.utils.clip_grad_norm_(ref, 1.0)
        ropt.step()
        ref_losses.append(float(rl))
    assert losses[-1] < 0.05 * losses[0], (losses[0], losses[-1])
    assert abs(losses[0] - ref_losses[0]) < 1e-6
    assert abs(losses[-1] - ref_losses[-1]) < 1e-3 * max(1.0, ref_losses[-1]) + 1e-4
    for p, r in zip(model.parameters(), ref):
        torch.testing.assert_close(p.t.detach(), r.detach(), atol=2e-3, rtol=2e-3)
