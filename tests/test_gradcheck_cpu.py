"""Finite-difference checks of the differentiable op surface (the reference checks its ops the same
way: central differences against backward, flodl/src/autograd/mod.rs `numerical_grad`).

Every case builds a scalar from `Variable` ops in fp64, runs backward, and compares each input's
gradient with (f(x + h) - f(x - h)) / 2h element by element."""
import math

import pytest
import torch

from flodl_b200 import nn
from flodl_b200.autograd import Variable, ops as A

H = 1e-6
TOL = 1e-6


def numerical_grad(fn, tensors, i):
    x = tensors[i]
    g = torch.zeros_like(x)
    flat, gf = x.view(-1), g.view(-1)
    for k in range(flat.numel()):
        old = flat[k].item()
        flat[k] = old + H
        up = fn(*[Variable(t.clone()) for t in tensors]).t.sum().item()
        flat[k] = old - H
        dn = fn(*[Variable(t.clone()) for t in tensors]).t.sum().item()
        flat[k] = old
        gf[k] = (up - dn) / (2 * H)
    return g


def check(fn, *shapes, positive=False, seed=0, tol=TOL, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    tensors = []
    for s in shapes:
        t = torch.randn(*s, generator=g, dtype=torch.float64) * scale
        if positive:
            t = t.abs() + 0.5
        tensors.append(t)
    vs = [Variable(t.clone(), requires_grad=True) for t in tensors]
    out = fn(*vs)
    out.t.sum().backward()
    for i, v in enumerate(vs):
        num = numerical_grad(fn, tensors, i)
        ana = v.grad() if v.grad() is not None else torch.zeros_like(num)
        err = (ana - num).abs().max().item()
        assert err <= tol * max(1.0, num.abs().max().item()), f"input {i}: max |analytic - numeric| = {err}"


W = torch.linspace(-1.0, 1.0, 12, dtype=torch.float64).view(3, 4)
IDX = torch.tensor([[0, 2, 1, 0], [1, 1, 0, 2], [2, 0, 2, 1]])
PERM = torch.tensor([[3, 0, 2, 1], [1, 2, 0, 3], [0, 3, 1, 2]])      # a permutation per row: scatter without collisions

UNARY = {
    "neg": lambda x: x.neg(), "relu": lambda x: x.relu(), "sigmoid": lambda x: x.sigmoid(), "tanh": lambda x: x.tanh(),
    "gelu": lambda x: x.gelu(), "gelu_tanh": lambda x: x.gelu_tanh(), "silu": lambda x: x.silu(), "leaky_relu": lambda x: x.leaky_relu(0.1),
    "elu": lambda x: x.elu(1.0), "softplus": lambda x: x.softplus(1.0, 20.0), "mish": lambda x: x.mish(), "selu": lambda x: x.selu(),
    "hardswish": lambda x: x.hardswish(), "hardsigmoid": lambda x: x.hardsigmoid(), "exp": lambda x: x.exp(), "sin": lambda x: x.sin(),
    "cos": lambda x: x.cos(), "tan": lambda x: x.mul_scalar(0.3).tan(), "atan": lambda x: x.atan(), "erf": lambda x: x.erf(),
    "erfc": lambda x: x.erfc(), "abs": lambda x: x.abs(), "pow3": lambda x: x.pow_scalar(3.0), "mul_scalar": lambda x: x.mul_scalar(2.5),
    "div_scalar": lambda x: x.div_scalar(4.0), "add_scalar": lambda x: x.add_scalar(1.5), "clamp": lambda x: x.clamp(-0.5, 0.5),
    "clamp_min": lambda x: x.clamp_min(0.1), "clamp_max": lambda x: x.clamp_max(0.1), "expm1": lambda x: x.expm1(),
    "sum": lambda x: x.sum(), "mean": lambda x: x.mean(), "sum_dim": lambda x: x.sum_dim(1), "mean_dim": lambda x: x.mean_dim(0, True),
    "sum_dims": lambda x: x.sum_dims([0, 1]), "prod": lambda x: x.prod(), "prod_dim": lambda x: x.prod_dim(1), "cumsum": lambda x: x.cumsum(1),
    "cumprod": lambda x: x.cumprod(1), "logsumexp": lambda x: x.logsumexp(1), "min": lambda x: x.min(), "max": lambda x: x.max(),
    "min_dim": lambda x: x.min_dim(1), "max_dim": lambda x: x.max_dim(0), "var": lambda x: x.var(), "std": lambda x: x.std(),
    "var_dim": lambda x: x.var_dim(1), "std_dim": lambda x: x.std_dim(0), "norm": lambda x: x.norm(), "norm_p_dim": lambda x: x.norm_p_dim(3.0, 1),
    "median": lambda x: x.median(), "median_dim": lambda x: x.median_dim(1)[0], "softmax": lambda x: x.softmax(1).mul(Variable(W)),
    "log_softmax": lambda x: x.log_softmax(1).mul(Variable(W)), "normalize": lambda x: x.normalize(2.0, 1).mul(Variable(W)),
    "triu": lambda x: x.triu(0), "tril": lambda x: x.tril(-1), "reshape": lambda x: x.reshape([4, 3]).mul(Variable(W.t().contiguous())),
    "transpose": lambda x: x.transpose(0, 1).mul(Variable(W.t())), "permute": lambda x: x.permute([1, 0]).mul(Variable(W.t())),
    "unsqueeze_squeeze": lambda x: x.unsqueeze(1).squeeze(1).mul(Variable(W)), "flatten": lambda x: x.flatten().mul(Variable(W.flatten())),
    "expand": lambda x: x.unsqueeze(0).expand([2, 3, 4]).mul(Variable(torch.stack([W, 2 * W]))), "narrow": lambda x: x.narrow(1, 1, 2),
    "select": lambda x: x.select(0, 1), "index_select": lambda x: x.index_select(1, torch.tensor([3, 0, 0])),
    "gather": lambda x: x.gather(1, IDX.clamp(max=3)), "repeat": lambda x: x.repeat([2, 1]).mul(Variable(torch.cat([W, 3 * W]))),
    "tile": lambda x: x.tile([1, 2]).mul(Variable(torch.cat([W, -W], 1))), "pad": lambda x: x.pad([1, 2], 0.0),
    "pad_reflect": lambda x: x.unsqueeze(0).pad_mode([1, 1], 1), "flip": lambda x: x.flip([0, 1]).mul(Variable(W)),
    "roll": lambda x: x.roll(1, 1).mul(Variable(W)), "movedim": lambda x: x.movedim(0, 1).mul(Variable(W.t())),
    "diagonal": lambda x: x.diagonal(0, 0, 1), "chunk": lambda x: x.chunk(2, 1)[1], "split": lambda x: x.split(3, 1)[0].mul(Variable(W[:, :3])),
    "unbind": lambda x: x.unbind(0)[2], "masked_fill": lambda x: x.masked_fill(W > 0, 0.0), "topk": lambda x: x.topk(2, 1)[0],
    "sort": lambda x: x.sort(1)[0].mul(Variable(W)), "lerp": lambda x: x.lerp(Variable(W), 0.3), "fmod": lambda x: x.fmod_scalar(0.7),
    "remainder": lambda x: x.remainder_scalar(0.7), "frac": lambda x: x.frac(), "where": lambda x: Variable(W > 0).where(x, x.mul_scalar(2.0)),
    "scatter": lambda x: Variable(torch.zeros(3, 4, dtype=torch.float64)).scatter(1, PERM, x).mul(Variable(W)),
    "scatter_add": lambda x: Variable(torch.zeros(3, 4, dtype=torch.float64)).scatter_add(0, IDX, x).mul(Variable(W)),
    "select_scatter": lambda x: Variable(W).select_scatter(x.select(0, 0), 0, 1), "narrow_scatter": lambda x: Variable(W).narrow_scatter(x.narrow(1, 0, 2), 1, 1),
    "index_add": lambda x: Variable(W).index_add(0, torch.tensor([0, 0, 2]), x).mul(Variable(W)),
    "interpolate": lambda x: x.reshape([1, 1, 3, 4]).interpolate([6, 8], 1).mul_scalar(0.5),
    "layer_norm": lambda x: A.layer_norm(x, Variable(W[0]), Variable(W[1])).mul(Variable(W)),
    "dropout_eval": lambda x: A.dropout(x, 0.5, training=False),
}

POSITIVE = {"log": lambda x: x.log(), "sqrt": lambda x: x.sqrt(), "reciprocal": lambda x: x.reciprocal(), "log1p": lambda x: x.log1p(),
            "log2": lambda x: x.log2(), "log10": lambda x: x.log10(), "pow_half": lambda x: x.pow_scalar(0.5), "asin": lambda x: x.mul_scalar(0.2).asin(),
            "acos": lambda x: x.mul_scalar(0.2).acos()}

BINARY = {
    "add": lambda a, b: a.add(b), "sub": lambda a, b: a.sub(b), "mul": lambda a, b: a.mul(b), "div": lambda a, b: a.div(b.abs().add_scalar(0.5)),
    "matmul": lambda a, b: a.matmul(b.transpose(0, 1)), "atan2": lambda a, b: a.atan2(b.abs().add_scalar(0.5)), "maximum": lambda a, b: a.maximum(b),
    "minimum": lambda a, b: a.minimum(b), "cat": lambda a, b: a.cat(b, 1).mul(Variable(torch.cat([W, 2 * W], 1))), "cat2": lambda a, b: a.cat2(b, 0),
    "stack": lambda a, b: Variable.stack([a, b], 0).mul(Variable(torch.stack([W, -W]))), "lerp_tensor": lambda a, b: a.lerp_tensor(b, Variable(W.abs())),
    "fmod_tensor": lambda a, b: a.fmod_tensor(b.abs().add_scalar(1.0)), "addcmul": lambda a, b: Variable(W).addcmul(a, b, 0.5),
    "addcdiv": lambda a, b: Variable(W).addcdiv(a, b.abs().add_scalar(0.5), 0.5), "cosine_similarity": lambda a, b: a.cosine_similarity(b, 1, 1e-8),
    "cdist": lambda a, b: a.cdist(b), "mse_loss": lambda a, b: nn.mse_loss(a, b), "l1_loss": lambda a, b: nn.l1_loss(a, b),
    "smooth_l1": lambda a, b: nn.smooth_l1_loss(a, b, 0.5), "bce_logits": lambda a, b: nn.bce_with_logits_loss(a, b.sigmoid()),
    "kl_div": lambda a, b: nn.kl_div_loss(a.log_softmax(1), b.softmax(1)),
}


@pytest.mark.parametrize("name", sorted(UNARY))
def test_unary_and_shape_ops(name):
    check(UNARY[name], (3, 4), seed=sum(map(ord, name)))


@pytest.mark.parametrize("name", sorted(POSITIVE))
def test_positive_domain_ops(name):
    check(POSITIVE[name], (3, 4), positive=True, seed=sum(map(ord, name)))


@pytest.mark.parametrize("name", sorted(BINARY))
def test_binary_ops_and_losses(name):
    check(BINARY[name], (3, 4), (3, 4), seed=sum(map(ord, name)))


def test_linear_bilinear_and_addmm():
    check(lambda x, w, b: A.linear(x, w, b), (5, 4), (3, 4), (3,))
    check(lambda x, w: A.linear(x, w), (2, 5, 4), (3, 4))
    check(lambda a, m1, m2: a.addmm(m1, m2, 0.5, 2.0), (3, 3), (3, 4), (4, 3))
    check(lambda x1, x2, w, b: A.bilinear(x1, x2, w, b), (4, 3), (4, 2), (5, 3, 2), (5,))


def test_normalisations():
    check(lambda x, w, b: A.group_norm(x, 2, w, b), (2, 4, 3), (4,), (4,), tol=1e-5)
    check(lambda x, w, b: A.instance_norm(x, w, b), (2, 3, 5), (3,), (3,), tol=1e-5)
    check(lambda x, w, b: A.batch_norm(x, None, None, w, b, training=True), (4, 3, 2, 2), (3,), (3,), tol=1e-5)
    rms = nn.RMSNorm(4)
    rms.weight.t.data = torch.linspace(0.5, 1.5, 4, dtype=torch.float64)
    check(lambda x: rms.forward(x).mul(Variable(W)), (3, 4), tol=1e-5)


def test_convolutions_and_pooling():
    check(lambda x, w, b: A.conv1d(x, w, b, stride=2, padding=1), (2, 3, 8), (4, 3, 3), (4,))
    check(lambda x, w, b: A.conv2d(x, w, b, stride=1, padding=1), (1, 2, 5, 5), (3, 2, 3, 3), (3,))
    check(lambda x, w: A.conv2d(x, w, None, stride=2, padding=1, dilation=1, groups=2), (1, 4, 6, 6), (4, 2, 3, 3))
    check(lambda x, w: A.conv3d(x, w, None, padding=1), (1, 2, 3, 4, 4), (2, 2, 3, 3, 3))
    check(lambda x, w: A.conv_transpose1d(x, w, None, stride=2, padding=1, output_padding=1), (1, 3, 5), (3, 2, 3))
    check(lambda x, w, b: A.conv_transpose2d(x, w, b, stride=2, padding=1, output_padding=1), (1, 2, 3, 3), (2, 3, 3, 3), (3,))
    check(lambda x, w: A.conv_transpose3d(x, w, None, stride=1), (1, 2, 2, 3, 3), (2, 2, 2, 2, 2))
    check(lambda x: A.max_pool2d(x, 2), (1, 2, 4, 4))
    check(lambda x: A.avg_pool2d(x, 2, stride=1, padding=1), (1, 2, 4, 4))
    check(lambda x: A.max_pool1d(x, 2), (1, 2, 6))
    check(lambda x: A.avg_pool1d(x, 3, stride=2), (1, 2, 7))
    check(lambda x: A.adaptive_avg_pool2d(x, [2, 2]), (1, 2, 5, 5))
    check(lambda x: A.adaptive_max_pool2d(x, [2, 2]), (1, 2, 4, 4))
    check(lambda x: A.im2col(x, [2, 2]), (1, 2, 3, 3))
    check(lambda x: A.col2im(x, [3, 3], [2, 2]), (1, 8, 4))
    check(lambda x: A.pixel_shuffle(x, 2).mul_scalar(1.5), (1, 4, 2, 2))
    check(lambda x: A.pixel_unshuffle(x, 2).mul_scalar(1.5), (1, 1, 4, 4))


def test_attention_embedding_and_cells():
    check(lambda q, k, v: A.scaled_dot_product_attention(q, k, v), (1, 2, 3, 4), (1, 2, 5, 4), (1, 2, 5, 4), tol=1e-5)
    check(lambda q, k, v: A.scaled_dot_product_attention(q, k, v, is_causal=True), (1, 1, 4, 4), (1, 1, 4, 4), (1, 1, 4, 4), tol=1e-5)
    ids = torch.tensor([[0, 2], [3, 3]])
    check(lambda w: A.embedding(w, ids), (5, 3))
    w = Variable(torch.randn(5, 3, dtype=torch.float64), requires_grad=True)
    A.embedding(w, ids, padding_idx=3).sum().backward()       # the padding row is frozen: its gradient is zero by definition
    assert torch.all(w.grad()[3] == 0) and torch.all(w.grad()[0] == 1)
    check(lambda w: A.embedding_bag(w, torch.tensor([0, 2, 3, 3, 1]), torch.tensor([0, 2]), "sum"), (5, 3))
    check(lambda x, h, wi, wh, bi, bh: A.gru_cell(x, h, wi, wh, bi, bh), (2, 3), (2, 4), (12, 3), (12, 4), (12,), (12,), tol=1e-5)
    check(lambda x, h, c, wi, wh: A.lstm_cell(x, h, c, wi, wh)[0], (2, 3), (2, 4), (2, 4), (16, 3), (16, 4), tol=1e-5)
    grid = torch.tensor([[[[-0.5, -0.5], [0.3, 0.1]], [[0.0, 0.7], [0.9, -0.2]]]], dtype=torch.float64)
    check(lambda x: A.grid_sample(x, Variable(grid)), (1, 2, 3, 3), tol=1e-5)


def test_classification_losses():
    tgt = torch.tensor([1, 0, 3])
    check(lambda x: nn.cross_entropy_loss(x, Variable(tgt)), (3, 4))
    check(lambda x: nn.nll_loss(x.log_softmax(1), Variable(tgt)), (3, 4))
    check(lambda x: nn.bce_loss(x.sigmoid(), Variable(torch.tensor([[1.0, 0.0, 1.0, 0.0]] * 3, dtype=torch.float64))), (3, 4))
    check(lambda x: nn.focal_loss(x, Variable(tgt)), (3, 4), tol=1e-5)
    check(lambda a, p, n: nn.triplet_margin_loss(a, p, n, 1.0), (3, 4), (3, 4), (3, 4), tol=1e-5)
    lab = torch.tensor([1.0, -1.0, 1.0], dtype=torch.float64)
    check(lambda a, b: nn.cosine_embedding_loss(a, b, Variable(lab)), (3, 4), (3, 4), tol=1e-5)
    check(lambda a, b: nn.margin_ranking_loss(a.sum_dim(1), b.sum_dim(1), Variable(lab), 0.1), (3, 4), (3, 4))
    check(lambda x: nn.hinge_embedding_loss(x.sum_dim(1), Variable(lab)), (3, 4))
    check(lambda x: nn.poisson_nll_loss(x, Variable(W.abs())), (3, 4))
