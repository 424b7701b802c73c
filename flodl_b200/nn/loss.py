"""Loss functions (flodl/src/nn/loss.rs): every one returns a scalar `Variable` (mean reduction).

`cross_entropy_loss` is the fused softmax-CE kernel on CUDA; the others are the PyTorch fused
losses or the same compositions the reference writes out."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops as _ops
from ..autograd import Variable
from ..autograd.variable import _t
from ..tensor import TensorError

W = Variable.wrap


def mse_loss(pred, target) -> Variable:
    return W(F.mse_loss(_t(pred), _t(target)))


def cross_entropy_loss(pred, target) -> Variable:
    """2-D `[rows, classes]` logits; class-index targets use ignore_index -100; float targets are
    treated as class probabilities (flodl/src/nn/loss.rs:34-43)."""
    p, t = _t(pred), _t(target)
    if p.dim() != 2:
        raise TensorError("cross_entropy_loss expects [batch, classes] predictions")
    if t.is_floating_point():
        return W(F.cross_entropy(p, t))
    return W(_ops.cross_entropy(p, t.long(), -100))


def bce_loss(pred, target) -> Variable:
    return W(F.binary_cross_entropy(_t(pred), _t(target)))


def bce_with_logits_loss(pred, target) -> Variable:
    return W(F.binary_cross_entropy_with_logits(_t(pred), _t(target)))


def l1_loss(pred, target) -> Variable:
    return W(F.l1_loss(_t(pred), _t(target)))


def smooth_l1_loss(pred, target, beta: float = 1.0) -> Variable:
    return W(F.smooth_l1_loss(_t(pred), _t(target), beta=beta))


def kl_div_loss(input, target) -> Variable:
    """`input` holds log-probabilities; batchmean reduction."""
    return W(F.kl_div(_t(input), _t(target), reduction="batchmean"))


def nll_loss(input, target) -> Variable:
    return W(F.nll_loss(_t(input), _t(target).long()))


def ctc_loss(log_probs, targets, input_lengths, target_lengths, blank: int = 0) -> Variable:
    return W(F.ctc_loss(_t(log_probs), _t(targets), _t(input_lengths), _t(target_lengths), blank=blank))


def focal_loss(pred, target, alpha: float = 0.25, gamma: float = 2.0) -> Variable:
    logp = torch.log_softmax(_t(pred), -1)
    idx = _t(target).long().unsqueeze(-1)
    log_pt = logp.gather(1, idx).squeeze(-1)
    pt = log_pt.exp()
    return W((-(alpha * (1 - pt).pow(gamma)) * log_pt).mean())


def triplet_margin_loss(anchor, positive, negative, margin: float = 1.0) -> Variable:
    a, p, n = _t(anchor), _t(positive), _t(negative)
    d_pos = (a - p).pow(2).sum(1).sqrt()
    d_neg = (a - n).pow(2).sum(1).sqrt()
    return W((d_pos - d_neg + margin).clamp_min(0).mean())


def cosine_embedding_loss(x1, x2, label, margin: float = 0.0) -> Variable:
    cos = F.cosine_similarity(_t(x1), _t(x2), 1, 1e-8)
    lab = _t(label)
    pos, neg = (1 + lab) * 0.5, (1 - lab) * 0.5
    return W((pos * (1 - cos) + neg * (cos - margin).clamp_min(0)).mean())


def hinge_embedding_loss(input, label, margin: float = 1.0) -> Variable:
    x, lab = _t(input), _t(label)
    pos, neg = (1 + lab) * 0.5, (1 - lab) * 0.5
    return W((pos * x + neg * (margin - x).clamp_min(0)).mean())


def margin_ranking_loss(x1, x2, label, margin: float = 0.0) -> Variable:
    return W((-_t(label) * (_t(x1) - _t(x2)) + margin).clamp_min(0).mean())


def poisson_nll_loss(input, target, log_input: bool = True) -> Variable:
    x, t = _t(input), _t(target)
    loss = x.exp() - t * x if log_input else x - t * (x + 1e-8).log()
    return W(loss.mean())
