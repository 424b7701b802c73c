"""The remaining `Tensor` methods of the reference by their own names (flodl/src/tensor/ops.rs,
shape.rs, nn_ops.rs, mod.rs), over `torch.Tensor`: scalar arithmetic, per-dimension reductions,
activations, the raw NN ops (convolutions, pooling, norms, RNN cells, losses with integer reduction
codes), conversions and the optimizer primitives.

`flodl_b200.tensor_ops` holds the comparison / math-extension set; this module the rest, so that every
`t.name(args)` of the reference has a `name(t, args)` here (`tensor_ops.surface()` lists both). These are
the no-autograd-wrapper forms: they take and return `torch.Tensor`s. Integer codes follow the C shim:
reduction 0 = none, 1 = mean, 2 = sum; `grid_sample` mode 0 = bilinear, 1 = nearest, 2 = bicubic and
padding 0 = zeros, 1 = border, 2 = reflection; `embedding_bag` mode 0 = sum, 1 = mean, 2 = max.
"""
from __future__ import annotations

import struct
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .tensor import DType, TensorError, TensorOptions, _dev

T = torch.Tensor
_RED = {0: "none", 1: "mean", 2: "sum"}


def _red(code) -> str:
    if isinstance(code, str):
        return code
    if int(code) not in _RED:
        raise TensorError(f"reduction code {code}: expected 0 (none), 1 (mean) or 2 (sum)")
    return _RED[int(code)]


# ---- scalar arithmetic (ops.rs "Scalar ops") --------------------------------------------------------
def add_scalar(t: T, s: float) -> T: return t + s
def mul_scalar(t: T, s: float) -> T: return t * s
def div_scalar(t: T, s: float) -> T: return t / s
def pow_scalar(t: T, exponent: float) -> T: return t.pow(exponent)
def add_scalar_(t: T, s: float) -> None: t.add_(s)
def mul_scalar_(t: T, s: float) -> None: t.mul_(s)
def div_scalar_(t: T, s: float) -> None: t.div_(s)


# ---- reductions along one dimension (values only; ops.rs "Reductions") ------------------------------
def sum_dim(t: T, dim: int, keepdim: bool = False) -> T: return t.sum(dim, keepdim)
def mean_dim(t: T, dim: int, keepdim: bool = False) -> T: return t.mean(dim, keepdim)
def prod_dim(t: T, dim: int, keepdim: bool = False) -> T: return t.prod(dim, keepdim)
def max_dim(t: T, dim: int, keepdim: bool = False) -> T: return t.max(dim, keepdim).values
def min_dim(t: T, dim: int, keepdim: bool = False) -> T: return t.min(dim, keepdim).values
def var_dim(t: T, dim: int, keepdim: bool = False) -> T: return t.var(dim, keepdim=keepdim)
def std_dim(t: T, dim: int, keepdim: bool = False) -> T: return t.std(dim, keepdim=keepdim)
def norm_p(t: T, p: float, dim: int, keepdim: bool = False) -> T: return torch.linalg.vector_norm(t, p, dim, keepdim)
def normalize(t: T, p: float = 2.0, dim: int = 1) -> T: return F.normalize(t, p, dim)
def cosine_similarity(t: T, other: T, dim: int = 1, eps: float = 1e-8) -> T: return F.cosine_similarity(t, other, dim, eps)
def cdist_p(t: T, other: T, p: float) -> T: return torch.cdist(t, other, p)


# ---- activations (ops.rs "Activations") --------------------------------------------------------------
def gelu(t: T) -> T: return F.gelu(t)
def gelu_tanh(t: T) -> T: return F.gelu(t, approximate="tanh")
def silu(t: T) -> T: return F.silu(t)
def selu(t: T) -> T: return F.selu(t)
def mish(t: T) -> T: return F.mish(t)
def hardswish(t: T) -> T: return F.hardswish(t)
def hardsigmoid(t: T) -> T: return F.hardsigmoid(t)
def elu(t: T, alpha: float = 1.0) -> T: return F.elu(t, alpha)
def leaky_relu(t: T, negative_slope: float = 0.01) -> T: return F.leaky_relu(t, negative_slope)
def softplus(t: T, beta: float = 1.0, threshold: float = 20.0) -> T: return F.softplus(t, beta, threshold)
def dropout(t: T, p: float, training: bool) -> T: return F.dropout(t, p, training)
def feature_dropout(t: T, p: float, training: bool) -> T: return torch.feature_dropout(t, p, training)


# ---- shape helpers (shape.rs) ------------------------------------------------------------------------
def cat(t: T, other: T, dim: int = 0) -> T: return torch.cat([t, other], dim)
def cat_many(tensors: Sequence[T], dim: int = 0) -> T: return torch.cat(list(tensors), dim)
def stack(tensors: Sequence[T], dim: int = 0) -> T: return torch.stack(list(tensors), dim)
def where_cond(condition: T, x: T, y: T) -> T: return torch.where(condition if condition.dtype == torch.bool else condition != 0, x, y)
def pad(t: T, padding: Sequence[int], value: float = 0.0) -> T: return F.pad(t, list(padding), value=value)


def unsqueeze_many(t: T, dims: Sequence[int]) -> T:
    """Insert size-1 dimensions one after the other, each index read against the tensor so far."""
    for d in dims:
        t = t.unsqueeze(d)
    return t


def batches(t: T, batch_size: int) -> List[T]:
    """Views of at most `batch_size` rows each, covering dimension 0 in order (shape.rs:328-338)."""
    if batch_size <= 0:
        raise TensorError("batches: batch_size must be positive")
    n = t.shape[0]
    return [t.narrow(0, s, min(batch_size, n - s)) for s in range(0, n, batch_size)]


# ---- raw NN ops (nn_ops.rs; argument order of the C shim) -------------------------------------------
def linear(t: T, weight: T, bias: Optional[T] = None) -> T: return F.linear(t, weight, bias)
def conv1d(t, weight, bias=None, stride=1, padding=0, dilation=1, groups=1): return F.conv1d(t, weight, bias, stride, padding, dilation, groups)
def conv2d(t, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1): return F.conv2d(t, weight, bias, tuple(stride), tuple(padding), tuple(dilation), groups)
def conv3d(t, weight, bias=None, stride=(1, 1, 1), padding=(0, 0, 0), dilation=(1, 1, 1), groups=1): return F.conv3d(t, weight, bias, tuple(stride), tuple(padding), tuple(dilation), groups)


def conv_transpose1d(t, weight, bias=None, stride=1, padding=0, output_padding=0, dilation=1, groups=1):
    return F.conv_transpose1d(t, weight, bias, stride, padding, output_padding, groups, dilation)


def conv_transpose2d(t, weight, bias=None, stride=(1, 1), padding=(0, 0), output_padding=(0, 0), dilation=(1, 1), groups=1):
    return F.conv_transpose2d(t, weight, bias, tuple(stride), tuple(padding), tuple(output_padding), groups, tuple(dilation))


def conv_transpose3d(t, weight, bias=None, stride=(1, 1, 1), padding=(0, 0, 0), output_padding=(0, 0, 0), dilation=(1, 1, 1), groups=1):
    return F.conv_transpose3d(t, weight, bias, tuple(stride), tuple(padding), tuple(output_padding), groups, tuple(dilation))


def max_pool1d(t, kernel_size, stride, padding=0, dilation=1, ceil_mode=False): return F.max_pool1d(t, kernel_size, stride, padding, dilation, ceil_mode)
def max_pool2d(t, kernel_size, stride, padding=(0, 0), dilation=(1, 1), ceil_mode=False): return F.max_pool2d(t, tuple(kernel_size), tuple(stride), tuple(padding), tuple(dilation), ceil_mode)
def avg_pool1d(t, kernel_size, stride, padding=0, ceil_mode=False, count_include_pad=True): return F.avg_pool1d(t, kernel_size, stride, padding, ceil_mode, count_include_pad)
def avg_pool2d(t, kernel_size, stride, padding=(0, 0), ceil_mode=False, count_include_pad=True): return F.avg_pool2d(t, tuple(kernel_size), tuple(stride), tuple(padding), ceil_mode, count_include_pad)
def adaptive_avg_pool2d(t, output_size): return F.adaptive_avg_pool2d(t, tuple(output_size))
def adaptive_max_pool2d(t, output_size): return F.adaptive_max_pool2d(t, tuple(output_size))
def im2col(t, kernel_size, dilation, padding, stride): return F.unfold(t, tuple(kernel_size), tuple(dilation), tuple(padding), tuple(stride))
def col2im(t, output_size, kernel_size, dilation, padding, stride): return F.fold(t, tuple(output_size), tuple(kernel_size), tuple(dilation), tuple(padding), tuple(stride))
def pixel_shuffle(t, upscale_factor): return F.pixel_shuffle(t, upscale_factor)
def pixel_unshuffle(t, downscale_factor): return F.pixel_unshuffle(t, downscale_factor)
def bilinear(input1, input2, weight, bias=None): return F.bilinear(input1, input2, weight, bias)


def grid_sample(t, grid, mode: int = 0, padding_mode: int = 0, align_corners: bool = False):
    return F.grid_sample(t, grid, mode=("bilinear", "nearest", "bicubic")[mode], padding_mode=("zeros", "border", "reflection")[padding_mode],
                         align_corners=align_corners)


def native_layer_norm(t, weight, bias, normalized_size: int, eps: float) -> Tuple[T, T, T]:
    """(output, mean, rstd) of a LayerNorm over the last dimension (ops_tensor.cpp:442-460)."""
    return torch.native_layer_norm(t, [int(normalized_size)], weight, bias, eps)


def group_norm(t, num_groups, weight=None, bias=None, eps=1e-5): return F.group_norm(t, num_groups, weight, bias, eps)


def batch_norm(t, weight=None, bias=None, running_mean=None, running_var=None, training=False, momentum=0.1, eps=1e-5):
    return F.batch_norm(t, running_mean, running_var, weight, bias, training, momentum, eps)


def instance_norm(t, weight=None, bias=None, running_mean=None, running_var=None, use_input_stats=True, momentum=0.1, eps=1e-5):
    return F.instance_norm(t, running_mean, running_var, weight, bias, use_input_stats, momentum, eps)


def embedding(weight: T, indices: T, padding_idx: int = -1) -> T:
    return F.embedding(indices, weight, padding_idx if padding_idx >= 0 else None)


def embedding_bag(weight: T, indices: T, offsets: T, mode: int = 1) -> T:
    return F.embedding_bag(indices, weight, offsets, mode=("sum", "mean", "max")[mode])


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None):
    return F.scaled_dot_product_attention(query, key, value, attn_mask, dropout_p, is_causal, scale=scale)


def gru_cell(t, hx, w_ih, w_hh, b_ih, b_hh): return torch.gru_cell(t, hx, w_ih, w_hh, b_ih, b_hh)
def lstm_cell(t, hx, cx, w_ih, w_hh, b_ih, b_hh): return tuple(torch.lstm_cell(t, (hx, cx), w_ih, w_hh, b_ih, b_hh))


class RnnParams:
    """The weight list of a multi-layer GRU / LSTM kept in the order the fused sequence op wants
    (`w_ih, w_hh, b_ih, b_hh` per layer), so that repeated calls do not rebuild it
    (`RnnParams`, flodl/src/tensor/nn_ops.rs)."""

    def __init__(self, params: Sequence[T], num_layers: int, has_biases: bool = True):
        self.params, self.num_layers, self.has_biases = list(params), int(num_layers), bool(has_biases)

    @classmethod
    def new(cls, params, num_layers, has_biases=True): return cls(params, num_layers, has_biases)


def gru_seq(t, h_0, params: Sequence[T], num_layers: int, batch_first: bool, flatten: bool = False) -> Tuple[T, T]:
    """Fused multi-layer GRU over a sequence: (output, h_n). `flatten` asks cuDNN to re-pack the weights first."""
    ps = list(params)
    if flatten and t.is_cuda:
        torch._cudnn_rnn_flatten_weight(ps, 4, ps[0].shape[1], 3, ps[1].shape[1], 0, num_layers, batch_first, False)
    return torch.gru(t, h_0, ps, True, num_layers, 0.0, False, False, batch_first)


def gru_seq_cached(t, h_0, params: RnnParams, num_layers: int, batch_first: bool) -> Tuple[T, T]:
    return torch.gru(t, h_0, params.params, params.has_biases, num_layers, 0.0, False, False, batch_first)


def lstm_seq(t, h_0, c_0, params: Sequence[T], num_layers: int, batch_first: bool, flatten: bool = False) -> Tuple[T, T, T]:
    ps = list(params)
    if flatten and t.is_cuda:
        torch._cudnn_rnn_flatten_weight(ps, 4, ps[0].shape[1], 2, ps[1].shape[1], 0, num_layers, batch_first, False)
    return torch.lstm(t, (h_0, c_0), ps, True, num_layers, 0.0, False, False, batch_first)


def lstm_seq_cached(t, h_0, c_0, params: RnnParams, num_layers: int, batch_first: bool) -> Tuple[T, T, T]:
    return torch.lstm(t, (h_0, c_0), params.params, params.has_biases, num_layers, 0.0, False, False, batch_first)


# ---- losses with the shim's integer reduction codes (ops_training.cpp:916-1021) ----------------------
def mse_loss(t, target, reduction=1): return F.mse_loss(t, target, reduction=_red(reduction))
def l1_loss(t, target, reduction=1): return F.l1_loss(t, target, reduction=_red(reduction))
def smooth_l1_loss(t, target, reduction=1, beta=1.0): return F.smooth_l1_loss(t, target, reduction=_red(reduction), beta=beta)
def bce_loss(t, target, reduction=1): return F.binary_cross_entropy(t, target, reduction=_red(reduction))
def bce_with_logits_loss(t, target, reduction=1): return F.binary_cross_entropy_with_logits(t, target, reduction=_red(reduction))
def nll_loss(t, target, reduction=1, ignore_index=-100): return F.nll_loss(t, target, reduction=_red(reduction), ignore_index=ignore_index)


def kl_div_loss(t, target, reduction=1, log_target=False):
    r = _red(reduction)
    return F.kl_div(t, target, reduction="batchmean" if r == "batchmean" else r, log_target=log_target)


def cross_entropy_loss(t, target, reduction=1, ignore_index=-100, label_smoothing=0.0):
    return F.cross_entropy(t, target, reduction=_red(reduction), ignore_index=ignore_index, label_smoothing=label_smoothing)


def ctc_loss(t, targets, input_lengths, target_lengths, blank=0, reduction=1):
    return F.ctc_loss(t, targets, input_lengths, target_lengths, blank, _red(reduction))


# ---- creation and conversion (mod.rs) -----------------------------------------------------------------
def _opts(opts: Optional[TensorOptions]):
    o = opts or TensorOptions()
    return dict(dtype=o.dtype.torch if hasattr(o.dtype, "torch") else o.dtype, device=_dev(o.device))


def empty(shape: Sequence[int], opts: Optional[TensorOptions] = None) -> T:
    return torch.empty(list(shape), **_opts(opts))


def from_f64(data: Sequence[float], shape: Sequence[int], device=None) -> T:
    return torch.tensor(list(data), dtype=torch.float64).reshape(list(shape)).to(_dev(device))


def from_blob(data: bytes, shape: Sequence[int], dtype, device=None) -> T:
    """A tensor from raw little-endian bytes in row-major order (a copy is made: the bytes may go away)."""
    td = dtype.torch if hasattr(dtype, "torch") else dtype
    t = torch.frombuffer(bytearray(data), dtype=td).reshape(list(shape)).clone()
    return t.to(_dev(device))


def to_blob(t: T) -> bytes:
    """The tensor's elements as raw little-endian bytes, row-major (what `.fdl` checkpoints store)."""
    c = t.detach().to("cpu").contiguous()
    return c.view(torch.uint8).numpy().tobytes() if c.numel() else b""


def to_f64_vec(t: T) -> List[float]: return t.detach().to("cpu", torch.float64).reshape(-1).tolist()
def to_i64_vec(t: T) -> List[int]: return t.detach().to("cpu", torch.int64).reshape(-1).tolist()
def to_dtype(t: T, dtype) -> T: return t.to(dtype.torch if hasattr(dtype, "torch") else dtype)
def to_device(t: T, device) -> T: return t.to(_dev(device))
def to_device_async(t: T, device) -> T: return t.to(_dev(device), non_blocking=True)
def to_device_of(t: T, other: T) -> T: return t.to(other.device)
def to_channels_last(t: T) -> T: return t.contiguous(memory_format=torch.channels_last)
def is_channels_last(t: T) -> bool: return t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last) and not t.is_contiguous()


# ---- autograd plumbing on raw tensors (ops_training.cpp:40-170) ---------------------------------------
def set_requires_grad(t: T, requires_grad: bool) -> T: return t.requires_grad_(requires_grad)


def set_grad(t: T, grad: T) -> None:
    t.grad = grad


def zero_grad(t: T) -> None:
    if t.grad is not None:
        t.grad.detach_().zero_()


def zero_grad_set_to_none(t: T) -> None:
    t.grad = None


class GradAccumulatorHandle:
    """Keeps the gradient-accumulator node of a leaf alive. The autograd engine looks that node up
    through a weak pointer; pinning it makes backward passes started from other threads find the
    same node instead of racing to create one (ops_training.cpp:62-77, tensor/mod.rs:1227-1245)."""

    def __init__(self, node):
        self.node = node


def ensure_grad_accumulator(t: T) -> Optional[GradAccumulatorHandle]:
    if not (t.requires_grad and t.is_leaf):
        return None
    return GradAccumulatorHandle(t.view_as(t).grad_fn.next_functions[0][0])


def autograd_node_count(t: T) -> int:
    """Number of distinct autograd nodes reachable from this tensor's `grad_fn` (0 for a leaf)."""
    root = t.grad_fn
    if root is None:
        return 0
    seen, stack = {}, [root]          # the wrappers are kept alive so that their ids stay distinct
    while stack:
        n = stack.pop()
        if n is None or id(n) in seen:
            continue
        seen[id(n)] = n
        stack.extend(f for f, _ in n.next_functions)
    return len(seen)


# ---- optimizer primitives (ops_training.cpp:576-800) --------------------------------------------------
def adam_step(param: T, grad: T, m: T, v: T, lr, beta1, beta2, eps, weight_decay, step: int) -> None:
    """One decomposed Adam(W) update of a single tensor: decoupled decay `p *= 1 - lr wd`, moment
    updates, bias correction by `step` (1-based), `p -= lr/bc1 * m / (sqrt(v/bc2) + eps)`."""
    with torch.no_grad():
        p = param.detach()
        if weight_decay > 0.0:
            p.mul_(1.0 - lr * weight_decay)
        m.mul_(beta1).add_(grad, alpha=1.0 - beta1)
        v.mul_(beta2).addcmul_(grad, grad, value=1.0 - beta2)
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        p.addcdiv_(m, (v / bc2).sqrt_().add_(eps), value=-lr / bc1)


def adam_step_batched(params, grads, ms, vs, lrs: Sequence[float], beta1, beta2, eps, weight_decay, step: int) -> None:
    for p, g, m, v, lr in zip(params, grads, ms, vs, lrs):
        adam_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step)


def _fused(fn, params, grads, exp_avgs, exp_avg_sqs, lr, beta1, beta2, eps, weight_decay, step, grad_scale, found_inf):
    ps = [p.detach() for p in params]
    if not ps:
        return
    steps = [torch.full((), float(step), dtype=torch.float32, device=p.device) for p in ps]
    with torch.no_grad():
        fn(ps, list(grads), list(exp_avgs), list(exp_avg_sqs), [], steps, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay,
           eps=eps, amsgrad=False, maximize=False, grad_scale=grad_scale, found_inf=found_inf)


def fused_adam_(params, grads, exp_avgs, exp_avg_sqs, lr, beta1, beta2, eps, weight_decay, step: int, grad_scale=None, found_inf=None) -> None:
    """Multi-tensor Adam in one call (`_fused_adam_`). `step` is the 1-based count of this update: the
    kernel reads its step tensors as they are (the caller counts), it does not advance them."""
    _fused(torch._fused_adam_, params, grads, exp_avgs, exp_avg_sqs, lr, beta1, beta2, eps, weight_decay, step, grad_scale, found_inf)


def fused_adamw_(params, grads, exp_avgs, exp_avg_sqs, lr, beta1, beta2, eps, weight_decay, step: int, grad_scale=None, found_inf=None) -> None:
    _fused(torch._fused_adamw_, params, grads, exp_avgs, exp_avg_sqs, lr, beta1, beta2, eps, weight_decay, step, grad_scale, found_inf)


def clip_grad_norm_fused(params: Sequence[T], max_norm: float) -> float:
    """Scale the gradients of `params` so that their global L2 norm is at most `max_norm`; returns the
    norm before scaling. Scale factor `max_norm / (norm + 1e-6)`, applied only when below 1
    (ops_training.cpp:769-800)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return 0.0
    total = float(torch.linalg.vector_norm(torch.stack(torch._foreach_norm(grads)), 2))
    coef = max_norm / (total + 1e-6)
    if coef < 1.0:
        torch._foreach_mul_(grads, coef)
    return total
