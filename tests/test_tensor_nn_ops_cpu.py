"""The reference's `Tensor` method names all resolve (as a `torch.Tensor` method, or as a function of
`tensor_ops` / `tensor_nn_ops` / `tensor`), and the functions added for them compute what the names say."""
import math

import pytest
import torch
import torch.nn.functional as F

from flodl_b200 import tensor, tensor_nn_ops as N, tensor_ops as T
from flodl_b200.tensor import TensorError

# every `pub fn` of `impl Tensor` in flodl/src/tensor/{mod,ops,shape,nn_ops}.rs
REFERENCE_TENSOR_METHODS = """
abs acos adam_step adam_step_batched adaptive_avg_pool2d adaptive_max_pool2d add add_ add_scalar add_scalar_ addcdiv addcmul addmm all
all_finite any arange argmax argmin argsort asin atan atan2 autograd_node_count avg_pool1d avg_pool2d backward batch_norm batches bce_loss
bce_with_logits_loss bernoulli bilinear cat cat_many cdist cdist_p ceil chunk clamp clamp_max clamp_min clip_grad_norm_fused col2im
contiguous conv1d conv2d conv3d conv_transpose1d conv_transpose2d conv_transpose3d copy_ cos cosine_similarity count_nonzero
count_nonzero_dim cross_entropy_loss ctc_loss cumprod cumsum detach detach_ device diagonal div div_ div_scalar div_scalar_ dropout dtype
elu embedding embedding_bag empty ensure_grad_accumulator eq_scalar eq_tensor erf erfc exp expand expm1 eye feature_dropout fill_ flatten
flip floor fmod fmod_tensor foreach_add_list_ foreach_add_scalar_ foreach_lerp_scalar_ foreach_mul_scalar_ foreach_norm foreach_sqrt_
foreach_zero_ frac from_blob from_f32 from_f64 from_i64 full full_like fused_adam_ fused_adamw_ gather ge ge_scalar gelu gelu_tanh grad
grid_sample group_norm gru_cell gru_seq gru_seq_cached gt gt_scalar hardsigmoid hardswish im2col index_add index_select instance_norm
interpolate is_channels_last is_contiguous is_leaf is_pinned isclose isinf isnan item kl_div_loss l1_loss le le_scalar leaky_relu lerp
lerp_tensor linear linspace log log10 log1p log2 log_softmax logical_and logical_not logical_or logsumexp lstm_cell lstm_seq
lstm_seq_cached lt lt_scalar masked_fill matmul max max_dim max_pool1d max_pool2d maximum mean mean_dim median median_dim meshgrid min
min_dim minimum mish movedim mse_loss mul mul_ mul_scalar mul_scalar_ multinomial narrow narrow_scatter native_layer_norm nbytes ndim
ne_scalar ne_tensor neg nll_loss nonzero norm norm_p normalize numel one_hot ones ones_like pad pad_mode permute pin_memory pixel_shuffle
pixel_unshuffle pow_scalar prelu prod prod_dim rand rand_like randint randn randn_like randperm reciprocal relu remainder
remainder_tensor repeat requires_grad reshape roll round scaled_dot_product_attention scatter scatter_add searchsorted select
select_scatter selu set_grad set_requires_grad shape sigmoid sign silu sin smooth_l1_loss softmax softplus sort split sqrt squeeze stack
std std_dim sub sub_ sum sum_dim sum_dims tan tanh tile to_blob to_channels_last to_device to_device_async to_device_of to_dtype
to_f32_vec to_f64_vec to_i64_vec topk transpose tril triu trunc unbind unique unsqueeze unsqueeze_many var var_dim where_cond zero_
zero_grad zero_grad_set_to_none zeros zeros_like
""".split()


@pytest.mark.parametrize("name", REFERENCE_TENSOR_METHODS)
def test_reference_tensor_method_name_resolves(name):
    assert hasattr(torch.Tensor, name) or hasattr(T, name) or hasattr(N, name) or hasattr(tensor, name), name


def test_surface_lists_both_modules():
    s = T.surface()
    assert {"gt_scalar", "mul_scalar", "conv2d", "adam_step", "to_blob"} <= set(s) and "RnnParams" not in s


X = torch.arange(12.0).reshape(3, 4) - 5.0


def test_scalar_arithmetic_and_in_place_forms():
    assert torch.equal(N.add_scalar(X, 2.0), X + 2) and torch.equal(N.mul_scalar(X, 3.0), X * 3)
    assert torch.equal(N.div_scalar(X, 2.0), X / 2) and torch.equal(N.pow_scalar(X, 2.0), X ** 2)
    y = X.clone()
    assert N.add_scalar_(y, 1.0) is None and N.mul_scalar_(y, 2.0) is None and N.div_scalar_(y, 4.0) is None
    assert torch.equal(y, (X + 1) * 2 / 4)


def test_dim_reductions_return_values_only():
    assert torch.equal(N.sum_dim(X, 1, True), X.sum(1, True)) and torch.equal(N.mean_dim(X, 0), X.mean(0))
    assert torch.equal(N.max_dim(X, 1), X.max(1).values) and torch.equal(N.min_dim(X, 0, True), X.min(0, True).values)
    assert torch.equal(N.prod_dim(X, 1), X.prod(1))
    torch.testing.assert_close(N.var_dim(X, 1), X.var(1))
    torch.testing.assert_close(N.std_dim(X, 0, True), X.std(0, keepdim=True))
    torch.testing.assert_close(N.norm_p(X, 3.0, 1), X.abs().pow(3).sum(1).pow(1 / 3))
    torch.testing.assert_close(N.normalize(X, 2.0, 1).norm(dim=1), torch.ones(3))
    torch.testing.assert_close(N.cdist_p(X, X, 1.0), torch.cdist(X, X, 1.0))
    torch.testing.assert_close(N.cosine_similarity(X, X + 1, 1, 1e-8), F.cosine_similarity(X, X + 1))


@pytest.mark.parametrize("name,ref", [("gelu", F.gelu), ("silu", F.silu), ("selu", F.selu), ("mish", F.mish), ("hardswish", F.hardswish),
                                      ("hardsigmoid", F.hardsigmoid), ("gelu_tanh", lambda t: F.gelu(t, approximate="tanh"))])
def test_activations(name, ref):
    torch.testing.assert_close(getattr(N, name)(X), ref(X))


def test_parametrised_activations_and_dropout():
    torch.testing.assert_close(N.elu(X, 0.5), F.elu(X, 0.5))
    torch.testing.assert_close(N.leaky_relu(X, 0.2), F.leaky_relu(X, 0.2))
    torch.testing.assert_close(N.softplus(X, 2.0, 10.0), F.softplus(X, 2.0, 10.0))
    assert torch.equal(N.dropout(X, 0.5, False), X) and N.dropout(X, 1.0, True).abs().sum() == 0
    assert torch.equal(N.feature_dropout(X.reshape(1, 3, 4), 0.5, False), X.reshape(1, 3, 4))


def test_shape_helpers():
    assert N.cat(X, X, 0).shape == (6, 4) and N.cat_many([X, X, X], 1).shape == (3, 12) and N.stack([X, X], 0).shape == (2, 3, 4)
    assert torch.equal(N.where_cond(T.gt_scalar(X, 0.0), X, -X), X.abs())
    assert torch.equal(N.pad(X, [1, 0], 9.0)[:, 0], torch.full((3,), 9.0))
    assert N.unsqueeze_many(X, [0, 2]).shape == (1, 3, 1, 4)
    parts = N.batches(torch.arange(10).reshape(10, 1), 4)
    assert [p.shape[0] for p in parts] == [4, 4, 2] and parts[2][0, 0] == 8
    with pytest.raises(TensorError):
        N.batches(X, 0)


def test_raw_convolutions_and_pooling_take_the_shim_argument_order():
    x = torch.randn(2, 3, 8, 8)
    w = torch.randn(4, 3, 3, 3)
    torch.testing.assert_close(N.conv2d(x, w, None, [2, 2], [1, 1], [1, 1], 1), F.conv2d(x, w, None, 2, 1))
    wt = torch.randn(3, 5, 3, 3)
    torch.testing.assert_close(N.conv_transpose2d(x, wt, None, [2, 2], [1, 1], [1, 1], [1, 1], 1), F.conv_transpose2d(x, wt, None, 2, 1, 1))
    x1, w1 = torch.randn(2, 3, 9), torch.randn(4, 3, 3)
    torch.testing.assert_close(N.conv1d(x1, w1, None, 1, 1, 2, 1), F.conv1d(x1, w1, None, 1, 1, 2))
    torch.testing.assert_close(N.conv_transpose1d(x1, torch.randn(3, 2, 3), None, 2, 0, 1, 1, 1).shape, torch.Size([2, 2, 20]))
    x3, w3 = torch.randn(1, 2, 4, 4, 4), torch.randn(3, 2, 3, 3, 3)
    assert N.conv3d(x3, w3, None, [1, 1, 1], [1, 1, 1], [1, 1, 1], 1).shape == (1, 3, 4, 4, 4)
    assert N.conv_transpose3d(x3, torch.randn(2, 3, 2, 2, 2), None, [2, 2, 2], [0, 0, 0], [0, 0, 0], [1, 1, 1], 1).shape == (1, 3, 8, 8, 8)
    assert torch.equal(N.max_pool2d(x, [2, 2], [2, 2], [0, 0], [1, 1], False), F.max_pool2d(x, 2))
    torch.testing.assert_close(N.avg_pool2d(x, [2, 2], [2, 2], [0, 0], False, True), F.avg_pool2d(x, 2))
    assert torch.equal(N.max_pool1d(x1, 3, 3, 0, 1, False), F.max_pool1d(x1, 3))
    torch.testing.assert_close(N.avg_pool1d(x1, 3, 3, 0, False, True), F.avg_pool1d(x1, 3))
    assert N.adaptive_avg_pool2d(x, [1, 1]).shape == (2, 3, 1, 1) and N.adaptive_max_pool2d(x, [2, 2]).shape == (2, 3, 2, 2)
    cols = N.im2col(x, [3, 3], [1, 1], [1, 1], [1, 1])
    assert cols.shape == (2, 27, 64)
    ones = N.col2im(N.im2col(torch.ones(1, 1, 4, 4), [2, 2], [1, 1], [0, 0], [2, 2]), [4, 4], [2, 2], [1, 1], [0, 0], [2, 2])
    assert torch.equal(ones, torch.ones(1, 1, 4, 4))
    assert N.pixel_unshuffle(N.pixel_shuffle(torch.randn(1, 8, 2, 2), 2), 2).shape == (1, 8, 2, 2)
    assert N.bilinear(torch.randn(2, 3), torch.randn(2, 4), torch.randn(5, 3, 4), None).shape == (2, 5)
    grid = F.affine_grid(torch.eye(2, 3).unsqueeze(0).repeat(2, 1, 1), [2, 3, 8, 8], align_corners=False)
    torch.testing.assert_close(N.grid_sample(x, grid, 0, 0, False), x, atol=1e-5, rtol=1e-5)


def test_norms_embedding_attention_and_rnn_cells():
    x = torch.randn(4, 6)
    y, mean, rstd = N.native_layer_norm(x, torch.ones(6), torch.zeros(6), 6, 1e-5)
    torch.testing.assert_close(y, F.layer_norm(x, [6]))
    torch.testing.assert_close(mean.reshape(-1), x.mean(1))
    img = torch.randn(2, 4, 3, 3)
    torch.testing.assert_close(N.group_norm(img, 2, None, None, 1e-5), F.group_norm(img, 2))
    rm, rv = torch.zeros(4), torch.ones(4)
    out = N.batch_norm(img, None, None, rm, rv, True, 0.1, 1e-5)
    assert out.shape == img.shape and rm.abs().sum() > 0
    assert N.instance_norm(img, None, None, None, None, True, 0.1, 1e-5).shape == img.shape
    w = torch.arange(12.0).reshape(4, 3)
    assert torch.equal(N.embedding(w, torch.tensor([[1, 3]]), -1), w[[1, 3]].unsqueeze(0))
    bag = N.embedding_bag(w, torch.tensor([0, 1, 2, 3]), torch.tensor([0, 2]), 0)
    assert torch.equal(bag, torch.stack([w[0] + w[1], w[2] + w[3]]))
    q = torch.randn(1, 2, 5, 8)
    torch.testing.assert_close(N.scaled_dot_product_attention(q, q, q, None, 0.0, True, None), F.scaled_dot_product_attention(q, q, q, is_causal=True))
    gru, lstm = torch.nn.GRUCell(3, 5), torch.nn.LSTMCell(3, 5)
    xi, h, c = torch.randn(2, 3), torch.randn(2, 5), torch.randn(2, 5)
    torch.testing.assert_close(N.gru_cell(xi, h, gru.weight_ih, gru.weight_hh, gru.bias_ih, gru.bias_hh), gru(xi, h))
    h1, c1 = N.lstm_cell(xi, h, c, lstm.weight_ih, lstm.weight_hh, lstm.bias_ih, lstm.bias_hh)
    rh, rc = lstm(xi, (h, c))
    torch.testing.assert_close(h1, rh)
    torch.testing.assert_close(c1, rc)


def test_fused_sequence_rnns_match_the_modules():
    seq = torch.randn(2, 7, 3)
    gru = torch.nn.GRU(3, 5, num_layers=2, batch_first=True)
    h0 = torch.zeros(2, 2, 5)
    out, hn = N.gru_seq(seq, h0, list(gru._flat_weights), 2, True, False)
    ro, rh = gru(seq, h0)
    torch.testing.assert_close(out, ro)
    torch.testing.assert_close(hn, rh)
    out2, _ = N.gru_seq_cached(seq, h0, N.RnnParams.new(gru._flat_weights, 2), 2, True)
    torch.testing.assert_close(out2, ro)
    lstm = torch.nn.LSTM(3, 5, num_layers=1, batch_first=True)
    h0, c0 = torch.zeros(1, 2, 5), torch.zeros(1, 2, 5)
    out, hn, cn = N.lstm_seq(seq, h0, c0, list(lstm._flat_weights), 1, True, False)
    ro, (rh, rc) = lstm(seq, (h0, c0))
    torch.testing.assert_close(out, ro)
    torch.testing.assert_close(cn, rc)
    out3, _, _ = N.lstm_seq_cached(seq, h0, c0, N.RnnParams(lstm._flat_weights, 1), 1, True)
    torch.testing.assert_close(out3, ro)


def test_losses_take_integer_reduction_codes():
    p, t = torch.rand(4, 3), torch.rand(4, 3)
    assert N.mse_loss(p, t, 0).shape == (4, 3)
    torch.testing.assert_close(N.mse_loss(p, t, 1), F.mse_loss(p, t))
    torch.testing.assert_close(N.mse_loss(p, t, 2), F.mse_loss(p, t, reduction="sum"))
    torch.testing.assert_close(N.l1_loss(p, t, 1), F.l1_loss(p, t))
    torch.testing.assert_close(N.smooth_l1_loss(p, t, 1, 0.5), F.smooth_l1_loss(p, t, beta=0.5))
    torch.testing.assert_close(N.bce_loss(p, t, 1), F.binary_cross_entropy(p, t))
    torch.testing.assert_close(N.bce_with_logits_loss(p, t, 2), F.binary_cross_entropy_with_logits(p, t, reduction="sum"))
    torch.testing.assert_close(N.kl_div_loss(p.log(), t, 2, False), F.kl_div(p.log(), t, reduction="sum"))
    y = torch.tensor([0, 2, -100, 1])
    torch.testing.assert_close(N.cross_entropy_loss(p, y, 1, -100, 0.1), F.cross_entropy(p, y, label_smoothing=0.1))
    torch.testing.assert_close(N.nll_loss(p.log_softmax(1), y, 1, -100), F.nll_loss(p.log_softmax(1), y))
    lp = torch.randn(6, 2, 5).log_softmax(2)
    got = N.ctc_loss(lp, torch.tensor([[1, 2], [3, 3]]), torch.tensor([6, 6]), torch.tensor([2, 2]), 0, 1)
    torch.testing.assert_close(got, F.ctc_loss(lp, torch.tensor([[1, 2], [3, 3]]), torch.tensor([6, 6]), torch.tensor([2, 2])))
    with pytest.raises(TensorError):
        N.mse_loss(p, t, 7)


def test_blob_round_trip_and_conversions():
    t = torch.tensor([[1.5, -2.0], [3.25, 4.0]])
    raw = N.to_blob(t)
    assert len(raw) == 16 and torch.equal(N.from_blob(raw, [2, 2], torch.float32), t)
    assert N.to_blob(torch.empty(0)) == b""
    assert torch.equal(N.from_blob(N.to_blob(torch.tensor([1, 2, 3])), [3], tensor.DType.Int64), torch.tensor([1, 2, 3]))
    assert N.to_f64_vec(t) == [1.5, -2.0, 3.25, 4.0] and N.to_i64_vec(torch.tensor([[1, 2]])) == [1, 2]
    assert N.from_f64([1.0, 2.0], [2]).dtype == torch.float64 and N.empty([2, 3]).shape == (2, 3)
    assert N.to_dtype(t, tensor.DType.Float64).dtype == torch.float64 and N.to_dtype(t, torch.float16).dtype == torch.float16
    assert N.to_device(t, None).device.type == "cpu" and N.to_device_of(t, t) is t and N.to_device_async(t, "cpu").device.type == "cpu"
    img = torch.randn(2, 3, 4, 4)
    cl = N.to_channels_last(img)
    assert N.is_channels_last(cl) and not N.is_channels_last(img) and torch.equal(cl, img)


def test_autograd_plumbing_on_raw_tensors():
    w = N.set_requires_grad(torch.randn(3), True)
    assert w.requires_grad and N.autograd_node_count(w) == 0
    y = (w * 2).sin().sum()
    assert N.autograd_node_count(y) == 4                  # sum, sin, mul, accumulate-grad
    h = N.ensure_grad_accumulator(w)
    assert h is not None and "AccumulateGrad" in type(h.node).__name__
    assert N.ensure_grad_accumulator(torch.randn(2)) is None
    y.backward()
    g = w.grad.clone()
    N.zero_grad(w)
    assert w.grad is not None and w.grad.abs().sum() == 0
    N.set_grad(w, g)
    assert torch.equal(w.grad, g)
    N.zero_grad_set_to_none(w)
    assert w.grad is None


def test_adam_primitives_agree_with_each_other_and_with_torch():
    torch.manual_seed(0)
    p0, g = torch.randn(7), torch.randn(7)
    ref = p0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    pa, ma, va = p0.clone(), torch.zeros(7), torch.zeros(7)
    pb, mb, vb = p0.clone(), torch.zeros(7), torch.zeros(7)
    pc, mc, vc = p0.clone(), torch.zeros(7), torch.zeros(7)
    for step in (1, 2, 3):
        ref.grad = g.clone()
        opt.step()
        N.adam_step(pa, g, ma, va, 1e-2, 0.9, 0.999, 1e-8, 0.01, step)
        N.adam_step_batched([pb], [g], [mb], [vb], [1e-2], 0.9, 0.999, 1e-8, 0.01, step)
        N.fused_adamw_([pc], [g], [mc], [vc], 1e-2, 0.9, 0.999, 1e-8, 0.01, step)
    torch.testing.assert_close(pa, ref.detach(), atol=1e-6, rtol=1e-5)
    assert torch.equal(pa, pb)
    torch.testing.assert_close(pc, pa, atol=1e-6, rtol=1e-5)
    pd, md, vd = p0.clone(), torch.zeros(7), torch.zeros(7)
    N.fused_adam_([pd], [g], [md], [vd], 1e-2, 0.9, 0.999, 1e-8, 0.0, 1)
    pe, me, ve = p0.clone(), torch.zeros(7), torch.zeros(7)
    N.adam_step(pe, g, me, ve, 1e-2, 0.9, 0.999, 1e-8, 0.0, 1)
    torch.testing.assert_close(pd, pe, atol=1e-6, rtol=1e-5)
    N.fused_adam_([], [], [], [], 1e-2, 0.9, 0.999, 1e-8, 0.0, 1)          # nothing to do is fine


def test_clip_grad_norm_fused_scales_only_above_the_limit():
    a, b = torch.ones(4, requires_grad=True), torch.ones(9, requires_grad=True)
    a.grad, b.grad = torch.full((4,), 3.0), torch.full((9,), 4.0)
    total = math.sqrt(4 * 9 + 9 * 16)
    assert abs(N.clip_grad_norm_fused([a, b], 1.0) - total) < 1e-4
    assert abs(math.sqrt(float(a.grad.pow(2).sum() + b.grad.pow(2).sum())) - 1.0) < 1e-4
    before = a.grad.clone()
    assert N.clip_grad_norm_fused([a, b], 10.0) < 1.01 and torch.equal(a.grad, before)
    assert N.clip_grad_norm_fused([torch.ones(2)], 1.0) == 0.0
