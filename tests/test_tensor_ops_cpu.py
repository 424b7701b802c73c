"""The reference-named tensor-op surface (`flodl_b200.tensor_ops`) and its `Variable` methods."""
import pytest
import torch

from flodl_b200 import tensor_ops as T
from flodl_b200.autograd import Variable


def test_comparisons_return_float_masks():
    x = torch.tensor([1.0, 2.0, 3.0])
    assert T.gt_scalar(x, 1.5).tolist() == [0.0, 1.0, 1.0]
    assert T.eq_tensor(x, torch.tensor([1.0, 0.0, 3.0])).dtype == torch.float32
    assert T.lt_scalar(torch.tensor([1, 5]), 3).dtype == torch.float32
    assert T.any(torch.zeros(3)).item() == 0.0 and T.all(torch.ones(3)).item() == 1.0
    assert T.logical_not(torch.tensor([0.0, 2.0])).tolist() == [1.0, 0.0]
    assert T.isclose(x, x + 1e-9).tolist() == [1.0, 1.0, 1.0]
    assert T.isnan(torch.tensor([float("nan"), 0.0])).tolist() == [1.0, 0.0]


def test_math_ext_matches_torch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 7, generator=g)
    v, i = T.median_dim(x, 1)
    assert torch.equal(v, x.median(1).values) and torch.equal(i, x.median(1).indices)
    assert torch.equal(T.median(x), x.median())
    assert torch.equal(T.cumprod(x, 0), x.cumprod(0))
    assert torch.equal(T.sum_dims(x, [0, 1]), x.sum())
    assert torch.allclose(T.norm_p_dim(x, 3.0, 1), x.norm(3.0, 1))
    s = torch.sort(torch.randn(20, generator=g)).values
    assert torch.equal(T.searchsorted(s, torch.tensor([0.0, 10.0])), torch.searchsorted(s, torch.tensor([0.0, 10.0])))
    assert torch.equal(T.nonzero(torch.tensor([0, 3, 0, 1])), torch.tensor([[1], [3]]))
    assert T.count_nonzero(torch.tensor([0, 3, 0, 1])).item() == 2
    out, inv = T.unique(torch.tensor([3, 1, 3]), True, True)
    assert out.tolist() == [1, 3] and inv.tolist() == [1, 0, 1]
    a, b, c = torch.randn(3, 4, generator=g), torch.randn(3, 5, generator=g), torch.randn(5, 4, generator=g)
    assert torch.allclose(T.addmm(a, b, c, 0.5, 2.0), 0.5 * a + 2.0 * (b @ c))
    assert torch.allclose(T.cdist(b, b), torch.cdist(b, b))
    assert T.one_hot(torch.tensor([0, 2]), 3).tolist() == [[1.0, 0.0, 0.0], [0.0, 0.0, 1.0]]
    assert sorted(T.randperm(6).tolist()) == list(range(6))
    m = T.meshgrid([torch.arange(2), torch.arange(3)])
    assert m[0].shape == (2, 3) and m[1][0].tolist() == [0, 1, 2]
    idx = torch.tensor([[0, 1], [1, 0]])
    assert torch.equal(T.scatter_add(torch.zeros(2, 2), 0, idx, torch.ones(2, 2)), torch.zeros(2, 2).scatter_add(0, idx, torch.ones(2, 2)))
    assert torch.equal(T.movedim(x, 0, 1), x.t()) and torch.equal(T.flip(x, [1]), x.flip(1))
    assert torch.equal(T.argsort(x, 1, True), x.argsort(1, True))
    assert T.multinomial(torch.tensor([0.0, 1.0]), 3, True).tolist() == [1, 1, 1]
    assert torch.equal(T.narrow_scatter(torch.zeros(4), torch.ones(2), 0, 1), torch.tensor([0.0, 1.0, 1.0, 0.0]))
    assert torch.equal(T.pad_mode(torch.arange(4.0).view(1, 1, 4), [1, 1], 1), torch.nn.functional.pad(torch.arange(4.0).view(1, 1, 4), [1, 1], "reflect"))
    with pytest.raises(Exception):
        T.pad_mode(x, [1, 1], 9)
    assert T.interpolate(torch.ones(1, 1, 2, 2), [4, 4], 1).shape == (1, 1, 4, 4)


def test_variable_methods_are_differentiable():
    x = Variable(torch.tensor([[1.0, 4.0, 2.0], [3.0, 0.5, 6.0]]), requires_grad=True)
    vals, idx = x.median_dim(1)
    vals.sum().backward()
    assert x.grad().tolist() == [[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]] and idx.t.tolist() == [2, 0]
    y = Variable(torch.ones(2, 3), requires_grad=True)
    out = y.scatter_add(1, torch.tensor([[0, 0, 1], [2, 2, 2]]), x.mul_scalar(2.0))
    out.sum().backward()
    assert torch.all(y.grad() == 1)
    z = Variable(torch.randn(3, 4), requires_grad=True)
    z.cumprod(1).sum().backward()
    assert z.grad() is not None and z.flip([0]).t.shape == (3, 4)
    assert isinstance(z.gt_scalar(0.0), Variable) and z.gt_scalar(0.0).t.dtype == torch.float32
    assert isinstance(z.split(2, 1), list) and isinstance(z.split(2, 1)[0], Variable)
    w = Variable(torch.randn(4, 4), requires_grad=True)
    w.addmm(z.transpose(0, 1).matmul(z).mul_scalar(0.0).add(w), w).sum().backward()
    assert w.grad() is not None


def test_surface_lists_the_math_ext_names():
    names = set(T.surface())
    for n in ("median", "searchsorted", "nonzero", "cumprod", "multinomial", "isclose", "addmm", "scatter_add", "movedim", "flip",
              "argsort", "randperm", "one_hot", "meshgrid", "cdist"):
        assert n in names, n
