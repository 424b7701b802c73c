"""More op-level checks of the drop-in C library on CPU: shape and indexing ops, list-returning ops, pooling and the
convolution variants, sorting, creation helpers (flodl-sys/shim.h argument lists)."""
import ctypes as C

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from test_abi_ops_cpu import D, H, I, I64, PVP, SHIM, VP, F32, I64T   # noqa: F401  (shared harness)
import os

pytestmark = pytest.mark.skipif(not os.path.isfile(SHIM), reason="libflodl_b200_shim.so not built")
PI64 = C.POINTER(C.c_int64)


@pytest.fixture(scope="module")
def lib():
    L = C.CDLL(SHIM)
    L.flodl_free_tensor.argtypes = [VP]
    L.flodl_free_string.argtypes = [VP]
    L.flodl_numel.argtypes, L.flodl_numel.restype = [VP], I64
    L.flodl_ndim.argtypes, L.flodl_ndim.restype = [VP], I
    L.flodl_shape.argtypes, L.flodl_shape.restype = [VP, I], I64
    L.flodl_dtype.argtypes, L.flodl_dtype.restype = [VP], I
    return L


@pytest.fixture()
def h(lib):
    return H(lib)


def arr(*v):
    return (C.c_int64 * len(v))(*v)


RNG = np.random.default_rng(1)
X = RNG.standard_normal((2, 3, 4)).astype(np.float32)
TX = torch.from_numpy(X)


def test_shape_ops(h):
    t = h.tensor(X)
    cases = [
        ("permute", [VP, PI64, I], (t, arr(2, 0, 1), 3), TX.permute(2, 0, 1)),
        ("select", [VP, I, I64], (t, 1, 2), TX.select(1, 2)),
        ("narrow", [VP, I, I64, I64], (t, 2, 1, 2), TX.narrow(2, 1, 2)),
        ("unsqueeze", [VP, I], (t, 1), TX.unsqueeze(1)),
        ("flatten", [VP, I, I], (t, 1, 2), TX.flatten(1, 2)),
        ("expand", [VP, PI64, I], (h.out("flodl_unsqueeze", [VP, I], t, 0), arr(5, 2, 3, 4), 4), TX.unsqueeze(0).expand(5, 2, 3, 4)),
        ("repeat", [VP, PI64, I], (t, arr(2, 1, 1), 3), TX.repeat(2, 1, 1)),
        ("tile", [VP, PI64, I], (t, arr(1, 2, 1), 3), TX.tile(1, 2, 1)),
        ("flip", [VP, PI64, I], (t, arr(0, 2), 2), TX.flip(0, 2)),
        ("roll", [VP, I64, I], (t, 1, 2), TX.roll(1, 2)),
        ("movedim", [VP, I64, I64], (t, 0, 2), TX.movedim(0, 2)),
        ("diagonal", [VP, I64, I, I], (t, 0, 1, 2), TX.diagonal(0, 1, 2)),
        ("tril", [VP, I64], (t, 0), TX.tril(0)),
        ("pad", [VP, PI64, I, D], (t, arr(1, 2), 2, 0.5), F.pad(TX, (1, 2), value=0.5)),
    ]
    for name, argt, args, want in cases:
        got = h.numpy(h.out("flodl_contiguous", [VP], h.out("flodl_" + name, argt, *args)))
        np.testing.assert_array_equal(got, want.contiguous().numpy(), err_msg=name)
    sq = h.out("flodl_squeeze", [VP, I], h.out("flodl_unsqueeze", [VP, I], t, 1), 1)
    assert h.numpy(sq).shape == X.shape
    is_c = h.fn("flodl_is_contiguous", [VP], I)
    assert is_c(t) == 1 and is_c(h.out("flodl_transpose", [VP, I, I], t, 0, 2)) == 0


def test_list_ops_cat_stack_chunk_split_unbind(h, lib):
    t = h.tensor(X)
    u = h.tensor(X * 2)
    np.testing.assert_array_equal(h.numpy(h.out("flodl_cat2", [VP, VP, I], t, u, 1)), torch.cat([TX, TX * 2], 1).numpy())
    pair = (VP * 2)(t, u)
    np.testing.assert_array_equal(h.numpy(h.out("flodl_cat", [PVP, I, I], pair, 2, 0)), torch.cat([TX, TX * 2], 0).numpy())
    np.testing.assert_array_equal(h.numpy(h.out("flodl_stack", [PVP, I, I], pair, 2, 1)), torch.stack([TX, TX * 2], 1).numpy())

    def lists(name, argt, *args):
        outp, n = PVP(), C.c_int()
        h.check(h.fn("flodl_" + name, list(argt) + [C.POINTER(PVP), C.POINTER(C.c_int)])(*args, C.byref(outp), C.byref(n)))
        got = [h.numpy(VP(outp[i])) for i in range(n.value)]
        lib.flodl_free_string(C.cast(outp, VP))          # the array itself is malloc'd by the library
        return got
    for got, want in ((lists("chunk", [VP, I, I], t, 2, 2), TX.chunk(2, 2)), (lists("split", [VP, I64, I], t, 3, 2), TX.split(3, 2)),
                      (lists("unbind", [VP, I], t, 1), TX.unbind(1))):
        assert len(got) == len(want)
        for a, b in zip(got, want):
            np.testing.assert_array_equal(a, b.numpy())


def test_indexing_and_scatter_family(h):
    t = h.tensor(X)
    idx = h.tensor(np.array([2, 0], dtype=np.int64))
    np.testing.assert_array_equal(h.numpy(h.out("flodl_index_select", [VP, I, VP], t, 1, idx)), TX.index_select(1, torch.tensor([2, 0])).numpy())
    src = h.tensor(np.ones((2, 2, 4), np.float32))
    np.testing.assert_array_equal(h.numpy(h.out("flodl_index_add", [VP, I, VP, VP], t, 1, idx, src)),
                                  TX.index_add(1, torch.tensor([2, 0]), torch.ones(2, 2, 4)).numpy())
    gi = np.array([[[0, 1, 2, 3]] * 3] * 2, dtype=np.int64)[:, :, ::-1].copy()
    np.testing.assert_array_equal(h.numpy(h.out("flodl_scatter", [VP, I, VP, VP], t, 2, h.tensor(gi), h.tensor(X * 3))),
                                  TX.scatter(2, torch.from_numpy(gi), TX * 3).numpy())
    np.testing.assert_array_equal(h.numpy(h.out("flodl_scatter_add", [VP, I, VP, VP], t, 2, h.tensor(gi), h.tensor(X))),
                                  TX.scatter_add(2, torch.from_numpy(gi), TX).numpy())
    cond = h.tensor((X > 0).astype(np.float32))
    np.testing.assert_array_equal(h.numpy(h.out("flodl_where", [VP, VP, VP], cond, t, h.tensor(-X))), np.abs(X))
    sl = h.tensor(np.full((2, 4), 9.0, np.float32))
    np.testing.assert_array_equal(h.numpy(h.out("flodl_select_scatter", [VP, VP, I, I64], t, sl, 1, 1)), TX.select_scatter(torch.full((2, 4), 9.0), 1, 1).numpy())
    nz = h.numpy(h.out("flodl_nonzero", [VP], h.tensor(np.array([0, 3, 0, 5], np.float32))))
    assert nz.reshape(-1).tolist() == [1, 3]


def test_sorting_and_topk(h):
    v = RNG.standard_normal((3, 7)).astype(np.float32)
    tv = torch.from_numpy(v)
    vals, idx = h.out("flodl_topk", [VP, I64, I, I, I], h.tensor(v), 3, 1, 1, 1, n=2)
    w = tv.topk(3, 1)
    np.testing.assert_array_equal(h.numpy(vals), w.values.numpy())
    np.testing.assert_array_equal(h.numpy(idx), w.indices.numpy())
    vals, idx = h.out("flodl_sort", [VP, I, I], h.tensor(v), 1, 1, n=2)
    w = tv.sort(1, descending=True)
    np.testing.assert_array_equal(h.numpy(vals), w.values.numpy())
    np.testing.assert_array_equal(h.numpy(h.out("flodl_argsort", [VP, I, I], h.tensor(v), 1, 0)), tv.argsort(1).numpy())
    seq = h.tensor(np.array([1.0, 3.0, 5.0], np.float32))
    got = h.numpy(h.out("flodl_searchsorted", [VP, VP], seq, h.tensor(np.array([0.0, 3.5, 9.0], np.float32))))
    assert got.tolist() == [0, 2, 3]


def test_creation_helpers(h):
    np.testing.assert_array_equal(h.numpy(h.out("flodl_eye", [I64, I, I, I], 3, F32, 0, 0)), np.eye(3, dtype=np.float32))
    np.testing.assert_array_equal(h.numpy(h.out("flodl_full", [PI64, I, D, I, I, I], arr(2, 2), 2, 1.5, F32, 0, 0)), np.full((2, 2), 1.5, np.float32))
    perm = h.numpy(h.out("flodl_randperm", [I64, I, I, I], 10, I64T, 0, 0))
    assert sorted(perm.tolist()) == list(range(10))
    ri = h.numpy(h.out("flodl_randint", [I64, I64, PI64, I, I, I, I], 3, 9, arr(50), 1, I64T, 0, 0))
    assert ri.min() >= 3 and ri.max() < 9
    oh = h.numpy(h.out("flodl_one_hot", [VP, I64], h.tensor(np.array([0, 2, 1], dtype=np.int64)), 3))
    np.testing.assert_array_equal(oh, np.eye(3)[[0, 2, 1]])
    t = h.tensor(X)
    assert h.numpy(h.out("flodl_ones_like", [VP], t)).sum() == X.size
    assert np.all(h.numpy(h.out("flodl_full_like", [VP, D], t, 2.0)) == 2.0)
    rn = h.numpy(h.out("flodl_randn_like", [VP], t))
    assert rn.shape == X.shape and np.isfinite(rn).all()
    mn = h.numpy(h.out("flodl_multinomial", [VP, I64, I], h.tensor(np.array([0.0, 1.0, 0.0], np.float32)), 4, 1))
    assert mn.tolist() == [1, 1, 1, 1]


def test_pooling_and_convolution_variants(h):
    x = RNG.standard_normal((2, 3, 8, 8)).astype(np.float32)
    tx = torch.from_numpy(x)
    mp = h.out("flodl_max_pool2d", [VP, PI64, PI64, PI64, PI64, I], h.tensor(x), arr(2, 2), arr(2, 2), arr(0, 0), arr(1, 1), 0)
    np.testing.assert_array_equal(h.numpy(mp), F.max_pool2d(tx, 2).numpy())
    av = h.out("flodl_avg_pool2d", [VP, PI64, PI64, PI64, I, I], h.tensor(x), arr(2, 2), arr(2, 2), arr(0, 0), 0, 1)
    np.testing.assert_allclose(h.numpy(av), F.avg_pool2d(tx, 2).numpy(), rtol=1e-6)
    am = h.out("flodl_adaptive_max_pool2d", [VP, PI64], h.tensor(x), arr(2, 2))
    np.testing.assert_array_equal(h.numpy(am), F.adaptive_max_pool2d(tx, 2).numpy())
    x1 = RNG.standard_normal((2, 3, 16)).astype(np.float32)
    w1 = (RNG.standard_normal((4, 3, 3)) * 0.3).astype(np.float32)
    c1 = h.out("flodl_conv1d", [VP, VP, VP, I64, I64, I64, I64], h.tensor(x1), h.tensor(w1), None, 2, 1, 1, 1)
    np.testing.assert_allclose(h.numpy(c1), F.conv1d(torch.from_numpy(x1), torch.from_numpy(w1), stride=2, padding=1).numpy(), rtol=1e-4, atol=1e-5)
    mp1 = h.out("flodl_max_pool1d", [VP, I64, I64, I64, I64, I], h.tensor(x1), 2, 2, 0, 1, 0)
    np.testing.assert_array_equal(h.numpy(mp1), F.max_pool1d(torch.from_numpy(x1), 2).numpy())
    wt = (RNG.standard_normal((3, 5, 3, 3)) * 0.2).astype(np.float32)
    ct = h.out("flodl_conv_transpose2d", [VP, VP, VP, PI64, PI64, PI64, PI64, I64], h.tensor(x), h.tensor(wt), None, arr(2, 2), arr(1, 1), arr(1, 1), arr(1, 1), 1)
    np.testing.assert_allclose(h.numpy(ct), F.conv_transpose2d(tx, torch.from_numpy(wt), stride=2, padding=1, output_padding=1).numpy(), rtol=1e-4, atol=1e-5)
    gn = h.out("flodl_group_norm", [VP, I64, VP, VP, D], h.tensor(x[:, :2]), 2, None, None, 1e-5)
    np.testing.assert_allclose(h.numpy(gn), F.group_norm(tx[:, :2], 2).numpy(), rtol=1e-4, atol=1e-5)
    ip = h.out("flodl_interpolate", [VP, PI64, I, I, I], h.tensor(x), arr(16, 16), 2, 0, 0)
    np.testing.assert_array_equal(h.numpy(ip), F.interpolate(tx, size=(16, 16), mode="nearest").numpy())
