"""Op-level checks of the drop-in C library (`libflodl_b200_shim.so`) on CPU: each `flodl_*` function is called
through ctypes with the argument list of the reference's C interface (flodl-sys/shim.h) and its result is
compared with the PyTorch op it stands for. Table-driven: one row per function."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "flodl_b200", "libflodl_b200_shim.so")
pytestmark = pytest.mark.skipif(not os.path.isfile(SHIM), reason="libflodl_b200_shim.so not built")

VP, PVP, I, I64, D = C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int64, C.c_double
F32, F64, I32, I64T = 6, 7, 3, 4
_NP = {F32: np.float32, F64: np.float64, I32: np.int32, I64T: np.int64}


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


class H:
    """Owns handles; call(name, argtypes, *args) -> new handle(s); converts to / from numpy."""

    def __init__(self, L):
        self.L, self.keep = L, []

    def fn(self, name, argtypes, restype=VP):
        f = getattr(self.L, name)
        f.argtypes, f.restype = argtypes, restype
        return f

    def check(self, err):
        if err:
            msg = C.string_at(err).decode(errors="replace")
            self.L.flodl_free_string(err)
            raise RuntimeError(msg)

    def tensor(self, a: np.ndarray):
        a = np.ascontiguousarray(a)
        tag = {np.dtype(np.float32): F32, np.dtype(np.float64): F64, np.dtype(np.int32): I32, np.dtype(np.int64): I64T}[a.dtype]
        shape = (C.c_int64 * max(1, a.ndim))(*a.shape)
        out = VP()
        f = self.fn("flodl_from_blob", [VP, C.POINTER(C.c_int64), I, I, I, I, PVP])
        self.check(f(a.ctypes.data_as(VP), shape, a.ndim, tag, 0, 0, C.byref(out)))
        self.keep.append(a)
        return out

    def out(self, name, argtypes, *args, n=1):
        outs = [VP() for _ in range(n)]
        self.check(self.fn(name, list(argtypes) + [PVP] * n)(*args, *[C.byref(o) for o in outs]))
        return outs[0] if n == 1 else outs

    def numpy(self, h) -> np.ndarray:
        L = self.L
        shape = [int(L.flodl_shape(h, d)) for d in range(int(L.flodl_ndim(h)))]
        dt = _NP[int(L.flodl_dtype(h))]
        buf = np.empty(int(L.flodl_numel(h)), dt)
        self.check(self.fn("flodl_copy_data", [VP, VP, I64])(h, buf.ctypes.data_as(VP), buf.nbytes))
        return buf.reshape(shape)


@pytest.fixture()
def h(lib):
    return H(lib)


RNG = np.random.default_rng(0)
A = RNG.standard_normal((3, 5)).astype(np.float32)
B = RNG.standard_normal((3, 5)).astype(np.float32)
POS = (np.abs(A) + 0.5).astype(np.float32)
UNIT = np.clip(A * 0.3, -0.9, 0.9).astype(np.float32)

UNARY = [
    ("neg", torch.neg, A), ("relu", torch.relu, A), ("sigmoid", torch.sigmoid, A), ("tanh_op", torch.tanh, A), ("gelu", torch.nn.functional.gelu, A),
    ("gelu_tanh", lambda t: torch.nn.functional.gelu(t, approximate="tanh"), A), ("silu", torch.nn.functional.silu, A), ("mish", torch.nn.functional.mish, A),
    ("selu", torch.selu, A), ("hardswish", torch.nn.functional.hardswish, A), ("hardsigmoid", torch.nn.functional.hardsigmoid, A),
    ("exp", torch.exp, A), ("log", torch.log, POS), ("sqrt", torch.sqrt, POS), ("abs", torch.abs, A), ("log1p", torch.log1p, POS), ("expm1", torch.expm1, A),
    ("log2", torch.log2, POS), ("log10", torch.log10, POS), ("sin", torch.sin, A), ("cos", torch.cos, A), ("tan", torch.tan, UNIT), ("asin", torch.asin, UNIT),
    ("acos", torch.acos, UNIT), ("atan", torch.atan, A), ("sign", torch.sign, A), ("floor", torch.floor, A), ("ceil", torch.ceil, A), ("round", torch.round, A),
    ("reciprocal", torch.reciprocal, POS), ("erf", torch.erf, A), ("erfc", torch.erfc, A), ("trunc", torch.trunc, A), ("frac", torch.frac, A),
    ("sum", torch.sum, A), ("mean", torch.mean, A), ("prod", torch.prod, UNIT), ("min", torch.min, A), ("max", torch.max, A), ("norm", torch.norm, A),
    ("var", torch.var, A), ("std_op", torch.std, A), ("median", torch.median, A),
]


@pytest.mark.parametrize("name,ref,x", UNARY, ids=[u[0] for u in UNARY])
def test_unary_and_full_reductions(h, name, ref, x):
    got = h.numpy(h.out("flodl_" + name, [VP], h.tensor(x)))
    np.testing.assert_allclose(got, ref(torch.from_numpy(x)).numpy(), rtol=2e-5, atol=2e-6)


BINARY = [("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div), ("atan2", torch.atan2), ("maximum", torch.maximum),
          ("minimum", torch.minimum), ("fmod_tensor", torch.fmod), ("remainder_tensor", torch.remainder)]


@pytest.mark.parametrize("name,ref", BINARY, ids=[b[0] for b in BINARY])
def test_binary(h, name, ref):
    got = h.numpy(h.out("flodl_" + name, [VP, VP], h.tensor(A), h.tensor(POS)))
    np.testing.assert_allclose(got, ref(torch.from_numpy(A), torch.from_numpy(POS)).numpy(), rtol=2e-5, atol=2e-6)


COMPARE = [("gt_tensor", torch.gt), ("lt_tensor", torch.lt), ("ge_tensor", torch.ge), ("le_tensor", torch.le), ("eq_tensor", torch.eq), ("ne_tensor", torch.ne)]


@pytest.mark.parametrize("name,ref", COMPARE, ids=[c[0] for c in COMPARE])
def test_comparisons_return_float_masks(h, name, ref):
    b = A.copy()
    b[0] = B[0]
    got = h.numpy(h.out("flodl_" + name, [VP, VP], h.tensor(A), h.tensor(b)))
    assert got.dtype == np.float32                                  # masks come back as 0.0 / 1.0 in the input's dtype
    np.testing.assert_array_equal(got, ref(torch.from_numpy(A), torch.from_numpy(b)).float().numpy())


SCALAR = [("add_scalar", lambda t, s: t + s), ("mul_scalar", lambda t, s: t * s), ("div_scalar", lambda t, s: t / s), ("pow_scalar", lambda t, s: t.abs().pow(s)),
          ("clamp_min", lambda t, s: t.clamp_min(s)), ("clamp_max", lambda t, s: t.clamp_max(s)), ("leaky_relu", torch.nn.functional.leaky_relu),
          ("elu", torch.nn.functional.elu), ("gt_scalar", lambda t, s: (t > s).float()), ("le_scalar", lambda t, s: (t <= s).float()),
          ("fmod_scalar", torch.fmod), ("remainder_scalar", torch.remainder)]


@pytest.mark.parametrize("name,ref", SCALAR, ids=[s[0] for s in SCALAR])
def test_scalar_ops(h, name, ref):
    x = np.abs(A) if name == "pow_scalar" else A
    got = h.numpy(h.out("flodl_" + name, [VP, D], h.tensor(x), 0.7))
    np.testing.assert_allclose(got, ref(torch.from_numpy(A), 0.7).numpy(), rtol=2e-5, atol=2e-6)


DIMRED = [("sum_dim", lambda t, d, k: t.sum(d, k)), ("mean_dim", lambda t, d, k: t.mean(d, k)), ("prod_dim", lambda t, d, k: t.prod(d, k)),
          ("logsumexp", lambda t, d, k: t.logsumexp(d, k)), ("min_dim", lambda t, d, k: t.min(d, k).values), ("max_dim", lambda t, d, k: t.max(d, k).values),
          ("argmax", lambda t, d, k: t.argmax(d, k)), ("argmin", lambda t, d, k: t.argmin(d, k)), ("var_dim", lambda t, d, k: t.var(d, keepdim=k)),
          ("std_dim", lambda t, d, k: t.std(d, keepdim=k))]


@pytest.mark.parametrize("keep", [0, 1])
@pytest.mark.parametrize("name,ref", DIMRED, ids=[d[0] for d in DIMRED])
def test_dim_reductions(h, name, ref, keep):
    got = h.numpy(h.out("flodl_" + name, [VP, I, I], h.tensor(A), 1, keep))
    want = ref(torch.from_numpy(A), 1, bool(keep)).numpy()
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-6)


def test_median_dim_returns_values_and_indices(h):
    vals, idx = h.out("flodl_median_dim", [VP, I, I], h.tensor(A), 1, 0, n=2)
    want = torch.from_numpy(A).median(1)
    np.testing.assert_array_equal(h.numpy(vals), want.values.numpy())
    np.testing.assert_array_equal(h.numpy(idx), want.indices.numpy())


def test_creation_shape_and_indexing(h):
    shape = (C.c_int64 * 2)(2, 3)
    z = h.out("flodl_zeros", [C.POINTER(C.c_int64), I, I, I, I], shape, 2, F32, 0, 0)
    o = h.out("flodl_ones", [C.POINTER(C.c_int64), I, I, I, I], shape, 2, F64, 0, 0)
    assert h.numpy(z).tolist() == [[0, 0, 0], [0, 0, 0]] and h.numpy(o).dtype == np.float64
    ar = h.out("flodl_arange", [D, D, D, I, I, I], 0.0, 6.0, 1.0, I64T, 0, 0)
    assert h.numpy(ar).tolist() == [0, 1, 2, 3, 4, 5]
    ls = h.out("flodl_linspace", [D, D, I64, I, I, I], 0.0, 1.0, 5, F32, 0, 0)
    np.testing.assert_allclose(h.numpy(ls), np.linspace(0, 1, 5, dtype=np.float32))
    t = h.tensor(A)
    r = h.out("flodl_reshape", [VP, C.POINTER(C.c_int64), I], t, (C.c_int64 * 2)(5, 3), 2)
    np.testing.assert_array_equal(h.numpy(r), A.reshape(5, 3))
    tr = h.out("flodl_transpose", [VP, I, I], t, 0, 1)
    np.testing.assert_array_equal(h.numpy(h.out("flodl_contiguous", [VP], tr)), A.T)
    mm = h.out("flodl_matmul", [VP, VP], t, tr)
    np.testing.assert_allclose(h.numpy(mm), A @ A.T, rtol=1e-5, atol=1e-5)
    idx = h.tensor(np.array([[0, 2], [1, 1], [4, 0]], dtype=np.int64))
    g = h.out("flodl_gather", [VP, I, VP], t, 1, idx)
    np.testing.assert_array_equal(h.numpy(g), np.take_along_axis(A, np.array([[0, 2], [1, 1], [4, 0]]), 1))
    tri = h.out("flodl_triu", [VP, I64], t, 1)
    np.testing.assert_array_equal(h.numpy(tri), np.triu(A, 1))
    cs = h.out("flodl_cumsum", [VP, I], t, 1)
    np.testing.assert_allclose(h.numpy(cs), np.cumsum(A, 1), rtol=1e-5, atol=1e-6)
    sm = h.out("flodl_softmax", [VP, I], t, 1)
    np.testing.assert_allclose(h.numpy(sm), torch.softmax(torch.from_numpy(A), 1).numpy(), rtol=1e-5, atol=1e-6)
    cl = h.out("flodl_clamp", [VP, D, D], t, -0.2, 0.3)
    np.testing.assert_array_equal(h.numpy(cl), np.clip(A, -0.2, 0.3))
    mask = h.tensor((A > 0).astype(np.float32))
    mf = h.out("flodl_masked_fill", [VP, VP, D], t, mask, -1.0)
    np.testing.assert_array_equal(h.numpy(mf), np.where(A > 0, -1.0, A).astype(np.float32))


def test_autograd_linear_losses_and_adam_step(h):
    x = h.tensor(RNG.standard_normal((8, 4)).astype(np.float32))
    w0 = (RNG.standard_normal((3, 4)) * 0.5).astype(np.float32)
    b0 = np.zeros(3, np.float32)
    tgt = h.tensor(np.array([0, 2, 1, 1, 0, 2, 2, 0], dtype=np.int64))
    w = h.out("flodl_set_requires_grad", [VP, I], h.tensor(w0.copy()), 1)
    b = h.out("flodl_set_requires_grad", [VP, I], h.tensor(b0.copy()), 1)
    logits = h.out("flodl_linear", [VP, VP, VP], x, w, b)
    loss = h.out("flodl_cross_entropy_loss", [VP, VP, I64, I64, D], logits, tgt, 1, -100, 0.0)
    h.check(h.fn("flodl_backward", [VP])(loss))
    gw, gb = h.out("flodl_grad", [VP], w), h.out("flodl_grad", [VP], b)
    xt, wt, bt = torch.from_numpy(h.numpy(x)), torch.from_numpy(w0.copy()).requires_grad_(True), torch.from_numpy(b0.copy()).requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(torch.nn.functional.linear(xt, wt, bt), torch.from_numpy(h.numpy(tgt)))
    ref.backward()
    np.testing.assert_allclose(h.numpy(loss), ref.detach().numpy(), rtol=1e-5)
    np.testing.assert_allclose(h.numpy(gw), wt.grad.numpy(), rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(h.numpy(gb), bt.grad.numpy(), rtol=1e-4, atol=1e-6)
    # one AdamW step through the interface against torch.optim.AdamW
    m, v = h.out("flodl_zeros_like", [VP], w), h.out("flodl_zeros_like", [VP], w)
    guard = h.fn("flodl_no_grad_guard_new", [], VP)()
    h.check(h.fn("flodl_adam_step", [VP, VP, VP, VP, D, D, D, D, D, I64])(w, gw, m, v, 1e-2, 0.9, 0.999, 1e-8, 0.01, 1))
    h.fn("flodl_no_grad_guard_delete", [VP], None)(guard)
    opt = torch.optim.AdamW([wt], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    opt.step()
    np.testing.assert_allclose(h.numpy(h.out("flodl_detach", [VP], w)), wt.detach().numpy(), rtol=1e-5, atol=1e-6)
    # mse / l1 / bce-with-logits: reduction 1 = mean
    p, q = h.tensor(A), h.tensor(B)
    for name, ref_fn in (("mse_loss", torch.nn.functional.mse_loss), ("l1_loss", torch.nn.functional.l1_loss)):
        got = h.numpy(h.out("flodl_" + name, [VP, VP, I64], p, q, 1))
        np.testing.assert_allclose(got, ref_fn(torch.from_numpy(A), torch.from_numpy(B)).numpy(), rtol=1e-5)
    got = h.numpy(h.out("flodl_bce_with_logits_loss", [VP, VP, I64], p, h.tensor((B > 0).astype(np.float32)), 1))
    np.testing.assert_allclose(got, torch.nn.functional.binary_cross_entropy_with_logits(torch.from_numpy(A), torch.from_numpy((B > 0).astype(np.float32))).numpy(), rtol=1e-5)


def test_layer_norm_conv_pool_and_embedding(h):
    x = RNG.standard_normal((2, 3, 8, 8)).astype(np.float32)
    wt = (RNG.standard_normal((4, 3, 3, 3)) * 0.2).astype(np.float32)
    two = lambda a, b: (C.c_int64 * 2)(a, b)  # noqa: E731
    y = h.out("flodl_conv2d", [VP, VP, VP, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64), I64],
              h.tensor(x), h.tensor(wt), None, two(1, 1), two(1, 1), two(1, 1), 1)
    np.testing.assert_allclose(h.numpy(y), torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(wt), padding=1).numpy(), rtol=1e-4, atol=1e-5)
    ap = h.out("flodl_adaptive_avg_pool2d", [VP, C.POINTER(C.c_int64)], h.tensor(x), two(1, 1))
    np.testing.assert_allclose(h.numpy(ap), x.mean((2, 3), keepdims=True), rtol=1e-5, atol=1e-6)
    g, b = np.ones(5, np.float32) * 1.5, np.full(5, 0.25, np.float32)
    o, mean, rstd = h.out("flodl_native_layer_norm", [VP, VP, VP, I64, D], h.tensor(A), h.tensor(g), h.tensor(b), 5, 1e-5, n=3)
    np.testing.assert_allclose(h.numpy(o), torch.nn.functional.layer_norm(torch.from_numpy(A), (5,), torch.from_numpy(g), torch.from_numpy(b)).numpy(), rtol=1e-5, atol=1e-5)
    assert h.numpy(mean).shape == (3, 1) and h.numpy(rstd).shape == (3, 1)
    table = RNG.standard_normal((7, 4)).astype(np.float32)
    ids = np.array([[1, 6, 0], [3, 3, 2]], dtype=np.int64)
    e = h.out("flodl_embedding", [VP, VP, I64, I, I], h.tensor(table), h.tensor(ids), -1, 0, 0)
    np.testing.assert_array_equal(h.numpy(e), table[ids])


def test_foreach_clip_and_norm(h):
    a, b = np.full((4,), 3.0, np.float32), np.full((2, 2), 4.0, np.float32)
    pa = h.out("flodl_set_requires_grad", [VP, I], h.tensor(a.copy()), 1)
    pb = h.out("flodl_set_requires_grad", [VP, I], h.tensor(b.copy()), 1)
    # loss = sum(pa^2)/2 + sum(pb^2)/2 -> grads equal the parameters
    sq = lambda t: h.out("flodl_sum", [VP], h.out("flodl_mul", [VP, VP], t, t))  # noqa: E731
    loss = h.out("flodl_mul_scalar", [VP, D], h.out("flodl_add", [VP, VP], sq(pa), sq(pb)), 0.5)
    h.check(h.fn("flodl_backward", [VP])(loss))
    arr = (VP * 2)(pa, pb)
    total = D()
    h.check(h.fn("flodl_clip_grad_norm", [PVP, I, D, C.POINTER(D)])(arr, 2, 1.0, C.byref(total)))
    want = float(np.sqrt((a ** 2).sum() + (b ** 2).sum()))
    assert abs(total.value - want) < 1e-4
    ga, gb = h.numpy(h.out("flodl_grad", [VP], pa)), h.numpy(h.out("flodl_grad", [VP], pb))
    assert abs(float(np.sqrt((ga ** 2).sum() + (gb ** 2).sum())) - 1.0) < 1e-3          # clipped to max_norm
    np.testing.assert_allclose(ga, a / (want + 1e-6), rtol=1e-4)
