"""The drop-in C library on a GPU: the hot ops of a BERT training step (linear, layer norm, GELU, attention,
cross-entropy, dropout) take the sm_100a kernels, and training through them tracks the same host sequence over
the ATen fallbacks (FLODL_B200_NATIVE=0)."""
import json
import math
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "flodl_b200", "libflodl_b200_shim.so")

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.isfile(SHIM), reason="libflodl_b200_shim.so not built")]

_CHILD = r"""
import sys, json, ctypes
sys.path.insert(0, {root!r})
import numpy as np
from baseline import reference_arm as R
shim = R.Shim({shim!r})
o = R.Ops(shim, R.CUDA, 0)
o.set_device(0)
o.manual_seed(7)
guard = o.autocast_new(o.dt, R.BF16) if {autocast} else None
B, S, V = 8, 64, 512
model = R.BertMLM(o, V=V, H=128, L=2, heads=2, I_=256, P=S, p={p})
opt = R.AdamW(o, model.params(), 1e-3, 0.01)
rng = np.random.default_rng(3)
ids = rng.integers(0, V, (B, S), dtype=np.int64)
labels = np.full((B, S), -100, dtype=np.int64)
m = rng.random((B, S)) < 0.3
labels[m] = ids[m]
am = np.ones((B, S), np.int64); am[:, S - 7:] = 0
pos = np.ascontiguousarray(np.broadcast_to(np.arange(S, dtype=np.int64), (B, S)))
batch = [o.to_device(o.from_numpy(a, R.I64)) for a in (ids, pos, np.zeros((B, S), np.int64), am, labels)]
losses = []
for i in range(12):
    loss = model.loss(*batch)
    losses.append(o.item(loss))
    o.backward(loss)
    opt.step(); opt.zero_grad()
calls = shim.fn("flodl_b200_native_calls", [], ctypes.c_longlong)()
print("RESULT " + json.dumps({{"losses": losses, "native_calls": int(calls)}}))
"""


def _run(native: bool, p: float, autocast: bool = True):
    env = dict(os.environ, FLODL_B200_NATIVE="1" if native else "0")
    res = subprocess.run([sys.executable, "-c", _CHILD.format(root=ROOT, shim=SHIM, p=p, autocast=autocast)], capture_output=True, text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_native_bf16_paths_track_fp32_aten():
    """The oracle is the same host sequence over plain fp32 ATen ops (no autocast, natives off)."""
    a, b = _run(True, 0.0), _run(False, 0.0, autocast=False)
    assert a["native_calls"] > 100 and b["native_calls"] == 0
    la, lb = a["losses"], b["losses"]
    assert all(math.isfinite(v) for v in la + lb)
    assert abs(la[0] - lb[0]) <= 2e-2 * abs(lb[0])
    assert la[-1] < 0.8 * la[0] and lb[-1] < 0.8 * lb[0]
    assert abs(la[-1] - lb[-1]) <= 0.1 * abs(lb[0])


def test_aten_fallbacks_under_autocast_still_train():
    b = _run(False, 0.0)
    assert b["native_calls"] == 0
    assert all(math.isfinite(v) for v in b["losses"]) and b["losses"][-1] < b["losses"][0]


def test_native_dropout_trains():
    a = _run(True, 0.1)
    assert all(math.isfinite(v) for v in a["losses"]) and a["losses"][-1] < a["losses"][0]


_GRADS = r"""
import sys, json, ctypes
sys.path.insert(0, {root!r})
import numpy as np
from baseline import reference_arm as R
shim = R.Shim({shim!r})
o = R.Ops(shim, R.CUDA, 0)
o.set_device(0)
guard = o.autocast_new(o.dt, R.BF16) if {autocast} else None
rng = np.random.default_rng(5)
M, K, N = 192, 128, 96
def leaf(a):
    t = o.to_device(o.from_numpy(a.astype(np.float32), R.F32))
    out = ctypes.c_void_p()
    o.check(o._set_rg(t.h, 1, ctypes.byref(out)))
    return R.T(out.value)
x, w, b = leaf(rng.standard_normal((M, K))), leaf(rng.standard_normal((N, K)) * 0.1), leaf(rng.standard_normal((N,)))
g, be = leaf(rng.standard_normal((N,)) * 0.2 + 1.0), leaf(rng.standard_normal((N,)) * 0.1)
c = o.to_device(o.from_numpy(rng.standard_normal((M, N)).astype(np.float32), R.F32))
y = o.linear(x, w, b)
y = o.un("gelu", y)
y = o.layer_norm(y, g, be, N, 1e-5)
loss = o.un("sum", o.bin("mul", o.to_dtype(y, R.F32), c))
o.backward(loss)
def host(t):
    n = 1
    shape = o.s.fn("flodl_shape", [R.VP, R.I], R.I6); nd = o.s.fn("flodl_ndim", [R.VP], R.I)
    for d in range(int(nd(t.h))): n *= int(shape(t.h, d))
    t32 = o.to_dtype(t, R.F32)
    buf = np.empty(n, np.float32)
    o.check(o._copy_data(t32.h, buf.ctypes.data_as(ctypes.c_void_p), n * 4))
    return buf.tolist()
calls = shim.fn("flodl_b200_native_calls", [], ctypes.c_longlong)()
print("RESULT " + json.dumps({{"loss": o.item(loss), "gx": host(o.grad(x)), "gw": host(o.grad(w)), "gb": host(o.grad(b)), "gg": host(o.grad(g)), "gbe": host(o.grad(be)),
                              "native_calls": int(calls)}}))
"""


def test_linear_gelu_layernorm_gradients_match_fp32_aten():
    """Every gradient of a linear -> GELU -> LayerNorm chain (inputs, weight, BIAS, gamma, beta) through the native
    bf16 paths against the same chain on fp32 ATen ops."""
    import numpy as np

    def run(native, autocast):
        env = dict(os.environ, FLODL_B200_NATIVE="1" if native else "0")
        res = subprocess.run([sys.executable, "-c", _GRADS.format(root=ROOT, shim=SHIM, autocast=autocast)], capture_output=True, text=True, timeout=600, env=env)
        assert res.returncode == 0, res.stderr[-3000:]
        return json.loads([l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    a, b = run(True, True), run(False, False)
    assert a["native_calls"] >= 3 and b["native_calls"] == 0
    for key in ("gx", "gw", "gb", "gg", "gbe"):
        x, y = np.array(a[key]), np.array(b[key])
        assert np.isfinite(x).all(), key
        err = np.abs(x - y).max() / max(1e-6, np.abs(y).max())
        assert err < 4e-2, (key, err)
