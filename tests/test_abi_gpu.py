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
