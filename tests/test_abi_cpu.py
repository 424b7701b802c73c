"""The drop-in C library (`flodl_b200/libflodl_b200_shim.so`, csrc/abi): it exports every function of the
reference's C interface (flodl-sys/shim.h) and a host that drives training through those functions, with the
reference host's call sequence (baseline/reference_arm.py), trains."""
import ctypes
import math
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "flodl_b200", "libflodl_b200_shim.so")
SYMBOLS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "flodl_abi_symbols.txt")

pytestmark = pytest.mark.skipif(not os.path.isfile(SHIM), reason="libflodl_b200_shim.so not built")


def test_exports_every_function_of_the_reference_interface():
    import torch  # noqa: F401  (resolves the library's libtorch imports)
    lib = ctypes.CDLL(SHIM)
    names = [n.strip() for n in open(SYMBOLS) if n.strip()]
    assert len(names) > 300
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"missing exports: {missing}"


_CHILD = r"""
import sys, json
sys.path.insert(0, {root!r})
import numpy as np
from baseline import reference_arm as R
shim = R.Shim({shim!r})
o = R.Ops(shim, R.CPU, 0)
o.manual_seed(7)
guard = o.autocast_new(o.dt, R.BF16)
out = {{}}
for name in ("lm", "bert-base", "resnet20"):
    model, opt, gen, B, desc, pub = R.make_workload(name, o, 4, True)
    rng = np.random.default_rng(3)
    batch = [o.from_numpy(a, dt) for a, dt in gen(rng)]
    losses = []
    for i in range(6):
        loss = model.loss(*batch)
        losses.append(o.item(loss))
        o.backward(loss)
        opt.step(); opt.zero_grad()
    out[name] = losses
o.autocast_del(guard)
print("RESULT " + json.dumps(out))
"""


def test_reference_host_call_sequence_trains_on_the_drop_in_library():
    """Forward, backward and optimizer of three model families through the C interface only
    (a child process: the library and the reference's own shim export the same names)."""
    import json
    res = subprocess.run([sys.executable, "-c", _CHILD.format(root=ROOT, shim=SHIM)], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    for name, losses in out.items():
        assert all(math.isfinite(v) for v in losses), (name, losses)
        assert losses[-1] < losses[0], (name, losses)       # the same batch six times: the loss must fall


def test_error_strings_and_handle_lifecycle():
    import torch  # noqa: F401
    lib = ctypes.CDLL(SHIM)
    VP, PVP = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
    lib.flodl_zeros.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, PVP]
    lib.flodl_zeros.restype = VP
    lib.flodl_matmul.argtypes = [VP, VP, PVP]
    lib.flodl_matmul.restype = VP
    lib.flodl_free_tensor.argtypes = [VP]
    lib.flodl_free_string.argtypes = [VP]
    lib.flodl_numel.argtypes = [VP]
    lib.flodl_numel.restype = ctypes.c_int64
    a, b, c = VP(), VP(), VP()
    assert lib.flodl_zeros((ctypes.c_int64 * 2)(2, 3), 2, 6, 0, 0, ctypes.byref(a)) is None
    assert lib.flodl_zeros((ctypes.c_int64 * 2)(4, 5), 2, 6, 0, 0, ctypes.byref(b)) is None
    assert lib.flodl_numel(a) == 6
    err = lib.flodl_matmul(a, b, ctypes.byref(c))           # shape mismatch -> a message, not an abort
    assert err is not None
    msg = ctypes.string_at(err).decode(errors="replace")
    assert "mat1 and mat2" in msg or "shape" in msg or "size" in msg
    lib.flodl_free_string(err)
    lib.flodl_free_tensor(a)
    lib.flodl_free_tensor(b)
