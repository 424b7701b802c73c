"""The allocation-free gradient-norm entry point, called the way a foreign runtime would call it:
through the exported C symbol with raw device pointers.

Some users of the library cannot ask for device memory where they need the norm (a captured step
without a pool of their own, a thread that must not touch the allocator while a collective is
pending, a host program that only links the C ABI). `fb_grad_norm_noalloc` serves them from a
fixed array inside the library; this test checks that it returns what `fb_grad_norm` returns, twice
in a row (the array is reused between calls), and that oversized requests are refused.
This file is named to be collected last."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from flodl_b200 import _ext
    _ext.require()
    lib = ctypes.CDLL(_ext.lib_path())
    lib.fb_grad_norm.restype = ctypes.c_int
    lib.fb_grad_norm.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_float, ctypes.c_float,
                                 ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.fb_grad_norm_noalloc.restype = ctypes.c_int
    lib.fb_grad_norm_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_float, ctypes.c_void_p,
                                         ctypes.c_int, ctypes.c_void_p]
    lib.fb_grad_norm_parts.restype = ctypes.c_int
    lib.fb_grad_norm_parts.argtypes = [ctypes.c_longlong]
    lib.fb_grad_norm_noalloc_max.restype = ctypes.c_longlong
    return lib


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_grad_norm_matches_allocating_entry_point(dtype):
    lib = _lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    out_ref = torch.zeros(2, device="cuda")
    out_new = torch.zeros(2, device="cuda")
    for call, n in enumerate((1_000_003, 4_194_304)):      # two calls in a row share the internal array
        g = (torch.randn(n, device="cuda") * (call + 1)).to(dtype)
        parts = lib.fb_grad_norm_parts(n)
        partial = torch.empty(parts, device="cuda")
        rc = lib.fb_grad_norm(g.data_ptr(), n, partial.data_ptr(), 1.0, 1.0, out_ref.data_ptr(), int(dtype == torch.bfloat16), stream)
        assert rc == 0
        rc = lib.fb_grad_norm_noalloc(g.data_ptr(), n, 1.0, 1.0, out_new.data_ptr(), int(dtype == torch.bfloat16), stream)
        assert rc == 0
        torch.cuda.synchronize()
        ref = g.double().norm().item()
        assert abs(out_new[0].item() - out_ref[0].item()) <= 1e-5 * ref
        assert abs(out_new[1].item() - out_ref[1].item()) <= 1e-6
        assert abs(out_new[0].item() - ref) / ref < 1e-4


def test_noalloc_grad_norm_rejects_oversize():
    lib = _lib()
    out = torch.zeros(2, device="cuda")
    g = torch.zeros(8, device="cuda")
    assert lib.fb_grad_norm_noalloc(g.data_ptr(), lib.fb_grad_norm_noalloc_max() + 1, 1.0, 1.0, out.data_ptr(), 0, None) == -4
