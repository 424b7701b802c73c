"""The reference arm: the unmodified flodl C++ shim, driven through its own C ABI.

The reference (flodl) is a Rust front-end over a C++ shim (`flodl-sys/shim.cpp`, a unity
translation unit over `ops_*.cpp`) that calls libtorch, cuBLAS/cuDNN and NCCL. Rust is not
available on this image, the shim is: `build_shim()` compiles the reference's own `shim.cpp`,
unpatched, with the flags of `flodl-sys/build.rs:60-99` (C++17, `-DFLODL_BUILD_CUDA=1`, linked
against torch, torch_cpu, c10, torch_cuda, c10_cuda, cudart, dl, nccl) into
`baseline/_ref/libflodl_shim.so`. Every GPU kernel of a reference training step is launched from
that library, so driving it with the call sequence of the Rust host gives the reference's device
work exactly; only the host loop is restated (here in Python over ctypes, which costs more host
time per call than the Rust FFI, never less).

Call sequences restated (reference paths):
  * encoder layer     flodl-hf/src/models/transformer_layer.rs:224-263
  * BERT embeddings   flodl-hf/src/models/bert.rs:317-340, MLM head :405-408, :707-752
  * MLM loss          flodl-hf/src/task_heads.rs:170-184
  * sync DDP step     flodl/src/graph/distributed.rs:405-437 -> flodl/src/distributed/ddp.rs:133-157
                      (one AllReduce(Avg) per parameter after backward, one collective per buffer)
  * AdamW             flodl/src/nn/optim/adam.rs:152-198 (`_fused_adamw_` over all parameters)
  * SGD               flodl/src/nn/optim/sgd.rs:132-172 (per-parameter tensor-op loop)
  * ResNet-20         ddp-bench/src/models/resnet.rs:126-301
  * decoder LM        ddp-bench/src/models/gpt_nano.rs (pre-LN blocks over
                      flodl/src/nn/attention.rs:108-151), scaled to the benchmark configuration
  * async averaging   flodl/src/distributed/ddp_run/worker.rs:515-584 (scratch copy, grouped
                      AllReduce(Avg) of all parameters on a side stream, host stream sync,
                      foreach norms for the divergence) and :604-662 (a loss `item()` every step)

One process drives one GPU; ranks use the shim's per-rank communicators
(`flodl_nccl_get_unique_id` on rank 0, `flodl_nccl_init_rank`, `flodl_nccl_all_reduce_rank`).
The shim has no per-rank broadcast, so the per-step BatchNorm buffer synchronisation of
`ddp.rs:150-157` is issued as one `AllReduce(Avg)` per buffer: the same number of NCCL launches.

Nothing from this repository's package, kernels or engine is imported or loaded here.
"""
from __future__ import annotations

import ctypes as C
import json
import math
import os
from typing import Optional
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
SHIM_SO = os.path.join(REF_DIR, "libflodl_shim.so")

F16, BF16, F32, F64, I32, I64 = 5, 15, 6, 7, 3, 4
CPU, CUDA = 0, 1
SUM, PROD, MAX, MIN, AVG = 0, 1, 2, 3, 4


# ------------------------------------------------------------------------------------------ build
def find_reference_source() -> str | None:
    for root in (os.environ.get("FLODL_REFERENCE_SRC"), "/root/reference", os.path.join(HERE, "..", "..", "reference")):
        if root and os.path.isfile(os.path.join(root, "flodl-sys", "shim.cpp")):
            return os.path.join(root, "flodl-sys")
    return None


def build_shim(force: bool = False) -> str:
    """Compile the reference's unmodified shim into `baseline/_ref/libflodl_shim.so`.

    Returns the path; raises `RuntimeError` with the compiler's message when it cannot be built.
    """
    if os.path.isfile(SHIM_SO) and not force:
        return SHIM_SO
    src = find_reference_source()
    if src is None:
        raise RuntimeError("reference sources (flodl-sys/shim.cpp) not found")
    import torch
    troot = os.path.dirname(torch.__file__)
    site = os.path.dirname(troot)
    nccl_root = os.path.join(site, "nvidia", "nccl")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-w", "-DFLODL_BUILD_CUDA=1",
           f"-I{src}", f"-I{troot}/include", f"-I{troot}/include/torch/csrc/api/include", f"-I{cuda_home}/include"]
    libdirs = [f"{troot}/lib", f"{cuda_home}/lib64"]
    nccl = "-lnccl"
    if os.path.isfile(os.path.join(nccl_root, "lib", "libnccl.so.2")):    # the NCCL torch itself runs on
        cmd.append(f"-I{nccl_root}/include")
        libdirs.append(f"{nccl_root}/lib")
        nccl = "-l:libnccl.so.2"
    cmd += [os.path.join(src, "shim.cpp"), "-o", SHIM_SO]
    for d in libdirs:
        cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
    cmd += ["-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda", "-lcudart", "-ldl", nccl]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference shim failed to compile: " + r.stderr[-400:].replace("\n", " "))
    return SHIM_SO


# --------------------------------------------------------------------------------------- bindings
class T:
    """Owns one `FlodlTensor` handle; frees it when the last Python reference goes (as Rust's Drop does)."""
    __slots__ = ("h",)
    free = None

    def __init__(self, h):
        self.h = h

    def __del__(self):
        if self.h and T.free is not None:
            T.free(self.h)
            self.h = None


class Shim:
    def __init__(self, path: str = SHIM_SO):
        import torch  # noqa: F401  (libtorch, the reference's own substrate, resolves the shim's imports)
        self.L = L = C.CDLL(path, mode=C.RTLD_GLOBAL)
        L.flodl_free_string.argtypes = [C.c_void_p]
        L.flodl_free_string.restype = None
        L.flodl_free_tensor.argtypes = [C.c_void_p]
        L.flodl_free_tensor.restype = None
        T.free = L.flodl_free_tensor
        self._fns = {}

    def fn(self, name, argtypes, restype=C.c_void_p):
        f = self._fns.get(name)
        if f is None:
            f = getattr(self.L, name)
            f.argtypes = argtypes
            f.restype = restype
            self._fns[name] = f
        return f

    def fail(self, err):
        msg = C.string_at(err).decode(errors="replace")
        self.L.flodl_free_string(err)
        raise RuntimeError(msg)


VP, I, I6, D = C.c_void_p, C.c_int, C.c_int64, C.c_double
PVP = C.POINTER(C.c_void_p)


def _arr64(xs):
    return (C.c_int64 * len(xs))(*xs)


def _harr(ts):
    return (C.c_void_p * len(ts))(*[t.h for t in ts])


class Ops:
    """The subset of the shim's ABI that the benchmark models use."""

    def __init__(self, shim: Shim, dev_type: int, dev_index: int):
        s, self.s = shim, shim
        self.dt, self.di = dev_type, dev_index
        f = shim.fn
        self._un = {n: f("flodl_" + n, [VP, PVP]) for n in ("gelu", "relu", "sum", "detach", "contiguous", "pin_memory", "grad",
                                                             "zeros_like", "shallow_clone")}
        self._bin = {n: f("flodl_" + n, [VP, VP, PVP]) for n in ("add", "sub", "mul", "matmul")}
        self._sc = {n: f("flodl_" + n, [VP, D, PVP]) for n in ("mul_scalar", "add_scalar")}
        self._inpl = {n: f("flodl_" + n, [VP, VP]) for n in ("add_", "sub_")}
        self._linear = f("flodl_linear", [VP, VP, VP, PVP])
        self._reshape = f("flodl_reshape", [VP, C.POINTER(C.c_int64), I, PVP])
        self._transpose = f("flodl_transpose", [VP, I, I, PVP])
        self._sdpa = f("flodl_scaled_dot_product_attention", [VP, VP, VP, VP, D, I, D, PVP])
        self._ln = f("flodl_native_layer_norm", [VP, VP, VP, I6, D, PVP, PVP, PVP])
        self._dropout = f("flodl_dropout", [VP, D, I, PVP])
        self._embedding = f("flodl_embedding", [VP, VP, I6, I, I, PVP])
        self._ce = f("flodl_cross_entropy_loss", [VP, VP, I6, I6, D, PVP])
        self._softmax = f("flodl_softmax", [VP, I, PVP])
        self._masked_fill = f("flodl_masked_fill", [VP, VP, D, PVP])
        self._triu = f("flodl_triu", [VP, I6, PVP])
        self._conv2d = f("flodl_conv2d", [VP, VP, VP, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64), I6, PVP])
        self._bn = f("flodl_batch_norm", [VP, VP, VP, VP, VP, I, D, D, PVP])
        self._aap = f("flodl_adaptive_avg_pool2d", [VP, C.POINTER(C.c_int64), PVP])
        self._to_dtype = f("flodl_to_dtype", [VP, I, PVP])
        self._to_dev = f("flodl_to_device_async", [VP, I, I, PVP])
        self._set_rg = f("flodl_set_requires_grad", [VP, I, PVP])
        self._backward = f("flodl_backward", [VP])
        self._zero_none = f("flodl_zero_grad_set_to_none", [VP], None)
        self._mul_scalar_ = f("flodl_mul_scalar_", [VP, D])
        self._copy_ = f("flodl_copy_", [VP, VP, I])
        self._copy_data = f("flodl_copy_data", [VP, VP, I6])
        self._create = {n: f("flodl_" + n, [C.POINTER(C.c_int64), I, I, I, I, PVP]) for n in ("zeros", "ones", "randn")}
        self._from_blob = f("flodl_from_blob", [VP, C.POINTER(C.c_int64), I, I, I, I, PVP])
        self._arange = f("flodl_arange", [D, D, D, I, I, I, PVP])
        self._adamw = f("flodl_fused_adamw_", [PVP, PVP, PVP, PVP, I, D, D, D, D, D, I6, VP, VP])
        self._fe_add_list = f("flodl_foreach_add_list_", [PVP, PVP, I, D])
        self._fe_norm = f("flodl_foreach_norm", [PVP, I, D, PVP])
        self.no_grad_new = f("flodl_no_grad_guard_new", [], VP)
        self.no_grad_del = f("flodl_no_grad_guard_delete", [VP], None)
        self.autocast_new = f("flodl_autocast_guard_new", [I, I], VP)
        self.autocast_del = f("flodl_autocast_guard_delete", [VP], None)
        self.sync = f("flodl_cuda_synchronize", [I], None)
        self.set_device = f("flodl_set_current_device", [I], None)
        self.manual_seed = f("flodl_manual_seed", [C.c_uint64], None)

    # -- helpers
    def _out(self, fn, *args):
        out = C.c_void_p()
        err = fn(*args, C.byref(out))
        if err:
            self.s.fail(err)
        return T(out.value)

    def un(self, name, a):
        return self._out(self._un[name], a.h)

    def bin(self, name, a, b):
        return self._out(self._bin[name], a.h, b.h)

    def add(self, a, b):
        return self._out(self._bin["add"], a.h, b.h)

    def sc(self, name, a, v):
        return self._out(self._sc[name], a.h, v)

    def linear(self, x, w, b=None):
        return self._out(self._linear, x.h, w.h, b.h if b is not None else None)

    def reshape(self, x, shape):
        return self._out(self._reshape, x.h, _arr64(shape), len(shape))

    def transpose(self, x, a, b):
        return self._out(self._transpose, x.h, a, b)

    def sdpa(self, q, k, v, mask, p, causal=0):
        return self._out(self._sdpa, q.h, k.h, v.h, mask.h if mask is not None else None, p, causal, 0.0)

    def layer_norm(self, x, w, b, size, eps):
        o, m, r = C.c_void_p(), C.c_void_p(), C.c_void_p()
        err = self._ln(x.h, w.h, b.h, size, eps, C.byref(o), C.byref(m), C.byref(r))
        if err:
            self.s.fail(err)
        T(m.value), T(r.value)       # the Rust wrapper drops mean and rstd at once (autograd/ops.rs:632-635)
        return T(o.value)

    def dropout(self, x, p, training=True):
        if not training or p == 0.0:
            return x
        return self._out(self._dropout, x.h, p, 1)

    def embedding(self, w, idx, padding_idx=-1):
        return self._out(self._embedding, w.h, idx.h, padding_idx, 0, 0)

    def cross_entropy(self, logits, target):
        return self._out(self._ce, logits.h, target.h, 1, -100, 0.0)

    def softmax(self, x, dim):
        return self._out(self._softmax, x.h, dim)

    def masked_fill(self, x, mask, v):
        return self._out(self._masked_fill, x.h, mask.h, v)

    def triu(self, x, d):
        return self._out(self._triu, x.h, d)

    def conv2d(self, x, w, stride, padding):
        return self._out(self._conv2d, x.h, w.h, None, _arr64([stride, stride]), _arr64([padding, padding]), _arr64([1, 1]), 1)

    def batch_norm(self, x, w, b, rm, rv, training=True):
        return self._out(self._bn, x.h, w.h, b.h, rm.h, rv.h, 1 if training else 0, 0.1, 1e-5)

    def adaptive_avg_pool2d(self, x, size):
        return self._out(self._aap, x.h, _arr64(size))

    def to_dtype(self, x, dt):
        return self._out(self._to_dtype, x.h, dt)

    def to_device(self, x):
        return self._out(self._to_dev, x.h, self.dt, self.di)

    def create(self, kind, shape, dtype=F32, device=True):
        return self._out(self._create[kind], _arr64(shape), len(shape), dtype, self.dt if device else CPU, self.di if device else 0)

    def from_numpy(self, a, dtype, device=False, pin=False):
        t = self._out(self._from_blob, a.ctypes.data, _arr64(a.shape), a.ndim, dtype, self.dt if device else CPU, self.di if device else 0)
        if pin and self.dt == CUDA:
            t = self.un("pin_memory", t)
        return t

    def arange(self, n, dtype=I64):
        return self._out(self._arange, 0.0, float(n), 1.0, dtype, self.dt, self.di)

    def param(self, shape, std=0.02, fill=None):
        if fill is None:
            t = self.sc("mul_scalar", self.create("randn", shape), std)
        else:
            t = self.create("ones" if fill == 1.0 else "zeros", shape)
        return self._out(self._set_rg, t.h, 1)

    def backward(self, loss):
        err = self._backward(loss.h)
        if err:
            self.s.fail(err)

    def grad(self, p):
        return self.un("grad", p)

    def zero_grad_none(self, p):
        self._zero_none(p.h)

    def check(self, err):
        if err:
            self.s.fail(err)

    def item(self, t) -> float:
        """`Tensor::item()`: a device -> host copy of one element."""
        buf = (C.c_float * 2)()
        self.check(self._copy_data(t.h, C.addressof(buf), 8))
        return float(buf[0])

    def item_f64(self, t) -> float:
        buf = (C.c_double * 1)()
        self.check(self._copy_data(t.h, C.addressof(buf), 8))
        return float(buf[0])


# ----------------------------------------------------------------------------------------- models
class Linear:
    def __init__(s, o: Ops, i, n, bias=True, weight=None):
        s.o = o
        s.w = weight if weight is not None else o.param([n, i])
        s.b = o.param([n], fill=0.0) if bias else None

    def __call__(s, x):
        return s.o.linear(x, s.w, s.b)

    def params(s):
        return [s.w] + ([s.b] if s.b is not None else [])


class LayerNorm:
    def __init__(s, o: Ops, n, eps=1e-5):
        s.o, s.n, s.eps = o, n, eps
        s.w, s.b = o.param([n], fill=1.0), o.param([n], fill=0.0)

    def __call__(s, x):
        return s.o.layer_norm(x, s.w, s.b, s.n, s.eps)

    def params(s):
        return [s.w, s.b]


class EncoderLayer:
    """transformer_layer.rs:224-263, post-LN."""

    def __init__(s, o, H, heads, I_, p, eps):
        s.o, s.H, s.heads, s.p = o, H, heads, p
        s.q, s.k, s.v, s.ao = (Linear(o, H, H) for _ in range(4))
        s.ln1 = LayerNorm(o, H, eps)
        s.up, s.down = Linear(o, H, I_), Linear(o, I_, H)
        s.ln2 = LayerNorm(o, H, eps)

    def __call__(s, x, mask, B, S):
        o, hd = s.o, s.H // s.heads
        q = o.transpose(o.reshape(s.q(x), [B, S, s.heads, hd]), 1, 2)
        k = o.transpose(o.reshape(s.k(x), [B, S, s.heads, hd]), 1, 2)
        v = o.transpose(o.reshape(s.v(x), [B, S, s.heads, hd]), 1, 2)
        ctx = o.sdpa(q, k, v, mask, s.p, 0)
        flat = o.reshape(o.transpose(ctx, 1, 2), [B, S, s.H])
        a = o.dropout(s.ao(flat), s.p)
        r1 = s.ln1(o.add(a, x))
        f = o.dropout(s.down(o.un("gelu", s.up(r1))), s.p)
        return s.ln2(o.add(f, r1))

    def params(s):
        return s.q.params() + s.k.params() + s.v.params() + s.ao.params() + s.ln1.params() + s.up.params() + s.down.params() + s.ln2.params()


class BertMLM:
    def __init__(s, o: Ops, V=30522, H=768, L=12, heads=12, I_=3072, P=512, p=0.1, eps=1e-12):
        s.o, s.V, s.p = o, V, p
        s.we, s.pe, s.te = o.param([V, H]), o.param([P, H]), o.param([2, H])
        s.ln = LayerNorm(o, H, eps)
        s.layers = [EncoderLayer(o, H, heads, I_, p, eps) for _ in range(L)]
        s.t_dense, s.t_ln = Linear(o, H, H), LayerNorm(o, H, eps)
        s.decoder = Linear(o, H, V, weight=s.we)          # tied to the word embedding (bert.rs:707-752)

    def params(s):
        ps = [s.we, s.pe, s.te] + s.ln.params()
        for l in s.layers:
            ps += l.params()
        return ps + s.t_dense.params() + s.t_ln.params() + [s.decoder.b]

    def buffers(s):
        return []

    def loss(s, ids, pos, tt, am, labels):
        o = s.o
        B, S = ids_shape(o, ids)
        # build_extended_attention_mask (bert.rs:42-48)
        m = o.reshape(o.sc("mul_scalar", o.sc("add_scalar", o.sc("mul_scalar", o.to_dtype(am, F32), -1.0), 1.0), -1e4), [B, 1, 1, S])
        x = o.add(o.add(o.embedding(s.we, ids, 0), o.embedding(s.pe, pos)), o.embedding(s.te, tt))
        x = o.dropout(s.ln(x), s.p)
        for l in s.layers:
            x = l(x, m, B, S)
        x = s.t_ln(o.un("gelu", s.t_dense(x)))
        logits = s.decoder(x)
        return o.cross_entropy(o.reshape(logits, [-1, s.V]), o.reshape(labels, [-1]))


_shape = None


def ids_shape(o: Ops, t):
    global _shape
    if _shape is None:
        _shape = o.s.fn("flodl_shape", [VP, I], I6)
    return int(_shape(t.h, 0)), int(_shape(t.h, 1))


class DecoderBlock:
    """gpt_nano.rs TransformerBlock over nn/attention.rs:108-151 (unfused attention)."""

    def __init__(s, o, Dm, heads, Dff, p):
        s.o, s.D, s.heads, s.p = o, Dm, heads, p
        s.ln1 = LayerNorm(o, Dm)
        s.q, s.k, s.v, s.out = (Linear(o, Dm, Dm) for _ in range(4))
        s.ln2 = LayerNorm(o, Dm)
        s.up, s.down = Linear(o, Dm, Dff), Linear(o, Dff, Dm)

    def __call__(s, x, mask, B, S):
        o, hd = s.o, s.D // s.heads
        n = s.ln1(x)
        q = o.transpose(o.reshape(s.q(n), [B, S, s.heads, hd]), 1, 2)
        k = o.transpose(o.reshape(s.k(n), [B, S, s.heads, hd]), 1, 2)
        v = o.transpose(o.reshape(s.v(n), [B, S, s.heads, hd]), 1, 2)
        scores = o.sc("mul_scalar", o.bin("matmul", q, o.transpose(k, 2, 3)), 1.0 / math.sqrt(hd))
        scores = o.masked_fill(scores, mask, float("-inf"))
        out = o.bin("matmul", o.softmax(scores, -1), v)
        a = s.out(o.reshape(o.transpose(out, 1, 2), [B, S, s.D]))
        x = o.add(x, o.dropout(a, s.p))
        n = s.ln2(x)
        f = o.dropout(s.down(o.un("gelu", s.up(n))), s.p)
        return o.add(x, f)

    def params(s):
        ps = s.ln1.params()
        for l in (s.q, s.k, s.v, s.out):
            ps += l.params()
        return ps + s.ln2.params() + s.up.params() + s.down.params()


class DecoderLM:
    def __init__(s, o: Ops, V=32000, Dm=512, L=6, heads=8, Dff=2048, S=256, p=0.0):
        s.o, s.V, s.S, s.p = o, V, S, p
        s.tok, s.pos = o.param([V, Dm]), o.param([S, Dm])
        s.blocks = [DecoderBlock(o, Dm, heads, Dff, p) for _ in range(L)]
        s.ln_f = LayerNorm(o, Dm)
        s.head = Linear(o, Dm, V)

    def params(s):
        ps = [s.tok, s.pos]
        for b in s.blocks:
            ps += b.params()
        return ps + s.ln_f.params() + s.head.params()

    def buffers(s):
        return []

    def loss(s, x, y):
        o = s.o
        B, S = ids_shape(o, x)
        tok = o.embedding(s.tok, x)
        pos = o.embedding(s.pos, o.arange(S))
        h = o.dropout(o.add(tok, pos), s.p)
        mask = o.triu(o.create("ones", [S, S]), 1)
        for b in s.blocks:
            h = b(h, mask, B, S)
        logits = s.head(s.ln_f(h))
        return o.cross_entropy(o.reshape(logits, [-1, s.V]), o.reshape(y, [-1]))


class BasicBlock:
    def __init__(s, o, cin, cout, stride):
        s.o, s.stride = o, stride
        s.c1, s.c2 = o.param([cout, cin, 3, 3], std=0.1), o.param([cout, cout, 3, 3], std=0.1)
        s.bn1, s.bn2 = BatchNorm(o, cout), BatchNorm(o, cout)
        s.dc = s.dbn = None
        if stride != 1 or cin != cout:
            s.dc, s.dbn = o.param([cout, cin, 1, 1], std=0.1), BatchNorm(o, cout)

    def __call__(s, x):
        o = s.o
        ident = s.dbn(o.conv2d(x, s.dc, s.stride, 0)) if s.dc is not None else x
        out = o.un("relu", s.bn1(o.conv2d(x, s.c1, s.stride, 1)))
        out = s.bn2(o.conv2d(out, s.c2, 1, 1))
        return o.un("relu", o.add(out, ident))

    def params(s):
        ps = [s.c1] + s.bn1.params() + [s.c2] + s.bn2.params()
        if s.dc is not None:
            ps += [s.dc] + s.dbn.params()
        return ps

    def buffers(s):
        return s.bn1.buffers() + s.bn2.buffers() + (s.dbn.buffers() if s.dbn is not None else [])


class BatchNorm:
    def __init__(s, o, c):
        s.o = o
        s.w, s.b = o.param([c], fill=1.0), o.param([c], fill=0.0)
        s.rm, s.rv = o.create("zeros", [c]), o.create("ones", [c])

    def __call__(s, x):
        return s.o.batch_norm(x, s.w, s.b, s.rm, s.rv, True)

    def params(s):
        return [s.w, s.b]

    def buffers(s):
        return [s.rm, s.rv]


class ResNet20:
    """resnet.rs:216-301."""

    def __init__(s, o: Ops):
        s.o = o
        s.c1, s.bn1 = o.param([16, 3, 3, 3], std=0.1), BatchNorm(o, 16)
        s.blocks = []
        for cin, cout, stride in ((16, 16, 1), (16, 32, 2), (32, 64, 2)):
            s.blocks.append(BasicBlock(o, cin, cout, stride))
            s.blocks += [BasicBlock(o, cout, cout, 1) for _ in range(2)]
        s.fc = Linear(o, 64, 10)

    def params(s):
        ps = [s.c1] + s.bn1.params()
        for b in s.blocks:
            ps += b.params()
        return ps + s.fc.params()

    def buffers(s):
        bs = s.bn1.buffers()
        for b in s.blocks:
            bs += b.buffers()
        return bs

    def loss(s, x, y):
        o = s.o
        h = o.un("relu", s.bn1(o.conv2d(x, s.c1, 1, 1)))
        for b in s.blocks:
            h = b(h)
        h = o.adaptive_avg_pool2d(h, [1, 1])
        B = int(ids_shape(o, h)[0])
        return o.cross_entropy(s.fc(o.reshape(h, [B, -1])), y)


# ------------------------------------------------------------------------------------- optimizers
class AdamW:
    """adam.rs:152-198: moments created on first use, one `_fused_adamw_` over every parameter."""

    def __init__(s, o: Ops, params, lr, wd):
        s.o, s.params, s.lr, s.wd, s.t = o, params, lr, wd, 0
        s.m = [None] * len(params)
        s.v = [None] * len(params)

    def step(s):
        o = s.o
        s.t += 1
        g = o.no_grad_new()
        try:
            ps, gs, ms, vs = [], [], [], []
            for i, p in enumerate(s.params):
                gr = o.grad(p)
                if not gr.h:
                    continue
                if s.m[i] is None:
                    s.m[i], s.v[i] = o.un("zeros_like", gr), o.un("zeros_like", gr)
                ps.append(p); gs.append(gr); ms.append(s.m[i]); vs.append(s.v[i])
            o.check(o._adamw(_harr(ps), _harr(gs), _harr(ms), _harr(vs), len(ps), s.lr, 0.9, 0.999, 1e-8, s.wd, s.t, None, None))
        finally:
            o.no_grad_del(g)

    def zero_grad(s):
        for p in s.params:
            s.o.zero_grad_none(p)


class SGD:
    """sgd.rs:132-172: a tensor-op loop per parameter (weight decay, momentum, update)."""

    def __init__(s, o: Ops, params, lr, momentum, wd):
        s.o, s.params, s.lr, s.mom, s.wd = o, params, lr, momentum, wd
        s.vel = [None] * len(params)

    def step(s):
        o = s.o
        g = o.no_grad_new()
        try:
            for i, p in enumerate(s.params):
                gr = o.grad(p)
                if not gr.h:
                    continue
                data = o.un("detach", p)
                if s.wd > 0.0:
                    gr = o.add(gr, o.sc("mul_scalar", data, s.wd))
                if s.vel[i] is not None:
                    v = s.vel[i]
                    o.check(o._mul_scalar_(v.h, s.mom))
                    o.check(o._inpl["add_"](v.h, gr.h))
                else:
                    v = o.sc("mul_scalar", gr, 1.0)
                scaled = o.sc("mul_scalar", v, s.lr)
                o.check(o._inpl["sub_"](data.h, scaled.h))
                s.vel[i] = v
        finally:
            o.no_grad_del(g)

    def zero_grad(s):
        for p in s.params:
            s.o.zero_grad_none(p)


# ------------------------------------------------------------------------------------------ comms
class RankComm:
    def __init__(s, o: Ops, rank, world):
        s.o, s.rank, s.world = o, rank, world
        f = o.s.fn
        s._uid = f("flodl_nccl_get_unique_id", [VP])
        s._init = f("flodl_nccl_init_rank", [I, I, VP, PVP])
        s._ar = f("flodl_nccl_all_reduce_rank", [VP, PVP, I, VP, I])
        s._destroy = f("flodl_nccl_destroy_rank", [VP], None)
        from torch.distributed import TCPStore
        addr, port = os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ["MASTER_PORT"])
        agent = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True"
        store = TCPStore(addr, port, world, is_master=(rank == 0 and not agent), wait_for_workers=False)
        key = "flodl_reference_arm/nccl_uid"
        if rank == 0:
            buf = (C.c_char * 128)()
            o.check(s._uid(C.addressof(buf)))
            store.set(key, bytes(buf))
        uid = store.get(key)
        h = C.c_void_p()
        o.check(s._init(rank, world, uid, C.byref(h)))
        s.h = h.value
        s.store = store

    def all_reduce(s, tensors, op=AVG, stream=None):
        s.o.check(s._ar(s.h, _harr(tensors), len(tensors), stream, op))

    def close(s):
        if s.h:
            s._destroy(s.h)
            s.h = None


# ------------------------------------------------------------------------------------------- data
def make_workload(name, o: Ops, batch, tiny=False):
    """`tiny` shrinks every model to a few layers of width 32 (CPU self-test only; the JSON line says so)."""
    import numpy as np
    if name == "bert-base":
        B, S, V = (batch or 32), 128, 30522
        if tiny:
            S, V = 16, 64
        model = BertMLM(o, V=V, H=32, L=2, heads=2, I_=64, P=S) if tiny else BertMLM(o)

        def gen(rng):
            ids = rng.integers(0, V, (B, S), dtype=np.int64)
            labels = np.full((B, S), -100, dtype=np.int64)
            m = rng.random((B, S)) < 0.15
            labels[m] = ids[m]
            ids[m] = min(103, V - 1)
            pos = np.ascontiguousarray(np.broadcast_to(np.arange(S, dtype=np.int64), (B, S)))
            return [(ids, I64), (pos, I64), (np.zeros((B, S), np.int64), I64), (np.ones((B, S), np.int64), I64), (labels, I64)]
        opt = AdamW(o, model.params(), 1e-4, 0.01)
        desc = {"model": "bert-base-mlm (12x768, 12 heads, ffn 3072, vocab 30522)", "seq_len": S, "optimizer": "AdamW lr 1e-4 wd 0.01", "dropout": 0.1}
        return model, opt, gen, B, desc, None
    if name == "lm":
        B, S, V = (batch or 32), 256, 32000
        if tiny:
            S, V = 16, 64
        model = DecoderLM(o, V=V, Dm=32, L=2, heads=2, Dff=64, S=S) if tiny else DecoderLM(o)

        def gen(rng):
            ids = rng.integers(0, V, (B, S + 1), dtype=np.int64)
            return [(np.ascontiguousarray(ids[:, :-1]), I64), (np.ascontiguousarray(ids[:, 1:]), I64)]
        opt = AdamW(o, model.params(), 3e-4, 0.01)
        desc = {"model": "decoder-lm (6x512, 8 heads, ffn 2048, vocab 32000, pre-LN, GELU)", "seq_len": S, "optimizer": "AdamW lr 3e-4"}
        return model, opt, gen, B, desc, None
    B = batch or 128
    model = ResNet20(o)

    def gen(rng):
        return [(rng.standard_normal((B, 3, 32, 32), dtype=np.float32), F32), (rng.integers(0, 10, (B,), dtype=np.int64), I64)]
    opt = SGD(o, model.params(), 0.1, 0.9, 1e-4)
    desc = {"model": "resnet20-cifar (3 stages x 3 BasicBlocks, 16/32/64 ch, BatchNorm)", "seq_len": None, "optimizer": "SGD lr 0.1 m 0.9 wd 1e-4"}
    return model, opt, gen, B, desc, 3340.0


AVG_EVERY = 8


def unavailable(reason: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}), flush=True)


def run(args, clock_sampler_cls=None, device: str = "cuda", shim_path: Optional[str] = None):
    """Run K timed steps of the reference's training step and print the JSON line (rank 0).
    `shim_path` (a library exporting the same `flodl_*` C interface) replaces the reference's own shim:
    the same host call sequence then measures that library; the line is tagged `"impl": "abi"`."""
    import numpy as np
    if shim_path is None:
        try:
            path = build_shim()
        except Exception as e:  # noqa: BLE001
            return unavailable(f"{type(e).__name__}: {str(e)[:200]}")
    else:
        path = shim_path
    shim = Shim(path)
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = device == "cuda"
    if cuda and not shim.fn("flodl_cuda_is_available", [], I)():
        return unavailable("no CUDA device visible to the reference shim")
    o = Ops(shim, CUDA if cuda else CPU, local if cuda else 0)
    if cuda:
        o.set_device(local)
    o.manual_seed(1234)
    comm = RankComm(o, rank, world) if world > 1 else None
    guard = o.autocast_new(o.dt, BF16)
    tiny = bool(getattr(args, "tiny", False))
    model, opt, gen, B, desc, published = make_workload(args.model, o, args.batch, tiny)
    if tiny:
        desc = dict(desc, tiny=True)
    params, buffers = model.params(), model.buffers()
    local_sgd = args.model == "lm" and world > 1
    per_step_item = args.model == "lm"          # the async worker reads the loss on the host every step, at any world size

    if comm is not None:                       # start-up: replicas begin from rank 0's weights
        g = o.no_grad_new()
        for p in params + buffers:
            d = o.un("detach", p)
            if rank != 0:
                o.check(o._mul_scalar_(d.h, 0.0))
            comm.all_reduce([d], SUM)
        o.no_grad_del(g)

    rng = np.random.default_rng(100 + rank)
    host_pool = [[o.from_numpy(a, dt, pin=True) for a, dt in gen(rng)] for _ in range(8)]
    dev_pool = [[o.to_device(t) for t in b] for b in host_pool]
    h2d = sum(a.nbytes for a, _ in gen(np.random.default_rng(0)))

    # async-DDP state (worker.rs:515-584): a scratch copy of every parameter and a side stream
    scratch = comm_stream = None
    if local_sgd:
        g = o.no_grad_new()
        scratch = [o.un("zeros_like", o.un("detach", p)) for p in params]
        o.no_grad_del(g)
        sp = C.c_void_p()
        o.check(shim.fn("flodl_cuda_stream_new", [I, I, PVP])(local, 0, C.byref(sp)))
        comm_stream = sp.value
    st_set = shim.fn("flodl_cuda_stream_set_current", [VP], None)
    st_restore = shim.fn("flodl_cuda_stream_restore_default", [I], None)
    st_sync = shim.fn("flodl_cuda_stream_synchronize", [VP])
    st_wait = shim.fn("flodl_cuda_stream_wait_event", [VP, VP])
    st_cur = shim.fn("flodl_cuda_stream_get_current", [I], VP)
    ev_new = shim.fn("flodl_cuda_event_new", [I, PVP])
    ev_rec = shim.fn("flodl_cuda_event_record", [VP])
    ev_rec_on = shim.fn("flodl_cuda_event_record_on_stream", [VP, VP])
    ev_sync = shim.fn("flodl_cuda_event_synchronize", [VP])
    ev_ms = shim.fn("flodl_cuda_event_elapsed_time", [VP, VP, C.POINTER(C.c_float)])

    def new_event():
        e = C.c_void_p()
        o.check(ev_new(0, C.byref(e)))
        return e.value

    avg_ready = new_event() if local_sgd else None

    def average_params():
        g = o.no_grad_new()
        try:
            pt = [o.un("detach", p) for p in params]
            # the side stream must see the optimizer's writes before it snapshots the parameters
            o.check(ev_rec(avg_ready))
            o.check(st_wait(comm_stream, avg_ready))
            st_set(comm_stream)
            for d, s_ in zip(scratch, pt):
                o.check(o._copy_(d.h, s_.h, 1))
            st_restore(local)
            comm.all_reduce(pt, AVG, comm_stream)
            o.check(st_sync(comm_stream))
            o.check(o._fe_add_list(_harr(scratch), _harr(pt), len(pt), -1.0))
            outs = (C.c_void_p * len(pt))()
            o.check(o._fe_norm(_harr(scratch), len(pt), 2.0, outs))
            dn = [T(h) for h in outs]
            outs2 = (C.c_void_p * len(pt))()
            o.check(o._fe_norm(_harr(pt), len(pt), 2.0, outs2))
            pn = [T(h) for h in outs2]
            dsq = sum(o.item(t) ** 2 for t in dn)
            psq = sum(o.item(t) ** 2 for t in pn)
            return math.sqrt(dsq) / math.sqrt(psq) if psq > 1e-20 else 0.0
        finally:
            o.no_grad_del(g)

    done = [0]

    def step(inputs):
        loss = model.loss(*inputs)
        val = None
        if per_step_item:
            val = o.item(loss)                                  # worker.rs:628: loss.data().item() every step
        o.backward(loss)
        if comm is not None and not local_sgd:
            for p in params:                                    # ddp.rs:133-147: one AllReduce(Avg) per parameter
                g_ = o.grad(p)
                if g_.h:
                    comm.all_reduce([g_], AVG)
            for b in buffers:                                   # ddp.rs:150-157: one collective per buffer
                comm.all_reduce([b], AVG)
        opt.step()
        opt.zero_grad()
        done[0] += 1
        if local_sgd and done[0] % AVG_EVERY == 0:
            average_params()
        return loss if val is None else val

    def sync_all():
        if comm is not None:
            t = o.create("zeros", [1])
            comm.all_reduce([t], SUM)
        if cuda:
            o.sync(local)

    def gmax(x: float) -> float:
        if comm is None:
            return x
        import numpy as np_
        t = o.from_numpy(np_.array([x], dtype=np_.float64), F64, device=True)
        comm.all_reduce([t], MAX)
        return o.item_f64(t)

    for i in range(max(args.warmup, 3)):
        step(dev_pool[i % 8])
    sync_all()

    sampler = clock_sampler_cls(local) if (clock_sampler_cls and cuda) else None
    if sampler:
        sampler.start()
    if cuda:
        e0, e1 = new_event(), new_event()
        sync_all()
        o.check(ev_rec(e0))
        for i in range(args.steps):
            step(dev_pool[i % 8])
        o.check(ev_rec(e1))
        sync_all()
        ms = C.c_float()
        o.check(ev_ms(e0, e1, C.byref(ms)))
        ms_dev = gmax(float(ms.value)) / args.steps
    else:
        t0 = time.perf_counter()
        for i in range(args.steps):
            step(dev_pool[i % 8])
        ms_dev = (time.perf_counter() - t0) * 1e3 / args.steps

    sync_all()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        inputs = [o.to_device(t) for t in host_pool[i % 8]]       # pinned host -> device, every step
        loss = step(inputs)
        last = loss if isinstance(loss, float) else o.item(loss)   # device -> host read of the loss
    sync_all()
    ms_e2e = gmax((time.perf_counter() - t0) * 1e3) / args.steps
    clocks = sampler.stop() if sampler else None

    if rank == 0:
        value = world * B / (ms_dev / 1e3)
        out = {
            "metric": "DDP samples/sec (max over ranks)", "value": round(value, 2), "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_dev, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (round(value / published, 3) if published else None), "dtype": "bf16",
            "data": "synthetic (random token ids / images of the named shape, random-init weights)", "impl": "reference",
            "config": dict(desc, global_batch=world * B, per_gpu_batch=B, parallelism=f"dp{world}", step="eager (libtorch ops through the reference's C++ shim)",
                           grad_sync=("none" if world == 1 else f"NCCL AllReduce(Avg) of all parameters every {AVG_EVERY} steps" if local_sgd
                                      else "NCCL AllReduce(Avg) per parameter after backward"),
                           l2="working set (weights + optimizer state + activations, > 1 GB) exceeds the 126 MB L2; no flush needed",
                           autocast="bf16 (flodl_autocast_guard)", device=device),
            "clocks": clocks,
            "e2e": {"value": round(world * B / (ms_e2e / 1e3), 2), "unit": "samples/s", "ms_per_step": round(ms_e2e, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "final_loss": round(last, 4),
            "reference_build": "flodl-sys/shim.cpp compiled unmodified (g++ -std=c++17 -DFLODL_BUILD_CUDA=1) into baseline/_ref/libflodl_shim.so; "
                               "host loop restated over the C ABI",
        }
        if shim_path is not None:
            calls = shim.fn("flodl_b200_native_calls", [], C.c_longlong)()
            out.update(impl="abi", native_calls=int(calls), reference_build=None, shim=os.path.basename(shim_path))
            out["config"]["step"] = "eager (the reference host's call sequence over this repository's drop-in flodl_* C library)"
        print(json.dumps(out), flush=True)
    o.autocast_del(guard)
    if comm is not None:
        sync_all()
        comm.close()
