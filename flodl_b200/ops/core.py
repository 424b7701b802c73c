"""Autograd functions over the native kernels (see the package docstring for the dispatch rule)."""
from __future__ import annotations

import math
import os
import threading
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _ext

BF16 = torch.bfloat16


class _Flags(threading.local):
    def __init__(self):
        self.native = True          # use the sm_100a kernels when the inputs allow it
        self.autocast = None        # torch dtype while an AutocastGuard is active
        self.count_launches = False
        self.launches = 0


FLAGS = _Flags()

# Called with the parameter tensor each time one of the ops below has written (or accumulated) its
# gradient straight into the flat gradient buffer. Process-wide on purpose: autograd runs backward
# on its own thread. The gradient-sync manager uses it to launch a bucket's all-reduce as soon as
# the bucket is complete.
GRAD_HOOK = {"fn": None}


def _touched(p) -> None:
    fn = GRAD_HOOK["fn"]
    if fn is not None and p is not None:
        fn(p)


def set_native(enabled: bool) -> None:
    """Switch the native kernels off (PyTorch ops only) or back on; used by A/B tests."""
    FLAGS.native = bool(enabled)


def native_enabled() -> bool:
    return FLAGS.native


def _C():
    return _ext.require()


def _launched(n: int = 1) -> None:
    if FLAGS.count_launches:
        FLAGS.launches += n


# ------------------------------------------------------------------------------- zeroed scratch
# Kernels that accumulate with atomics (the convolution's BatchNorm sums) need zeroed fp32 scratch.
# One `torch.zeros` chunk serves many requests, so a step pays for one fill instead of one per layer.
# A slice is handed out once and never again. A chunk made outside a CUDA-graph capture is not used
# inside one (and vice versa): a graph must own the fill of everything it accumulates into, or a replay
# would find the previous replay's sums.
_ARENA = threading.local()
_ARENA_FLOATS = 8192


def reset_zero_arena() -> None:
    _ARENA.state = None


def zero_scratch(n: int, device) -> torch.Tensor:
    """`n` zeroed fp32 elements on `device`, 128-byte aligned, valid for one use."""
    capturing = torch.cuda.is_current_stream_capturing()
    st = getattr(_ARENA, "state", None)
    if st is None or st["capturing"] != capturing or st["device"] != device or st["off"] + n > st["buf"].numel():
        st = {"buf": torch.zeros(max(_ARENA_FLOATS, n), device=device, dtype=torch.float32), "off": 0, "capturing": capturing, "device": device}
        _ARENA.state = st
        _launched()
    out = st["buf"][st["off"]:st["off"] + n]
    st["off"] += (n + 31) // 32 * 32
    return out


# ------------------------------------------------------------------------------------------ seeds
_SEED = {"base": 0x5EED, "counter": 0, "dev": {}}


def seed_state(device) -> torch.Tensor:
    """Per-device int64 scalar added to every dropout seed on the device side. A training step
    bumps it once (`seed_state(d).add_(k)`), also inside a captured CUDA graph, so replays draw
    fresh masks while forward and backward of one step agree."""
    key = str(device)
    t = _SEED["dev"].get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int64, device=device)
        _SEED["dev"][key] = t
    return t


def manual_seed(seed: int) -> None:
    _SEED["base"] = int(seed) & 0xFFFFFFFF
    _SEED["counter"] = 0
    for t in _SEED["dev"].values():
        t.zero_()


def next_seed() -> int:
    """Host-side seed of the next dropout site (deterministic given `manual_seed`)."""
    _SEED["counter"] += 1
    return (_SEED["base"] * 0x9E3779B1 + _SEED["counter"] * 0x85EBCA77) & 0x7FFFFFFFFFFF


# ---------------------------------------------------------------------------------------- helpers
# Below this many elements an eagerly launched op is bound by host time, and a Python autograd
# function around a native kernel costs several times an ATen op's dispatch (measured on B200: the
# small fp32 graph models of `benchmarks/` ran at 0.8x of plain PyTorch through the native path). So
# in plain eager mode small tensors take the PyTorch op; inside a CUDA-graph capture, and for the
# whole process once a flat-buffer engine exists (`set_eager_min_numel(0)`), the native kernels
# always run. Process-wide on purpose (autograd's backward thread must see the same value).
_EAGER = {"min_numel": int(os.environ.get("FLODL_B200_EAGER_MIN_NUMEL", str(1 << 20)))}


def set_eager_min_numel(n: int) -> None:
    _EAGER["min_numel"] = int(n)


def eager_min_numel() -> int:
    return _EAGER["min_numel"]


def _native_ok(x: torch.Tensor) -> bool:
    if not (FLAGS.native and x.is_cuda):
        return False
    n = _EAGER["min_numel"]
    return n <= 0 or x.numel() >= n or torch.cuda.is_current_stream_capturing()


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def _as_operand(t: torch.Tensor) -> torch.Tensor:
    """2-D bf16 view/copy a TMA descriptor can address: unit inner stride, row stride a multiple
    of 8 elements, 16-byte aligned base."""
    assert t.dim() == 2
    if t.dtype != BF16:
        t = t.to(BF16)
    if t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 and t.stride(0) >= t.size(1):
        return t
    rows, cols = t.shape
    buf = torch.empty(rows, _round_up(cols, 8), dtype=BF16, device=t.device)
    out = buf[:, :cols]
    out.copy_(t)
    return out


def _new_rows(rows: int, cols: int, dtype, device) -> torch.Tensor:
    """[rows, cols] tensor whose leading dimension is padded to 16 bytes."""
    mult = 8 if dtype == BF16 else 4
    ld = _round_up(cols, mult)
    buf = torch.empty(rows, ld, dtype=dtype, device=device)
    return buf if ld == cols else buf[:, :cols]


def _shadow(w: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a weight for the tensor cores: the flat-buffer engine keeps one up to date
    (`_fb_bf16`), otherwise cast on the fly."""
    s = getattr(w, "_fb_bf16", None)
    if s is not None:
        return s
    return w.detach() if w.dtype == BF16 else w.detach().to(BF16)


def _grad_slot(p: Optional[torch.Tensor]):
    return None if p is None else getattr(p, "_fb_grad", None)


def _f32(t: Optional[torch.Tensor]):
    if t is None:
        return None
    t = t.detach()
    return t if t.dtype == torch.float32 and t.is_contiguous() else t.float().contiguous()


def _pick_dw_plan(m_out: int, n_out: int, k_red: int):
    """(config, split_k) for a weight-gradient GEMM (few output tiles, long reduction), from
    measurements on B200: enough 256x256 pair tiles -> pair config, else split the reduction."""
    pair_tiles = math.ceil(m_out / 256) * math.ceil(n_out / 256)
    if pair_tiles >= 148 or k_red < 1024:
        return -1, 1
    if pair_tiles >= 24:
        return 0, 2 if k_red >= 2048 else 1
    return 2, max(1, min(4, k_red // 512))


# ---- weight gradients beside the data gradient ------------------------------------------------------
# dX and dW of a linear layer are independent products of the same upstream gradient. Issued on two
# streams they share the GPU: the blocks of one fill the SMs the other leaves idle in its last
# (partial) wave and behind its fixed latencies, and the small bias-gradient column sums vanish
# behind the GEMMs. The side stream forks from the current stream and is joined before backward()
# returns, so the saved activations outlive every kernel that reads them. FLODL_B200_SIDE_DW=0
# keeps everything on one stream.
_SIDE = {"on": os.environ.get("FLODL_B200_SIDE_DW", "1") not in ("0", "false", "off"), "streams": {}}


# Outside a capture a step of small layers is bound by the host's launch rate, not by the GPU: there the two extra
# stream switches, two waits and the event of a fork (measured on B200: 40..70 us of host time per linear backward,
# 1.5 ms of a 9 ms eager BERT-base step) cost more than the overlap returns. So an eager backward forks only for
# products large enough to keep the GPU busy longer than the host needs to issue them (`work`, in multiply-adds, at least
# FLODL_B200_EAGER_FORK_MACS, default 2^35); a capture always forks (replay pays no host time).
_EAGER_FORK_MACS = int(os.environ.get("FLODL_B200_EAGER_FORK_MACS", str(1 << 35)))


class _Fork:
    """`with fork: ...` runs the body on the side stream (after everything issued so far on the
    current stream); `fork.join()` makes the current stream wait for it."""

    def __init__(self, device: torch.device, work: int = 0):
        self.active = _SIDE["on"] and device.type == "cuda"
        if self.active:
            capturing = torch.cuda.is_current_stream_capturing()
            if not capturing and work < _EAGER_FORK_MACS:
                self.active = False
                return
            self.main = torch.cuda.current_stream(device)
            key = (device.index, capturing)
            side = _SIDE["streams"].get(key)
            if side is None:
                side = _SIDE["streams"][key] = torch.cuda.Stream(device)
            self.side = side
            self.used = False

    def __enter__(self):
        if self.active:
            self.side.wait_stream(self.main)
            torch.cuda.set_stream(self.side)          # the plain call: the `torch.cuda.stream()` context manager costs several times as much
            self.used = True
        return self

    def __exit__(self, *exc):
        if self.active:
            torch.cuda.set_stream(self.main)
        return False

    def join(self) -> None:
        if self.active and self.used:
            self.main.wait_stream(self.side)


_EPI = {None: 0, "gelu": 1, "gelu_tanh": 3}
_DEPI = {"gelu": 2, "gelu_tanh": 4}


def _weight_grad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, alpha=None, k_dyn=None, k_hint: Optional[int] = None):
    """dW[N,K] = dy2^T x2 on the tensor cores (both operands MN-major). Accumulates straight into
    the flat gradient buffer when the parameter has a slot there, else returns a tensor.
    `k_dyn` (device int32): only that many rows of the operands take part (compacted rows);
    `k_hint` is the host's estimate of it for choosing the split."""
    C = _C()
    N, K = dy2.shape[1], x2.shape[1]
    slot = _grad_slot(w)
    cfg, sk = _pick_dw_plan(N, K, dy2.shape[0] if k_hint is None else k_hint)
    if k_dyn is not None:
        sk = 1          # the split is over the static reduction length; a dynamic one runs unsplit
    if slot is not None:
        C.gemm(dy2, x2, slot.view(N, K), True, True, alpha=alpha, accumulate=True, split_k=sk, config=cfg, k_dyn=k_dyn)
        _launched()
        _touched(w)
        return None
    out = torch.zeros(N, K, dtype=torch.float32, device=dy2.device) if sk > 1 else torch.empty(N, K, dtype=torch.float32, device=dy2.device)
    C.gemm(dy2, x2, out, True, True, alpha=alpha, accumulate=sk > 1, split_k=sk, config=cfg, k_dyn=k_dyn)
    _launched()
    return out.to(w.dtype)


def _bias_grad(dy2: torch.Tensor, b: torch.Tensor, alpha=None, rows_dyn=None):
    C = _C()
    slot = _grad_slot(b)
    if slot is not None and alpha is None:
        C.colsum(dy2, slot.view(-1), rows_dyn)
        _launched()
        _touched(b)
        return None
    tmp = torch.zeros(dy2.shape[1], dtype=torch.float32, device=dy2.device)
    C.colsum(dy2, tmp, rows_dyn)
    _launched()
    if alpha is not None:
        tmp = tmp * alpha
    if slot is not None:
        slot.view(-1).add_(tmp)
        _touched(b)
        return None
    return tmp.to(b.dtype)


# ----------------------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act):
        C = _C()
        K = x.shape[-1]
        N = w.shape[0]
        x2 = _as_operand(x.reshape(-1, K))
        w16 = _as_operand(_shadow(w))
        out = _new_rows(x2.shape[0], N, BF16, x.device)
        aux = _new_rows(x2.shape[0], N, BF16, x.device) if act else None
        C.gemm(x2, w16, out, False, False, bias=None if b is None else b.detach(), epi=_EPI[act], aux=aux)
        _launched()
        ctx.save_for_backward(x2, w16, aux)
        ctx.w, ctx.b, ctx.act, ctx.xshape = w, b, act, x.shape
        return out.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x2, w16, aux = ctx.saved_tensors
        w, b, act = ctx.w, ctx.b, ctx.act
        N = w.shape[0]
        dy2 = dy.reshape(-1, N)
        if act:
            dy2 = C.gelu_bwd(dy2.contiguous().to(BF16), aux.contiguous(), act == "gelu_tanh")
            _launched()
        dy2 = _as_operand(dy2)
        dx = dw = db = None
        fork = _Fork(dy.device, dy2.shape[0] * dy2.shape[1] * x2.shape[1])
        with fork:
            if ctx.needs_input_grad[1]:
                dw = _weight_grad(dy2, x2, w)
            if b is not None and ctx.needs_input_grad[2]:
                db = _bias_grad(dy2, b)
        if ctx.needs_input_grad[0]:
            dx2 = _new_rows(x2.shape[0], x2.shape[1], BF16, dy.device)
            C.gemm(dy2, w16, dx2, False, True)
            _launched()
            dx = dx2.view(ctx.xshape)
        fork.join()
        return dx, dw, db, None


def _gemm_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    if not _native_ok(x) or w.dim() != 2:
        return False
    if x.dtype != BF16 and FLAGS.autocast != BF16:
        return False
    return x.shape[-1] % 8 == 0 and x.numel() > 0


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, activation: Optional[str] = None):
    """y = act(x W^T + b); `activation` in {None, "gelu", "gelu_tanh"} is fused into the GEMM epilogue.
    Counterpart of `autograd::linear` (flodl/src/autograd/ops.rs:570-581)."""
    if _gemm_eligible(x, weight):
        if x.dtype != BF16:
            x = x.to(BF16)
        return _LinearFn.apply(x, weight, bias, activation)
    w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
    b = bias if bias is None or bias.dtype == x.dtype else bias.to(x.dtype)
    y = F.linear(x, w, b)
    if activation == "gelu":
        y = F.gelu(y)
    elif activation == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    return y


# ------------------------------------------------------------------------------------ feed-forward
class _FeedForwardFn(torch.autograd.Function):
    """y = act(x W1^T + b1) W2^T + b2 with the activation in the first GEMM's epilogue and its
    derivative in the epilogue of the backward GEMM that produces d(pre-activation)."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, act):
        C = _C()
        K = x.shape[-1]
        x2 = _as_operand(x.reshape(-1, K))
        M = x2.shape[0]
        w1s, w2s = _as_operand(_shadow(w1)), _as_operand(_shadow(w2))
        F1, N = w1.shape[0], w2.shape[0]
        h_pre = _new_rows(M, F1, BF16, x.device)
        a = _new_rows(M, F1, BF16, x.device)
        C.gemm(x2, w1s, a, False, False, bias=None if b1 is None else b1.detach(), epi=_EPI[act], aux=h_pre)
        y = _new_rows(M, N, BF16, x.device)
        C.gemm(a, w2s, y, False, False, bias=None if b2 is None else b2.detach())
        _launched(2)
        ctx.save_for_backward(x2, w1s, w2s, h_pre, a)
        ctx.params = (w1, b1, w2, b2)
        ctx.act, ctx.xshape = act, x.shape
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        C = _C()
        x2, w1s, w2s, h_pre, a = ctx.saved_tensors
        w1, b1, w2, b2 = ctx.params
        N = w2.shape[0]
        dy2 = _as_operand(dy.reshape(-1, N))
        M, F1 = a.shape
        dpre = _new_rows(M, F1, BF16, dy.device)
        fork = _Fork(dy.device, M * F1 * N)
        with fork:       # the second layer's parameter gradients need only dy: beside the d(pre-activation) GEMM
            dw2 = _weight_grad(dy2, a, w2) if ctx.needs_input_grad[3] else None
            db2 = _bias_grad(dy2, b2) if (b2 is not None and ctx.needs_input_grad[4]) else None
        C.gemm(dy2, w2s, dpre, False, True, epi=_DEPI[ctx.act], aux=h_pre)
        _launched()
        with fork:       # the first layer's, beside the dX GEMM (the side stream waits for dpre here)
            dw1 = _weight_grad(dpre, x2, w1) if ctx.needs_input_grad[1] else None
            db1 = _bias_grad(dpre, b1) if (b1 is not None and ctx.needs_input_grad[2]) else None
        dx = None
        if ctx.needs_input_grad[0]:
            dx2 = _new_rows(M, x2.shape[1], BF16, dy.device)
            C.gemm(dpre, w1s, dx2, False, True)
            _launched()
            dx = dx2.view(ctx.xshape)
        fork.join()
        return dx, dw1, db1, dw2, db2, None


def feed_forward(x, w1, b1, w2, b2, activation: str = "gelu"):
    if _gemm_eligible(x, w1) and w1.shape[0] % 8 == 0:
        if x.dtype != BF16:
            x = x.to(BF16)
        return _FeedForwardFn.apply(x, w1, b1, w2, b2, activation)
    return linear(linear(x, w1, b1, activation), w2, b2)


# -------------------------------------------------------------------------------------- LayerNorm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, beta, eps, p_drop, seed):
        C = _C()
        xc = x.contiguous()
        rc = None if residual is None else residual.contiguous()
        want_pre = rc is not None or p_drop > 0.0
        sd = seed_state(x.device) if p_drop > 0.0 else None
        y, pre, mean, rstd = C.layernorm_fwd(xc, rc, _f32(gamma), _f32(beta), eps, p_drop, seed, want_pre, sd)
        _launched()
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(pre if want_pre else xc, mean, rstd)
        ctx.gamma, ctx.beta, ctx.p, ctx.seed = gamma, beta, p_drop, seed
        ctx.has_res = rc is not None
        if not want_pre:  # the pre-normalisation value is the input itself: hand back a placeholder
            pre = y.new_empty(0)
            ctx.mark_non_differentiable(pre)
        return y, pre

    @staticmethod
    def backward(ctx, dy, dpre_extra):
        C = _C()
        if dy is None:   # only the pre-normalisation output was used downstream
            pre0 = ctx.saved_tensors[0]
            return (dpre_extra if ctx.p == 0.0 else C.dropout(dpre_extra.contiguous(), ctx.p, ctx.seed, seed_state(pre0.device)),
                    dpre_extra if ctx.has_res else None, None, None, None, None, None)
        pre, mean, rstd = ctx.saved_tensors
        gamma, beta, p = ctx.gamma, ctx.beta, ctx.p
        want_pg = (gamma is not None and ctx.needs_input_grad[2]) or (beta is not None and ctx.needs_input_grad[3])
        gslot, bslot = _grad_slot(gamma), _grad_slot(beta)
        use_slots = want_pg and gslot is not None and bslot is not None
        sd = seed_state(dy.device) if p > 0.0 else None
        simple = dpre_extra is None or dpre_extra.numel() == 0
        dpre, dxd, dg, db = C.layernorm_bwd(dy.contiguous(), pre, mean, rstd, _f32(gamma), p, ctx.seed, p > 0.0 and simple,
                                            want_pg, gslot.view(-1) if use_slots else None,
                                            bslot.view(-1) if use_slots else None, sd)
        _launched(2 if want_pg else 1)
        if not simple:
            dpre = dpre + dpre_extra
            dxd = C.dropout(dpre, p, ctx.seed, sd) if p > 0.0 else None
        dx = dxd if p > 0.0 else dpre
        dres = dpre if ctx.has_res else None
        if use_slots:
            _touched(gamma)
            _touched(beta)
        if use_slots or not want_pg:
            dg = db = None
        else:
            dg = dg.to(gamma.dtype) if gamma is not None else None
            db = db.to(beta.dtype) if beta is not None else None
        return dx, dres, dg, db, None, None, None


def _ln_eligible(x: torch.Tensor) -> bool:
    if not _native_ok(x) or x.dtype not in (BF16, torch.float32):
        return False
    cols = x.shape[-1]
    return cols <= 1024 and cols % (8 if x.dtype == BF16 else 4) == 0 and x.numel() > 0


def layer_norm(x, gamma=None, beta=None, eps: float = 1e-5, residual=None, p_drop: float = 0.0,
               training: bool = False, return_pre: bool = False):
    """LayerNorm over the last dim of `residual + dropout(x)` (both optional), one fused kernel.
    With `return_pre` also returns the pre-normalisation sum (the next residual in pre-LN blocks).
    Counterpart of `autograd::layer_norm` (flodl/src/autograd/ops.rs:625-637)."""
    p = p_drop if training else 0.0
    if _ln_eligible(x) and (residual is None or residual.dtype == x.dtype):
        y, pre = _LayerNormFn.apply(x, residual, gamma, beta, float(eps), float(p), next_seed() if p > 0 else 0)
        if pre.numel() == 0 and x.numel() != 0:
            pre = x
        return (y, pre) if return_pre else y
    h = F.dropout(x, p, True) if p > 0 else x
    if residual is not None:
        h = h + residual
    g = None if gamma is None else gamma.to(h.dtype)
    b = None if beta is None else beta.to(h.dtype)
    y = F.layer_norm(h, (h.shape[-1],), g, b, eps)
    return (y, h) if return_pre else y


# --------------------------------------------------------------------------------- GELU / dropout
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tanh_approx):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        ctx.tanh = tanh_approx
        _launched()
        return _C().gelu_fwd(xc, tanh_approx)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        _launched()
        return _C().gelu_bwd(dy.contiguous(), x, ctx.tanh), None


def gelu(x: torch.Tensor, approximate: str = "none") -> torch.Tensor:
    if _native_ok(x) and x.dtype in (BF16, torch.float32) and x.numel() > 0:
        return _GeluFn.apply(x, approximate == "tanh")
    return F.gelu(x, approximate=approximate)


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed):
        ctx.p, ctx.seed = p, seed
        _launched()
        return _C().dropout(x.contiguous(), p, seed, seed_state(x.device))

    @staticmethod
    def backward(ctx, dy):
        _launched()
        return _C().dropout(dy.contiguous(), ctx.p, ctx.seed, seed_state(dy.device)), None, None


def dropout(x: torch.Tensor, p: float, training: bool = True) -> torch.Tensor:
    if not training or p <= 0.0:
        return x
    if p >= 1.0:
        return x * 0
    if _native_ok(x) and x.dtype in (BF16, torch.float32) and x.numel() > 0:
        return _DropoutFn.apply(x, float(p), next_seed())
    return F.dropout(x, p, True)


# ----------------------------------------------------------------------------------- cross entropy
class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index):
        lg = logits if logits.stride(1) == 1 else logits.contiguous()
        loss, dl, _ = _C().softmax_ce(lg, target.contiguous(), ignore_index, True, False)
        _launched(3)
        ctx.save_for_backward(dl)
        return loss.to(logits.dtype) if logits.dtype != torch.float32 else loss

    @staticmethod
    def backward(ctx, g):
        (dl,) = ctx.saved_tensors
        _C().scale_rows(dl, g.detach().float().reshape(1))
        _launched()
        return dl, None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean softmax cross-entropy over rows whose target is not `ignore_index`
    (`cross_entropy_loss`, flodl/src/nn/loss.rs:34-43: 2-D logits, class-index targets)."""
    if logits.dim() != 2:
        raise ValueError("cross_entropy expects [rows, classes] logits")
    if _native_ok(logits) and logits.dtype in (BF16, torch.float32) and target.dtype == torch.int64 and logits.numel() > 0:
        return _CrossEntropyFn.apply(logits, target, int(ignore_index))
    return F.cross_entropy(logits.float() if logits.dtype == BF16 else logits, target, ignore_index=ignore_index)


class _LinearCrossEntropyFn(torch.autograd.Function):
    """loss = CE(x W^T + b, target): logits are produced by the tensor-core GEMM into a padded
    buffer, the softmax kernel overwrites them with the gradient, and the backward GEMMs read that
    buffer with the upstream scalar as their `alpha`."""

    @staticmethod
    def forward(ctx, x, w, b, target, ignore_index, compact):
        C = _C()
        K = x.shape[-1]
        x2 = _as_operand(x.reshape(-1, K))
        w16 = _as_operand(_shadow(w))
        V = w.shape[0]
        rows = x2.shape[0]
        tgt = target.reshape(-1).contiguous()
        idx = counts = None
        if compact:
            # Rows whose target is `ignore_index` add nothing to the loss or to any gradient. Pack the
            # others to the front (device-side count, static buffer sizes), run the projection, the
            # softmax and the three backward GEMMs on those rows only, and scatter dX back.
            idx, tgt, counts = C.compact_targets(tgt, ignore_index)
            xc = _new_rows(rows, K, BF16, x.device)
            C.gather_rows(x2, idx, counts, xc)
            x2 = xc
            _launched(2)
        logits = _new_rows(rows, V, BF16, x.device)
        C.gemm(x2, w16, logits, False, False, bias=None if b is None else b.detach(), m_dyn=None if counts is None else counts[0:1])
        loss, dl, _ = C.softmax_ce(logits, tgt, ignore_index, True, True, counts)
        _launched(4)
        ctx.save_for_backward(x2, w16, dl, idx, counts)
        ctx.w, ctx.b, ctx.xshape = w, b, x.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        C = _C()
        x2, w16, dl, idx, counts = ctx.saved_tensors
        w, b = ctx.w, ctx.b
        alpha = g.detach().float().reshape(1)
        n_dyn = None if counts is None else counts[0:1]
        dx = dw = db = None
        fork = _Fork(dl.device, dl.shape[0] * dl.shape[1] * x2.shape[1])
        with fork:
            if ctx.needs_input_grad[1]:
                dw = _weight_grad(dl, x2, w, alpha=alpha, k_dyn=n_dyn, k_hint=None if counts is None else max(64, x2.shape[0] // 6))
            if b is not None and ctx.needs_input_grad[2]:
                db = _bias_grad(dl, b, alpha=alpha, rows_dyn=n_dyn)
        if ctx.needs_input_grad[0]:
            dx2 = _new_rows(x2.shape[0], x2.shape[1], BF16, dl.device)
            C.gemm(dl, w16, dx2, False, True, alpha=alpha, m_dyn=n_dyn)
            _launched()
            if counts is not None:
                full = torch.zeros_like(dx2)
                C.scatter_rows(dx2, idx, counts, full)
                _launched(2)
                dx2 = full
            dx = dx2.view(ctx.xshape)
        fork.join()
        return dx, dw, db, None, None, None


def linear_cross_entropy(x, weight, bias, target, ignore_index: int = -100, sparse_targets: bool = False) -> torch.Tensor:
    """Vocabulary projection + mean cross-entropy in one op (the masked-LM / LM head hot path:
    `masked_lm_loss`, flodl-hf/src/task_heads.rs:170-183, over the tied decoder of
    flodl-hf/src/models/bert.rs:707-752). `sparse_targets=True` says most targets are
    `ignore_index` (masked-LM): the projection and its gradients are then computed for the
    labelled rows only, which gives the same loss and the same gradients."""
    if _gemm_eligible(x, weight) and target.dtype == torch.int64:
        if x.dtype != BF16:
            x = x.to(BF16)
        rows = x.numel() // x.shape[-1]
        return _LinearCrossEntropyFn.apply(x, weight, bias, target, int(ignore_index), bool(sparse_targets) and rows >= 512)
    logits = linear(x, weight, bias)
    return cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1), ignore_index)


# -------------------------------------------------------------------------------------- attention
class _AttnQKVFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, mask, scale, causal, p_drop, seed):
        C = _C()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        sd = seed_state(qkv.device) if p_drop > 0 else None
        o, lse = C.attn_fwd(q, k, v, mask, scale, causal, p_drop, seed, sd)
        _launched()
        ctx.save_for_backward(qkv, o, lse, mask)
        ctx.cfg = (scale, causal, p_drop, seed)
        return o

    @staticmethod
    def backward(ctx, do):
        C = _C()
        qkv, o, lse, mask = ctx.saved_tensors
        scale, causal, p_drop, seed = ctx.cfg
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        sd = seed_state(qkv.device) if p_drop > 0 else None
        dqkv = C.attn_bwd(q, k, v, o, do.contiguous(), lse, mask, scale, causal, p_drop, seed, sd)
        _launched()
        return dqkv, None, None, None, None, None


def _key_mask(mask: Optional[torch.Tensor], B: int, S: int):
    """Reduce an additive mask to the [B, S] key-mask form the kernel takes, or None if it has
    per-query structure."""
    if mask is None:
        return True, None
    m = mask
    if m.dim() == 4 and m.shape[1] == 1 and m.shape[2] == 1:
        m = m[:, 0, 0]
    if m.dim() == 2 and m.shape[-1] == S and m.shape[0] in (1, B):
        return True, m.expand(B, S).float().contiguous()
    return False, None


def attention(qkv: Optional[torch.Tensor] = None, q=None, k=None, v=None, mask=None, causal: bool = False,
              p_drop: float = 0.0, training: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """softmax(Q K^T * scale + mask) V with optional causal masking and dropout on the probabilities.

    Takes either a packed `qkv` [B, S, 3, H, D] (what a fused QKV projection produces) or separate
    `q`, `k`, `v` [B, S, H, D]; returns [B, S, H, D]. Counterpart of
    `autograd::scaled_dot_product_attention` (flodl/src/autograd/ops.rs:947-963)."""
    p = p_drop if training else 0.0
    if qkv is None and (q.shape != k.shape or k.shape != v.shape or not (_native_ok(q) and q.dtype == BF16 and q.shape[-1] == 64)):
        # cross-attention (different query / key lengths) and everything the tensor-core kernel does
        # not take: no packing, straight to the library op
        D = q.shape[-1]
        scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
        qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    else:
        if qkv is None:
            qkv = torch.stack((q, k, v), dim=2)
        B, S, _, H, D = qkv.shape
        scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
        ok, km = _key_mask(mask, B, S)
        if _native_ok(qkv) and qkv.dtype == BF16 and D == 64 and ok and qkv.stride(4) == 1 and all(s % 8 == 0 for s in qkv.stride()[:4]):
            return _AttnQKVFn.apply(qkv, km, scale, bool(causal), float(p), next_seed() if p > 0 else 0)
        qh, kh, vh = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    am = None
    if mask is not None:
        am = mask.to(qh.dtype)
        while am.dim() < 4:
            am = am.unsqueeze(1) if am.dim() >= 2 else am.unsqueeze(0)
    o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=am, dropout_p=p, is_causal=bool(causal) and am is None, scale=scale) \
        if not (causal and am is not None) else _sdpa_causal_masked(qh, kh, vh, am, p, scale)
    return o.permute(0, 2, 1, 3)


def _sdpa_causal_masked(qh, kh, vh, am, p, scale):
    S = qh.shape[-2]
    causal = torch.full((S, S), float("-inf"), device=qh.device, dtype=qh.dtype).triu(1)
    return F.scaled_dot_product_attention(qh, kh, vh, attn_mask=am + causal, dropout_p=p, scale=scale)


# -------------------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, padding_idx):
        src = weight
        ctx.save_for_backward(ids)
        ctx.weight, ctx.pad = weight, -1 if padding_idx is None else int(padding_idx)
        return F.embedding(ids, src.detach())

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.weight
        slot = _grad_slot(w)
        dyc = dy.contiguous()
        if slot is not None:
            _C().embedding_bwd(dyc, ids.contiguous(), slot.view(w.shape), ctx.pad)
            _launched()
            _touched(w)
            return None, None, None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        _C().embedding_bwd(dyc, ids.contiguous(), dw, ctx.pad)
        _launched()
        return None, dw.to(w.dtype), None


def embedding(ids: torch.Tensor, weight: torch.Tensor, padding_idx=None) -> torch.Tensor:
    """Row gather; the backward scatter-add goes straight into the flat gradient buffer on CUDA
    (`at::embedding`, flodl-sys/ops_training.cpp:1080)."""
    if _native_ok(weight) and weight.dtype == torch.float32 and weight.requires_grad and ids.dtype == torch.int64:
        return _EmbeddingFn.apply(ids, weight, padding_idx)
    return F.embedding(ids, weight, padding_idx)


# ------------------------------------------------------------------------------------- batch norm
def batch_norm(x, running_mean, running_var, weight, bias, training: bool, momentum: float = 0.1, eps: float = 1e-5,
               relu: bool = False, residual=None):
    """BatchNorm over dim 1 (+ optional residual add and ReLU). Counterpart of `flodl_batch_norm`
    (flodl-sys/ops_training.cpp:1025-1046)."""
    from . import bn
    return bn.batch_norm(x, running_mean, running_var, weight, bias, training, momentum, eps, relu, residual)
