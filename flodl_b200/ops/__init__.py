"""Functional ops on `torch.Tensor`s, backed by this library's sm_100a kernels on CUDA.

Every function here has two paths:

* CUDA + a dtype/shape the native kernels cover  -> a `torch.autograd.Function` whose forward and
  backward launch kernels from `flodl_b200._C` (tcgen05 GEMM, flash attention, fused LayerNorm,
  GELU, softmax cross-entropy, ...). PyTorch's autograd engine still drives backward, the way
  libtorch's engine does in the reference (flodl/src/autograd/variable.rs:199-204).
* anything else (CPU, fp64, odd shapes)          -> the plain PyTorch op with the same semantics.

On a CUDA device the native library is mandatory: if it cannot be loaded these functions raise
instead of silently running the PyTorch path.
"""
from .core import (  # noqa: F401
    FLAGS,
    attention,
    batch_norm,
    cross_entropy,
    dropout,
    embedding,
    feed_forward,
    gelu,
    layer_norm,
    linear,
    linear_cross_entropy,
    native_enabled,
    next_seed,
    seed_state,
    set_native,
)
