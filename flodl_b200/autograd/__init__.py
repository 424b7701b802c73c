"""Autograd layer: `Variable`, gradient-mode guards and the differentiable op surface
(flodl/src/autograd/mod.rs:16-33)."""
from .context import NoGradGuard, is_grad_enabled, no_grad  # noqa: F401
from .ops import *  # noqa: F401,F403
from .variable import Variable  # noqa: F401
