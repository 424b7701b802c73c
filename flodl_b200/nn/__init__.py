"""Neural-network layer: modules, activations, losses, optimizers, schedulers, initialisers,
clipping, mixed precision, CUDA graphs and checkpoints (flodl/src/nn/mod.rs:1-108)."""
from . import init  # noqa: F401
from .activation import (ELU, GELU, SELU, Flatten, GeluApprox, Hardsigmoid, Hardswish, Identity, LeakyReLU,  # noqa: F401
                         LogSoftmax, Mish, PReLU, ReLU, Sigmoid, SiLU, Softmax, Softplus, Tanh)
from .amp import AutocastGuard, GradScaler, autocast, cast_parameters, is_autocast_enabled  # noqa: F401
from .checkpoint import (LoadReport, MigrateReport, checkpoint_keys, checkpoint_version, load_checkpoint,  # noqa: F401
                         load_checkpoint_file, migrate_checkpoint, migrate_checkpoint_file, save_checkpoint,
                         save_checkpoint_file)
from .clip import clip_grad_norm, clip_grad_norm_fused, clip_grad_value  # noqa: F401
from .cuda_graph import CaptureMode, CudaGraph, MemPoolId, cuda_graph_capture, cuda_graph_pool_handle  # noqa: F401
from .init import (kaiming_normal, kaiming_uniform, normal, orthogonal, trunc_normal, uniform, uniform_bias,  # noqa: F401
                   xavier_normal, xavier_uniform)
from .layers import (GRU, LSTM, AdaptiveAvgPool2d, AdaptiveMaxPool2d, AlphaDropout, AvgPool1d, AvgPool2d, BatchNorm,  # noqa: F401
                     BatchNorm2d, Bilinear, Conv1d, Conv1dBuilder, Conv2d, Conv2dBuilder, Conv3d, Conv3dBuilder, ConvTranspose1d, ConvTranspose1dBuilder, ConvTranspose2dBuilder, ConvTranspose3dBuilder, ConvTranspose2d, ConvTranspose3d,
                     Dropout, Dropout2d, Embedding, EmbeddingBag, Fold, GaussianBlur, GroupNorm, GRUCell, InstanceNorm,
                     LayerNorm, Linear, LSTMCell, MaxPool1d, MaxPool2d, MultiheadAttention, PixelShuffle, PixelUnshuffle,
                     ReflectionPad2d, RMSNorm, Unfold, Upsample, ZeroPad2d, gaussian_blur_2d)
from .loss import (bce_loss, bce_with_logits_loss, cosine_embedding_loss, cross_entropy_loss, ctc_loss, focal_loss,  # noqa: F401
                   hinge_embedding_loss, kl_div_loss, l1_loss, margin_ranking_loss, mse_loss, nll_loss, poisson_nll_loss,
                   smooth_l1_loss, triplet_margin_loss)
from .module import (Buffer, LoopBody, LoopBodyEmit, Module, NamedInputModule, Parameter, TraceEmit, collect_parameters,  # noqa: F401
                     forward_via_step, modules, walk_modules, walk_modules_visited)  # noqa: F401
from .optim import (SGD, Adagrad, AdagradBuilder, Adam, AdamBuilder, AdamW, AdamWBuilder, NAdam, Optimizer, RAdam, RMSprop,  # noqa: F401
                    RMSpropBuilder, SGDBuilder, Stateful)  # noqa: F401
from .scheduler import (CosineScheduler, CyclicLR, ExponentialLR, MultiStepLR, OneCycleLR, PlateauScheduler, Scheduler,  # noqa: F401
                        StepDecay, WarmupScheduler)
