"""flodl_b200: a deep-learning framework written for NVIDIA B200 (sm_100a).

PyTorch supplies tensors and the autograd engine; the hot operators (tcgen05 GEMM, flash
attention, LayerNorm, GELU, softmax cross-entropy, BatchNorm, fused Adam/SGD, gradient norm) and the
multi-GPU collectives (all-reduce, parameter averaging, broadcast over NVLink peer memory) are this
library's own CUDA kernels; the runtime around them (checkpoint format, RNG, prefetch, cadence
controller) is C++. The user-facing surface follows flodl's (flodl/src/lib.rs:54-108): the names
below are importable from the package root.
"""
from . import log  # noqa: F401
from .autograd import NoGradGuard, Variable, is_grad_enabled, no_grad  # noqa: F401
from .autograd.ops import (adaptive_avg_pool2d, embedding, embedding_bag, grid_sample, max_pool2d,  # noqa: F401
                           scaled_dot_product_attention)
from .data import (Batch, BatchDataSet, DataLoader, DataLoaderBuilder, DataSet, DistributedEpochIterator, EpochIterator,  # noqa: F401
                   RandomSampler, Sampler, SequentialSampler, TensorDataSet)
from .graph import (ActiveGraphEpochIterator, ArgmaxSelector, FixedSelector, FlowBuilder, Graph, GraphEpochIterator, LearnedHalt, LevelTiming,  # noqa: F401
                    LossContext, MapBuilder, MergeOp, ModelSnapshot, NodeTiming, PathKind, Profile, Reduce, Reshape,
                    SigmoidRouter, SoftmaxRouter, StateAdd, ThresholdHalt, Trend, TrendGroup, format_duration)
from .log import Verbosity, set_verbosity, verbosity  # noqa: F401
from .nn import *  # noqa: F401,F403
from .nn.module import walk_modules, walk_modules_visited  # noqa: F401
from .monitor import Monitor  # noqa: F401
from .parallel.comm import (CudaEvent, CudaEventFlags, CudaStream, NcclAbortHandle, NcclComms, NcclRankComm, NcclUniqueId, ReduceOp,  # noqa: F401
                            StreamGuard, SymmetricBuffer)
from .parallel.ddp import Ddp, DdpConfig, DistributedState, HasGraph, Trainer  # noqa: F401
from .parallel.ddp_run import (ApplyPolicy, AverageBackend, DdpBuilder, DdpHandle, DdpRunConfig, EpochMetrics, GpuWorker,  # noqa: F401
                               MetricsFn, TrainedState, drain_scalars, record_scalar)
from .parallel.el_che import ElChe  # noqa: F401
from .parallel.engine import TrainEngine  # noqa: F401
from .rng import Rng  # noqa: F401
from .tensor import (DeviceInfo, DType, Device, Result, Tensor, TensorError, TensorOptions, cuda_active_bytes,  # noqa: F401
                     cuda_active_bytes_idx, cuda_allocated_bytes, cuda_allocated_bytes_idx, cuda_available,
                     cuda_compute_capability, cuda_device_count, cuda_device_name, cuda_device_name_idx, cuda_devices,
                     cuda_empty_cache, cuda_manual_seed_all, cuda_memory_info, cuda_memory_info_idx, cuda_peak_active_bytes,
                     cuda_peak_active_bytes_idx, cuda_peak_allocated_bytes, cuda_peak_reserved_bytes,
                     cuda_peak_reserved_bytes_idx, cuda_reset_peak_stats, cuda_reset_peak_stats_idx, cuda_synchronize,
                     cuda_utilization, cuda_utilization_idx, current_cuda_device, hardware_summary, live_tensor_count,
                     malloc_trim, manual_seed, probe_device, rss_kb, set_cudnn_benchmark, set_current_cuda_device,
                     usable_cuda_devices)
from .worker import CpuWorker  # noqa: F401

__version__ = "0.1.0"
