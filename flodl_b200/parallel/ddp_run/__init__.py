"""Asynchronous data parallelism (Local SGD with periodic parameter averaging): thread or
process per GPU, a coordinator that decides when to average, three apply policies, two averaging
backends (flodl/src/distributed/ddp_run/)."""
from .channel import LocalTransport, StoreTransport, make_store_transport  # noqa: F401
from .chunk_pool import ChunkPool  # noqa: F401
from .convergence import ConvergenceAction, ConvergenceGuard, DivergenceReport  # noqa: F401
from .coordinator import (Coordinator, aggregate_epoch_metrics, average_and_divergence, average_params, divergence_of, equal_sizes,  # noqa: F401
                          ratio_to_sizes, throughput_sizes)
from .messages import (ApplyPolicy, AverageBackend, AveragedParams, ControlMsg, DdpRunConfig, EpochMetrics, EpochPlan,  # noqa: F401
                       MetricsFn, MetricsMsg, ParamSnapshot, TimingBatch, TimingExiting, TimingMsg, TimingSyncAck,
                       TrainedState, WorkerConfig, drain_scalars, make_partition, record_scalar)
from .orchestrator import DdpBuilder, DdpHandle  # noqa: F401
from .worker import GpuWorker  # noqa: F401
