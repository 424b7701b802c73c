"""Training monitor: per-epoch console line + ETA, resource sampling, live dashboard, timeline
(flodl/src/monitor/)."""
from .format import format_bytes, format_eta, format_metric  # noqa: F401
from .monitor import EpochRecord, GpuMetrics, Metrics, Monitor  # noqa: F401
from .resources import GpuSnapshot, ResourceSample, ResourceSampler  # noqa: F401
from .server import DashboardServer  # noqa: F401
from .timeline import (EVENT_KINDS, EventKind, GpuTimelineSample, Timeline, TimelineBroadcast, TimelineEvent, TimelineSample,  # noqa: F401
                       TimelineSummary)  # noqa: F401
