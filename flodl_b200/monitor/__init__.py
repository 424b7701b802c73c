"""Training monitor: per-epoch console line + ETA, resource sampling, live dashboard, timeline
(flodl/src/monitor/)."""
from .format import format_bytes, format_eta, format_metric  # noqa: F401
from .monitor import EpochRecord, GpuMetrics, Monitor  # noqa: F401
from .resources import GpuSnapshot, ResourceSample, ResourceSampler  # noqa: F401
from .server import DashboardServer  # noqa: F401
from .timeline import EVENT_KINDS, Timeline, TimelineEvent, TimelineSample, TimelineSummary  # noqa: F401
