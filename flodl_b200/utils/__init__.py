"""Small helpers that are not part of the training API: device-side timing for the benchmark scripts."""
from .timing import cuda_time_ms, flush_l2, graph_chain_us, median_ms  # noqa: F401
