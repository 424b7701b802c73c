"""Graph layer: `FlowBuilder` -> `Graph`, control-flow nodes, graph tree, observation, profiling,
rendering, snapshots (flodl/src/graph/mod.rs:21-92)."""
from .flow import FlowBuilder, LoopBuilder, MapBuilder, MergeOp  # noqa: F401
from .graph import Graph, sidecar_config_path, topological_levels  # noqa: F401
from .helpers import (ArgmaxSelector, FixedSelector, LearnedHalt, Reshape, SigmoidRouter, SoftmaxRouter, StateAdd,  # noqa: F401
                      ThresholdHalt)
from .observe import Reduce  # noqa: F401
from .profile import LevelTiming, NodeTiming, Profile  # noqa: F401
from .render import format_duration  # noqa: F401
from .snapshot import ModelSnapshot, snapshot_cpu  # noqa: F401
from .tree import PathKind  # noqa: F401
from .trend import Trend, TrendGroup  # noqa: F401
from .distributed import ActiveGraphEpochIterator, GraphEpochIterator, LossContext  # noqa: F401
