"""Symmetric-memory runtime, fused compute+collective kernels, optimizer and
training drivers."""
from .optimizer import FlatAdamW, cosine_lr  # noqa: F401
from .trainer import SyntheticTokens, Trainer  # noqa: F401
from .pipeline import PipelineStage, run_1f1b  # noqa: F401
from .metrics import MetricsSink  # noqa: F401
from .health import Heartbeat, RankFailure, Watchdog  # noqa: F401
