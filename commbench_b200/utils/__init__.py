"""Small shared helpers: configuration, device timing and latency statistics, CUDA-graph
capture, tracing."""
from ..config import Config, get_config  # noqa: F401
from .timing import DeviceTimer, latency_stats, time_each_ms, time_ms  # noqa: F401
