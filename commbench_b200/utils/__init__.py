"""Small shared helpers: configuration, device timing, logging of one JSON line."""
from ..config import Config, get_config  # noqa: F401
from .timing import DeviceTimer, time_ms  # noqa: F401
