"""Logging, errors, configuration and device timing helpers."""
from .errors import CamError, MoeCommTimeout, RecvOverflow, raise_for_status  # noqa: F401
from .log import get_logger  # noqa: F401
from .config import CamConfig  # noqa: F401
from .nvtx import nvtx_range  # noqa: F401
from .timing import ClockSampler, device_time_ms, flush_l2  # noqa: F401
