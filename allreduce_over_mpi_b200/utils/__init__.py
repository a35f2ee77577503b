from .clocks import ClockSampler  # noqa: F401
from .timing import Timer, cuda_time, flush_l2  # noqa: F401
from . import log  # noqa: F401
