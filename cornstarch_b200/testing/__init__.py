from .dcgm import DcgmContextManager  # noqa: F401
from .timer import TimerContextManager  # noqa: F401
