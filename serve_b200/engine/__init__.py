from .engine import Engine  # noqa: F401
from .runtime import Runtime  # noqa: F401
from .step import FROM_DEVICE, BatchShape, StepContext, StepEntry, Stepper  # noqa: F401
