"""Pure-PyTorch reference semantics (CPU oracle) of every collective."""
from . import oracle  # noqa: F401
