"""Utilities: stream/event wrappers, tracing, topology checks, benchmarking helpers."""
from .event import EventHandle, EventOverlap  # noqa: F401
