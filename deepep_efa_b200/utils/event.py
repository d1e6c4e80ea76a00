"""Stream/event plumbing shared by every collective call.

``EventHandle`` is a CUDA event recorded on a stream at construction; ``EventOverlap`` is the object
the public API returns: ``current_stream_wait()`` makes the caller's stream wait for the communication
kernels, and used as a context manager it does that on exit, so compute issued inside the ``with``
block overlaps the communication.

Reference counterparts: ``EventHandle`` (csrc/event.hpp:9-40) and ``EventOverlap``
(deep_ep/utils.py:10-61).
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch


class EventHandle:
    """A CUDA event recorded on ``stream`` (default: the current stream) when created.

    On a machine without CUDA the handle is inert, which keeps the CPU/gloo backend API-compatible."""

    def __init__(self, stream: Optional["torch.cuda.Stream"] = None, record: bool = True) -> None:
        self.event = None
        if torch.cuda.is_available():
            self.event = torch.cuda.Event(enable_timing=False)
            if record:
                self.event.record(stream if stream is not None else torch.cuda.current_stream())

    def current_stream_wait(self) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)


class EventOverlap:
    """Wrapper returned by every collective; see the module docstring.

    Attributes:
        event: the underlying :class:`EventHandle` (``None`` when the call was synchronous).
        extra_tensors: tensors kept alive until this object dies (their memory may still be in use by
            the communication stream).
    """

    def __init__(self, event: Optional[EventHandle] = None, extra_tensors: Optional[Tuple[Any, ...]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors

    def current_stream_wait(self) -> None:
        if self.event is not None:
            self.event.current_stream_wait()

    def __enter__(self) -> "EventOverlap":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        if self.event is not None:
            self.event.current_stream_wait()
