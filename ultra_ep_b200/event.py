"""Python face of a recorded CUDA event (the reference's ultra_ep/event.py:10-65 surface)."""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch


class EventHandle:
    """Wraps the native event an asynchronous weight_sync / grad_reduce returns.

    `event` is the native handle (None when the call finished synchronously);
    `extra_tensors` keeps tensors alive until the event has been waited for.
    Usable as a context manager: leaving the block makes the current stream wait.
    """

    def __init__(self, event=None, extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors

    def current_stream_wait(self) -> None:
        assert self.event is not None
        self.event.current_stream_wait()

    def __enter__(self) -> Any:
        return self

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        if self.event is not None:
            self.event.current_stream_wait()
