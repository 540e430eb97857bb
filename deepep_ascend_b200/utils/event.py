"""Stream-ordering handle returned by every communication call
(parity: deep_ep/utils/event.py:8-96, csrc/utils/event.hpp:10-42)."""
from typing import Any, Callable, Optional, Tuple

import torch


class EventHandle:
    """A CUDA event recorded on the stream that ran a communication kernel, plus the tensors that must
    stay alive until that work is done.  On CPU tensors it is an already-completed placeholder."""

    def __init__(self, stream: Optional['torch.cuda.Stream'] = None, keep_alive: Tuple[Any, ...] = ()):
        self.event = None
        self.keep_alive = keep_alive
        if torch.cuda.is_available() and (stream is not None or torch.cuda.is_initialized()):
            self.event = torch.cuda.Event()
            self.event.record(stream if stream is not None else torch.cuda.current_stream())

    def current_stream_wait(self) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)

    def synchronize(self) -> None:
        if self.event is not None:
            self.event.synchronize()


class EventOverlap:
    """Convenience wrapper: ``event.current_stream_wait()`` or ``with event: ...`` (waits on exit), with an
    optional hook that runs right after the wait (used to finalise lazily materialised outputs)."""

    def __init__(self, event: Optional[EventHandle] = None, extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None,
                 post_wait_hook: Optional[Callable[[], None]] = None):
        self.event = event
        self.extra_tensors = extra_tensors
        self._post_wait_hook = post_wait_hook

    def current_stream_wait(self) -> None:
        if self.event is not None:
            self.event.current_stream_wait()
        if self._post_wait_hook is not None:
            hook, self._post_wait_hook = self._post_wait_hook, None
            hook()

    def __enter__(self) -> 'EventOverlap':
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        if self.event is not None or self._post_wait_hook is not None:
            self.current_stream_wait()
