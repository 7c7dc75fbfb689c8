"""Per-request event trace in Chrome trace format, under the module path the reference uses
(``python/mlc_llm/serve/event_trace_recorder.py``: ``add_event(request_id, event)``, ``dump_json()``)."""

from .._core import EventTraceRecorder

__all__ = ["EventTraceRecorder"]
