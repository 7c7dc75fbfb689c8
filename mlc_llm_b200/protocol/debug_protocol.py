"""Per-request debug options (reference: ``protocol/debug_protocol.py:8-41``)."""
from typing import Literal, Optional

from pydantic import BaseModel


class DisaggConfig(BaseModel):
    """Prefill/decode disaggregation step of a request.

    ``kv_window_begin`` / ``kv_window_end`` select the KV range handled by this step and accept
    negative (from-the-end) indices; ``kv_append_metadata`` is an opaque base64 payload produced by
    the receiving engine's ``prepare_receive`` step.
    """

    kind: Optional[Literal["prepare_receive", "remote_send", "start_generation"]] = None
    kv_append_metadata: Optional[str] = None
    kv_window_begin: Optional[int] = None
    kv_window_end: Optional[int] = None
    dst_group_offset: Optional[int] = None


class DebugConfig(BaseModel):
    ignore_eos: bool = False
    pinned_system_prompt: bool = False
    special_request: Optional[Literal["query_engine_metrics"]] = None
    grammar_execution_mode: Literal["constraint", "jump_forward"] = "jump_forward"
    disagg_config: Optional[DisaggConfig] = None
