"""Bodies of the ``/microserving/*`` endpoints (reference: ``protocol/microserving_protocol.py``)."""
from pydantic import BaseModel

from .openai_api_protocol import CompletionRequest


class PrepRecvRequest(CompletionRequest):
    """Ask the decode engine to reserve KV entries ``[0:end)`` of the prompt."""

    end: int


class PrepRecvResponse(BaseModel):
    kv_append_metadata: str
    prefix_matched_length: int


class RemoteSendRequest(CompletionRequest):
    """Ask the prefill engine to compute KV ``[begin:end)`` and push it to the receiver."""

    begin: int
    end: int
    kv_addr_info: str
    recv_rank: int


class RemoteSendResponse(BaseModel):
    pass


class StartGenerateRequest(CompletionRequest):
    """Start decoding from position ``begin`` on the engine that received the KV."""

    begin: int
