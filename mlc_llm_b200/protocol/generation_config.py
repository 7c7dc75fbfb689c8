"""Low-level generation options passed to the engine (reference: ``protocol/generation_config.py``)."""
from typing import Dict, List, Optional

from pydantic import BaseModel

from .debug_protocol import DebugConfig
from .openai_api_protocol import RequestResponseFormat


class GenerationConfig(BaseModel):
    n: int = 1
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    repetition_penalty: Optional[float] = None
    logprobs: bool = False
    top_logprobs: int = 0
    logit_bias: Optional[Dict[int, float]] = None
    max_tokens: Optional[int] = -1
    seed: Optional[int] = None
    stop_strs: Optional[List[str]] = None
    stop_token_ids: Optional[List[int]] = None
    response_format: Optional[RequestResponseFormat] = None
    debug_config: Optional[DebugConfig] = None
