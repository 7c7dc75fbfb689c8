"""A generation request as handed to the synchronous engine (reference:
``python/mlc_llm/serve/request.py``: ``request_id``, ``inputs``, ``generation_config``)."""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Union

from .data import Data


@dataclasses.dataclass
class Request:
    """``inputs`` is a list of ``TextData`` / ``TokenData`` / ``ImageData`` (or plain strings and token
    lists); ``generation_config`` is a ``GenerationConfig`` or its dict form."""

    request_id: str
    inputs: List[Union[Data, str, List[int]]]
    generation_config: Union[Dict[str, Any], Any]
