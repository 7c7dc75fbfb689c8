"""OpenAI-compatible request / response models.

Field lists and validation rules follow the reference's ``protocol/openai_api_protocol.py``
(:56-447): penalties in [-2, 2], logit bias in [-100, 100] with integer keys, ``top_logprobs`` in
[0, 20] and only with ``logprobs``, ``stream_options`` only with ``stream``, system message only in
first position, ``best_of == 1`` only.
"""
# pylint: disable=missing-class-docstring
import json
import time
from typing import Any, Dict, List, Literal, Optional, Tuple, Union

import uuid
from pydantic import BaseModel, Field, field_validator, model_validator

from .debug_protocol import DebugConfig
from .error_protocol import BadRequestError


def _short_id() -> str:
    return uuid.uuid4().hex[:22]


# ------------------------------------------------------------------------------ shared pieces
class ListResponse(BaseModel):
    object: str = "list"
    data: List[Any]


class TopLogProbs(BaseModel):
    token: str
    logprob: float
    bytes: Optional[List[int]]


class LogProbsContent(BaseModel):
    token: str
    logprob: float
    bytes: Optional[List[int]]
    top_logprobs: List[TopLogProbs] = []


class LogProbs(BaseModel):
    content: List[LogProbsContent]


class CompletionLogProbs(BaseModel):
    """Log-probabilities in the layout of the legacy completions API (``logprobs=<int>``): parallel lists
    over the generated tokens (reference: ``protocol/openai_api_protocol.py:47-53``)."""

    text_offset: Optional[List[int]] = None  # offset of each token in the completion text
    token_logprobs: List[float]
    tokens: List[str]
    top_logprobs: List[Dict[str, float]]


COMPLETION_MAX_TOP_LOGPROBS = 5


class CompletionUsage(BaseModel):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0
    extra: Optional[Dict[str, Any]] = None


class StreamOptions(BaseModel):
    include_usage: Optional[bool] = None


class RequestResponseFormat(BaseModel):
    type: Literal["text", "json_object"] = "text"
    json_schema: Optional[str] = Field(default=None, alias="schema")

    model_config = {"populate_by_name": True}


# ------------------------------------------------------------------------------ /v1/models
class ModelResponse(BaseModel):
    id: str
    created: int = Field(default_factory=lambda: int(time.time()))
    object: str = "model"
    owned_by: str = "MLC-LLM"


# ------------------------------------------------------------------------------ /v1/embeddings
class EmbeddingRequest(BaseModel):
    input: Union[str, List[int], List[str], List[List[int]]]
    model: Optional[str] = None
    encoding_format: Literal["float", "base64"] = "float"
    dimensions: Optional[int] = None
    user: Optional[str] = None


class EmbeddingObject(BaseModel):
    object: str = "embedding"
    embedding: Union[List[float], str]
    index: int


class EmbeddingUsage(BaseModel):
    prompt_tokens: int = 0
    total_tokens: int = 0


class EmbeddingResponse(BaseModel):
    object: str = "list"
    data: List[EmbeddingObject]
    model: Optional[str] = None
    usage: EmbeddingUsage = Field(default_factory=EmbeddingUsage)


# ------------------------------------------------------------------------------ shared validation
def _check_penalty(name: str, value: Optional[float]) -> Optional[float]:
    if value is not None and (value < -2 or value > 2):
        raise ValueError(f"{name} must be in [-2, 2]")
    return value


def _check_logit_bias(value: Optional[Dict[Any, float]]) -> Optional[Dict[int, float]]:
    if value is None:
        return None
    out: Dict[int, float] = {}
    for token_id, bias in value.items():
        try:
            tid = int(token_id)
        except (TypeError, ValueError) as err:
            raise ValueError(f"logit bias token id {token_id!r} is not an integer") from err
        if tid < 0:
            raise ValueError(f"logit bias token id {tid} must be non-negative")
        if bias < -100 or bias > 100:
            raise ValueError(f"logit bias value {bias} out of range [-100, 100]")
        out[tid] = float(bias)
    return out


# ------------------------------------------------------------------------------ /v1/completions
class CompletionRequest(BaseModel):
    model: Optional[str] = None
    prompt: Union[str, List[int]]
    best_of: int = 1
    echo: bool = False
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    # an integer asks for that many alternatives per token in the legacy layout (``CompletionLogProbs``);
    # ``true`` with ``top_logprobs`` gives the chat layout
    logprobs: Union[bool, int, None] = None
    top_logprobs: int = 0
    legacy_logprobs: bool = Field(default=False, exclude=True)
    logit_bias: Optional[Dict[int, float]] = None
    max_tokens: Optional[int] = None
    n: int = 1
    seed: Optional[int] = None
    stop: Optional[Union[str, List[str]]] = None
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    suffix: Optional[str] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    user: Optional[str] = None
    response_format: Optional[RequestResponseFormat] = None
    debug_config: Optional[DebugConfig] = None

    @field_validator("frequency_penalty", "presence_penalty")
    @classmethod
    def _penalty(cls, v, info):
        return _check_penalty(info.field_name, v)

    @field_validator("logit_bias", mode="before")
    @classmethod
    def _bias(cls, v):
        return _check_logit_bias(v)

    @model_validator(mode="after")
    def _consistency(self):
        if self.logprobs is not None and not isinstance(self.logprobs, bool):
            if self.logprobs < 0 or self.logprobs > COMPLETION_MAX_TOP_LOGPROBS:
                raise ValueError(f'"logprobs" must be in range [0, {COMPLETION_MAX_TOP_LOGPROBS}]')
            object.__setattr__(self, "top_logprobs", int(self.logprobs))
            object.__setattr__(self, "legacy_logprobs", True)
            object.__setattr__(self, "logprobs", True)
        elif self.logprobs is None:
            object.__setattr__(self, "logprobs", False)
        if self.top_logprobs < 0 or self.top_logprobs > 20:
            raise ValueError('"top_logprobs" must be in [0, 20]')
        if not self.logprobs and self.top_logprobs > 0:
            raise ValueError('"logprobs" must be true to use "top_logprobs"')
        if self.stream_options is not None and not self.stream:
            raise ValueError('"stream" must be true to use "stream_options"')
        return self


class CompletionResponseChoice(BaseModel):
    finish_reason: Optional[Literal["stop", "length", "preempt"]] = None
    index: int = 0
    logprobs: Optional[Union[CompletionLogProbs, LogProbs]] = None
    text: str


class CompletionResponse(BaseModel):
    id: str
    choices: List[CompletionResponseChoice]
    created: int = Field(default_factory=lambda: int(time.time()))
    model: Optional[str] = None
    object: str = "text_completion"
    usage: Optional[CompletionUsage] = None


# ------------------------------------------------------------------------------ /v1/chat/completions
class ChatFunction(BaseModel):
    description: Optional[str] = None
    name: str
    parameters: Dict


class ChatTool(BaseModel):
    type: Literal["function"]
    function: ChatFunction


class ChatFunctionCall(BaseModel):
    name: str
    arguments: Union[None, Dict[str, Any]] = None


class ChatToolCall(BaseModel):
    id: str = Field(default_factory=lambda: f"call_{_short_id()}")
    type: Literal["function"]
    function: ChatFunctionCall


class ChatCompletionMessage(BaseModel):
    content: Optional[Union[str, List[Dict]]] = None
    role: Literal["system", "user", "assistant", "tool"]
    name: Optional[str] = None
    tool_calls: Optional[List[ChatToolCall]] = None
    tool_call_id: Optional[str] = None


class ChatCompletionRequest(BaseModel):
    messages: List[ChatCompletionMessage]
    model: Optional[str] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    logprobs: bool = False
    top_logprobs: int = 0
    logit_bias: Optional[Dict[int, float]] = None
    max_tokens: Optional[int] = None
    n: int = 1
    seed: Optional[int] = None
    stop: Optional[Union[str, List[str]]] = None
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    tools: Optional[List[ChatTool]] = None
    tool_choice: Optional[Union[Literal["none", "auto"], Dict]] = None
    user: Optional[str] = None
    response_format: Optional[RequestResponseFormat] = None
    debug_config: Optional[DebugConfig] = None

    @field_validator("frequency_penalty", "presence_penalty")
    @classmethod
    def _penalty(cls, v, info):
        return _check_penalty(info.field_name, v)

    @field_validator("logit_bias", mode="before")
    @classmethod
    def _bias(cls, v):
        return _check_logit_bias(v)

    @model_validator(mode="after")
    def _consistency(self):
        if self.top_logprobs < 0 or self.top_logprobs > 20:
            raise ValueError('"top_logprobs" must be in [0, 20]')
        if not self.logprobs and self.top_logprobs > 0:
            raise ValueError('"logprobs" must be true to use "top_logprobs"')
        if self.stream_options is not None and not self.stream:
            raise ValueError('"stream" must be true to use "stream_options"')
        special = self.debug_config is not None and self.debug_config.special_request is not None
        if special and not (self.stream and self.stream_options is not None
                            and self.stream_options.include_usage):
            raise ValueError("special requests need stream=True and stream_options.include_usage=True")
        return self

    def check_message_validity(self) -> None:
        """System message only first; list content only for user; no assistant tool_calls input."""
        for i, message in enumerate(self.messages):
            if message.role == "system" and i != 0:
                raise BadRequestError(
                    f"System prompt at position {i} in the message list is invalid.")
            if message.tool_call_id is not None and message.role != "tool":
                raise BadRequestError("Non-tool message having `tool_call_id` is invalid.")
            if isinstance(message.content, list) and message.role != "user":
                raise BadRequestError("Non-user message having a list of content is invalid.")
            if message.tool_calls is not None:
                if message.role != "assistant":
                    raise BadRequestError("Non-assistant message having `tool_calls` is invalid.")
                raise BadRequestError("Assistant message having `tool_calls` is not supported yet.")

    def check_function_call_usage(self, conv_template) -> None:
        """Wire ``tools`` / ``tool_choice`` into the conversation template's function string."""
        if self.tools is None or (isinstance(self.tool_choice, str) and self.tool_choice == "none"):
            conv_template.use_function_calling = False
            return
        if isinstance(self.tool_choice, dict):
            if self.tool_choice.get("type") != "function":
                raise BadRequestError("Only 'function' tool choice is supported")
            if "function" not in self.tool_choice or "name" not in self.tool_choice["function"]:
                raise BadRequestError("Invalid tool choice: missing function name")
            name = self.tool_choice["function"]["name"]
            for tool in self.tools:
                if tool.function.name == name:
                    conv_template.use_function_calling = True
                    conv_template.function_string = tool.function.model_dump_json(by_alias=True)
                    return
            raise BadRequestError(f"The tool_choice function {name} is not found in the tools list")
        if isinstance(self.tool_choice, str) and self.tool_choice != "auto":
            raise BadRequestError(f"Invalid tool_choice value: {self.tool_choice}")
        fns = []
        for tool in self.tools:
            if tool.type != "function":
                raise BadRequestError("Only 'function' tool type is supported")
            fns.append(tool.function.model_dump(by_alias=True))
        conv_template.use_function_calling = True
        conv_template.function_string = json.dumps(fns)


class ChatCompletionResponseChoice(BaseModel):
    finish_reason: Optional[Literal["stop", "length", "tool_calls", "error"]] = None
    index: int = 0
    message: ChatCompletionMessage
    logprobs: Optional[LogProbs] = None


class ChatCompletionStreamResponseChoice(BaseModel):
    finish_reason: Optional[Literal["stop", "length", "tool_calls", "error"]] = None
    index: int = 0
    delta: ChatCompletionMessage
    logprobs: Optional[LogProbs] = None


class ChatCompletionResponse(BaseModel):
    id: str
    choices: List[ChatCompletionResponseChoice]
    created: int = Field(default_factory=lambda: int(time.time()))
    model: Optional[str] = None
    system_fingerprint: str = ""
    object: Literal["chat.completion"] = "chat.completion"
    usage: Optional[CompletionUsage] = None


class ChatCompletionStreamResponse(BaseModel):
    id: str
    choices: List[ChatCompletionStreamResponseChoice]
    created: int = Field(default_factory=lambda: int(time.time()))
    model: Optional[str] = None
    system_fingerprint: str = ""
    object: Literal["chat.completion.chunk"] = "chat.completion.chunk"
    usage: Optional[CompletionUsage] = None


# ------------------------------------------------------------------------------ helpers
def openai_api_get_unsupported_fields(request: Union[CompletionRequest, ChatCompletionRequest]) -> List[str]:
    """Fields the engine accepts syntactically but ignores (reported as a warning)."""
    unsupported = []
    if isinstance(request, CompletionRequest):
        if request.best_of != 1:
            unsupported.append("best_of")
        if request.suffix is not None:
            unsupported.append("suffix")
    return unsupported


def openai_api_get_generation_config(request: Union[CompletionRequest, ChatCompletionRequest]) -> Dict[str, Any]:
    """Extract the generation options of an OpenAI request as keyword arguments."""
    kwargs: Dict[str, Any] = {}
    for name in ("n", "temperature", "top_p", "top_k", "max_tokens", "frequency_penalty",
                 "presence_penalty", "logit_bias", "seed", "response_format", "debug_config"):
        kwargs[name] = getattr(request, name)
    kwargs["logprobs"] = request.logprobs
    kwargs["top_logprobs"] = request.top_logprobs
    if kwargs["max_tokens"] is None:
        kwargs["max_tokens"] = -1
    if request.stop is not None:
        kwargs["stop_strs"] = [request.stop] if isinstance(request.stop, str) else list(request.stop)
    return kwargs
