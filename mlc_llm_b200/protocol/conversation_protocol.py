"""Conversation template model and prompt rendering.

Semantics follow the reference's ``protocol/conversation_protocol.py:23-208``: the prompt is the
system template followed, per message, by ``role + role_content_sep + templated content + sep``
(``seps[1]`` after assistant messages, ``seps[0]`` otherwise); a ``None`` content renders the bare
generation prompt ``role + role_empty_sep``; the last ``{function_string}`` placeholder receives the
tool description.
"""
import re
from enum import Enum
from typing import Any, Dict, List, Optional, Tuple, Union

from pydantic import BaseModel, Field, field_validator


class MessagePlaceholders(Enum):
    SYSTEM = "{system_message}"
    USER = "{user_message}"
    ASSISTANT = "{assistant_message}"
    TOOL = "{tool_message}"
    FUNCTION = "{function_string}"


_THINK_RE = re.compile(r"<think>.*?</think>\s*", re.DOTALL)


def _strip_reasoning_in_history(messages):
    """Drop ``<think>...</think>`` from assistant turns that precede the last user turn."""
    last_user = max((i for i, (role, _) in enumerate(messages) if role == "user"), default=-1)
    out = []
    for i, (role, content) in enumerate(messages):
        if role == "assistant" and i < last_user and isinstance(content, str):
            content = _THINK_RE.sub("", content)
        out.append((role, content))
    return out


def _merge_adjacent_strings(parts: List[Any]) -> List[Any]:
    merged: List[Any] = []
    for part in parts:
        if isinstance(part, str) and merged and isinstance(merged[-1], str):
            merged[-1] += part
        else:
            merged.append(part)
    return merged


class Conversation(BaseModel):
    """A conversation template plus the message history to render."""

    name: Optional[str] = None
    system_template: str = MessagePlaceholders.SYSTEM.value
    system_message: str = ""
    system_prefix_token_ids: Optional[List[int]] = None
    add_role_after_system_message: bool = True
    roles: Dict[str, str]
    role_templates: Dict[str, str]
    messages: List[Tuple[str, Optional[Union[str, List[Dict]]]]] = Field(default_factory=list)
    seps: List[str]
    role_content_sep: str = ""
    role_empty_sep: str = ""
    stop_str: List[str] = Field(default_factory=list)
    stop_token_ids: List[int] = Field(default_factory=list)
    strip_reasoning_in_history: bool = False
    function_string: str = ""
    use_function_calling: bool = False

    def __init__(self, role_templates: Optional[Dict[str, str]] = None, **kwargs):
        templates = {
            "user": MessagePlaceholders.USER.value,
            "assistant": MessagePlaceholders.ASSISTANT.value,
            "tool": MessagePlaceholders.TOOL.value,
        }
        if role_templates is not None:
            templates.update(role_templates)
        super().__init__(role_templates=templates, **kwargs)

    @field_validator("seps")
    @classmethod
    def _check_seps(cls, seps: List[str]) -> List[str]:
        if len(seps) == 0 or len(seps) > 2:
            raise ValueError("seps should have size 1 or 2.")
        return seps

    def to_json_dict(self) -> Dict[str, Any]:
        return self.model_dump(by_alias=True, exclude_none=True)

    @classmethod
    def from_json_dict(cls, json_dict: Dict[str, Any]) -> "Conversation":
        return Conversation.model_validate(json_dict)

    def as_prompt(self, config=None) -> List[Any]:
        """Render to a list whose items are strings or image payloads (``ImageData``)."""
        from ..serve import data  # pylint: disable=import-outside-toplevel

        system_msg = self.system_template.replace(MessagePlaceholders.SYSTEM.value, self.system_message)
        seps = list(self.seps) * 2 if len(self.seps) == 1 else list(self.seps)
        parts: List[Any] = [system_msg] if system_msg != "" else []
        history = _strip_reasoning_in_history(self.messages) if self.strip_reasoning_in_history \
            else self.messages
        for i, (role, content) in enumerate(history):
            if role not in self.roles:
                raise ValueError(f'Role "{role}" is not a supported role in {list(self.roles)}')
            sep = seps[1] if role == "assistant" else seps[0]
            if content is None:
                parts.append(self.roles[role] + self.role_empty_sep)
                continue
            omit_prefix = (not self.add_role_after_system_message) and system_msg != "" and i == 0
            prefix = "" if omit_prefix else self.roles[role] + self.role_content_sep
            placeholder = MessagePlaceholders[role.upper()].value
            if isinstance(content, str):
                parts.append(prefix + self.role_templates[role].replace(placeholder, content) + sep)
                continue
            parts.append(prefix)
            for item in content:
                if not isinstance(item, dict) or "type" not in item:
                    raise ValueError("Content should be a string or a list of typed dicts")
                if item["type"] == "text":
                    parts.append(self.role_templates[role].replace(placeholder, item["text"]))
                elif item["type"] == "image_url":
                    if config is None:
                        raise ValueError("Model config is required for image inputs")
                    url = item["image_url"]
                    url = url["url"] if isinstance(url, dict) else url
                    parts.append(data.ImageData.from_url(url, config))
                    parts.append("\n")
                else:
                    raise ValueError(f"Unsupported content type: {item['type']}")
            parts.append(sep)
        prompt = _merge_adjacent_strings(parts)
        if prompt and not any(isinstance(p, data.ImageData) for p in prompt):
            head, found, tail = prompt[0].rpartition(MessagePlaceholders.FUNCTION.value)
            if found:
                prompt[0] = head + self.function_string + tail
            prompt[0] = prompt[0].replace(MessagePlaceholders.FUNCTION.value, "")
        return prompt
