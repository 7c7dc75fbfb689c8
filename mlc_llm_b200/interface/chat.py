"""Interactive chat REPL (reference: ``python/mlc_llm/interface/chat.py:1-311``).

Commands: ``/help``, ``/exit``, ``/stats``, ``/metrics``, ``/reset``, ``/set k=v;k=v`` (temperature,
top_p, max_tokens, presence_penalty, frequency_penalty, n, stop...).  ``Ctrl+C`` while generating
aborts the current reply."""

from __future__ import annotations

import dataclasses
import json
import sys
from typing import Any, Callable, Dict, List, Optional


@dataclasses.dataclass
class ChatCompletionOverride:
    """Sampling options changed with ``/set`` or ``--overrides``."""

    temperature: Optional[float] = None
    top_p: Optional[float] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    max_tokens: Optional[int] = None
    seed: Optional[int] = None
    stop: Optional[List[str]] = None

    @staticmethod
    def from_str(source: str) -> "ChatCompletionOverride":
        out = ChatCompletionOverride()
        types = {"temperature": float, "top_p": float, "frequency_penalty": float, "presence_penalty": float,
                 "max_tokens": int, "seed": int}
        for item in filter(None, (x.strip() for x in source.split(";"))):
            if "=" not in item:
                raise ValueError(f"{item!r} is not of the form key=value")
            k, v = (x.strip() for x in item.split("=", 1))
            if k == "stop":
                out.stop = [s for s in v.split(",") if s]
            elif k in types:
                setattr(out, k, types[k](v))
            else:
                raise ValueError(f"unknown option {k!r}")
        return out

    def merged(self, other: "ChatCompletionOverride") -> "ChatCompletionOverride":
        d = dataclasses.asdict(self)
        d.update({k: v for k, v in dataclasses.asdict(other).items() if v is not None})
        return ChatCompletionOverride(**d)


HELP = """You can use the following special commands:
  /help               print the special commands
  /exit               quit the cli
  /stats              print out stats of last request (token/sec)
  /metrics            print out full engine metrics
  /reset              restart a fresh chat
  /set [overrides]    override settings in the generation config. For example,
                      `/set temperature=0.5;top_p=0.8;seed=23;max_tokens=100;stop=str1,str2`
                      Note: Separate stop words in the `stop` option with commas (,).
  Multi-line input: Use escape+enter to start a new line.
"""


class ChatState:
    """Conversation history plus the loop that talks to the engine."""

    def __init__(self, engine, write: Callable[[str], None] = None):
        self.engine = engine
        self.history: List[Dict[str, Any]] = []
        self.overrides = ChatCompletionOverride()
        self.last_usage: Optional[Dict[str, Any]] = None
        self.write = write or (lambda s: (sys.stdout.write(s), sys.stdout.flush()))

    def reset(self) -> None:
        self.history.clear()
        self.last_usage = None

    def stats(self) -> str:
        if not self.last_usage:
            return "no request has run yet"
        extra = self.last_usage.get("extra") or {}
        parts = [f"prompt_tokens: {self.last_usage.get('prompt_tokens')}",
                 f"completion_tokens: {self.last_usage.get('completion_tokens')}"]
        for key in ("prefill_tokens_per_s", "decode_tokens_per_s", "ttft_s", "end_to_end_latency_s"):
            if key in extra:
                parts.append(f"{key}: {extra[key]:.3f}")
        return ", ".join(parts)

    def generate(self, prompt: str) -> str:
        self.history.append({"role": "user", "content": prompt})
        kwargs = {k: v for k, v in dataclasses.asdict(self.overrides).items() if v is not None}
        text = ""
        stream = self.engine.chat.completions.create(messages=self.history, stream=True,
                                                     stream_options={"include_usage": True}, **kwargs)
        try:
            for chunk in stream:
                if chunk.usage is not None:
                    self.last_usage = chunk.usage.model_dump()
                for choice in chunk.choices:
                    delta = choice.delta.content or ""
                    text += delta
                    self.write(delta)
        except KeyboardInterrupt:
            stream.close()
            self.write("\n[interrupted]")
        self.write("\n")
        self.history.append({"role": "assistant", "content": text})
        return text

    def handle(self, line: str) -> bool:
        """Process one input line; returns False when the REPL should stop."""
        cmd = line.strip()
        if cmd == "/exit":
            return False
        if cmd == "/help":
            self.write(HELP)
        elif cmd == "/stats":
            self.write(self.stats() + "\n")
        elif cmd == "/metrics":
            self.write(json.dumps(self.engine.metrics().metrics, indent=2) + "\n")
        elif cmd == "/reset":
            self.reset()
            self.write("[chat reset]\n")
        elif cmd.startswith("/set"):
            try:
                self.overrides = self.overrides.merged(ChatCompletionOverride.from_str(cmd[4:].strip()))
            except ValueError as err:
                self.write(f"error: {err}\n")
        elif cmd:
            self.generate(line)
        return True


def chat(model: str, device: str = "auto", model_lib: Optional[str] = None,
         overrides: Optional[ChatCompletionOverride] = None, engine=None, read: Callable[[], str] = None) -> None:
    from ..serve.engine import MLCEngine  # pylint: disable=import-outside-toplevel

    own = engine is None
    engine = engine or MLCEngine(model, device, model_lib=model_lib, mode="interactive")
    state = ChatState(engine)
    if overrides is not None:
        state.overrides = overrides
    state.write(HELP)
    read = read or (lambda: input(">>> "))
    try:
        while True:
            try:
                line = read()
            except (EOFError, KeyboardInterrupt):
                break
            if not state.handle(line):
                break
    finally:
        if own:
            engine.terminate()
