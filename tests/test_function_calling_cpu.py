"""Function calling: ``tools`` enter the prompt through the conversation template's function placeholder, and
generated text of the form ``[f(a=1)]`` or a JSON call object comes back as ``tool_calls`` (reference behaviour:
``python/mlc_llm/serve/engine_base.py`` function-call post-processing, ``tests/python/serve/server/
test_server_function_call.py``)."""
import json

import pytest

from mlc_llm_b200.protocol import openai_api_protocol as openai
from mlc_llm_b200.protocol.error_protocol import BadRequestError
from mlc_llm_b200.serve import engine_base
from mlc_llm_b200.serve.config import EngineConfig

TOOLS = [{"type": "function", "function": {
    "name": "get_current_weather", "description": "Get the current weather in a given location",
    "parameters": {"type": "object", "properties": {"location": {"type": "string"},
                                                     "unit": {"type": "string", "enum": ["celsius", "fahrenheit"]}},
                   "required": ["location"]}}},
    {"type": "function", "function": {"name": "get_time", "description": "time of day",
                                      "parameters": {"type": "object", "properties": {"zone": {"type": "string"}}}}}]


def test_call_text_forms_are_parsed():
    f = engine_base.convert_function_str_to_json
    assert f("[get_current_weather(location='Paris', unit='celsius')]") == [
        {"name": "get_current_weather", "arguments": {"location": "Paris", "unit": "celsius"}}]
    assert f(" get_time(zone='UTC') ") == [{"name": "get_time", "arguments": {"zone": "UTC"}}]
    assert f("[a(x=-3, y=[1, 2.5], z={'k': True}), b()]") == [
        {"name": "a", "arguments": {"x": -3, "y": [1, 2.5], "z": {"k": True}}}, {"name": "b", "arguments": {}}]
    assert f('{"name": "get_time", "arguments": {"zone": "CET"}}') == [{"name": "get_time", "arguments": {"zone": "CET"}}]
    assert f('[{"name": "a", "parameters": {"q": 1}}, {"name": "b", "arguments": {}}]') == [
        {"name": "a", "arguments": {"q": 1}}, {"name": "b", "arguments": {}}]
    assert f("The weather is nice today.") == []
    assert f("[1, 2, 3]") == []
    assert f("f(x=__import__('os').system('true'))") == []  # a call inside an argument is not evaluated, the call is dropped


def test_generated_calls_become_tool_calls_and_flip_the_finish_reason():
    finish = ["stop", "length"]
    ok, calls = engine_base.process_function_call_output(
        ["[get_time(zone='UTC')]", '{"name": "get_current_weather", "arguments": {"location": "Oslo"}}'], finish)
    assert ok and finish == ["tool_calls", "length"]
    assert calls[0][0].function.name == "get_time" and calls[0][0].function.arguments == {"zone": "UTC"}
    assert calls[1][0].function.arguments == {"location": "Oslo"}
    finish = ["stop", "stop"]
    ok, _ = engine_base.process_function_call_output(["[get_time(zone='UTC')]", "just text"], finish)
    assert not ok  # one plain answer: the response keeps the texts


def _runtime(template):
    from mlc_llm_b200.serve.engine_base import EngineRuntime
    import torch

    return EngineRuntime(EngineConfig(model=f"random://tiny-llama?quant=q0f32&seed=1&conv_template={template}",
                                      mode="local"), torch.device("cpu"))


def test_tools_reach_the_prompt_through_the_template_placeholder():
    rt = _runtime("gorilla")
    req = openai.ChatCompletionRequest(messages=[{"role": "user", "content": "Weather in Paris?"}], tools=TOOLS)
    inputs, _gen, use_fn, _n = engine_base.process_chat_completion_request(req, "r0", rt, 4096)
    text = rt.tokenizer.decode([int(t) for t in inputs[0]])
    assert use_fn
    assert "<<question>> Weather in Paris? <<function>> " in text
    listed = json.loads(text.split("<<function>> ", 1)[1].split("\n", 1)[0])
    assert [fn["name"] for fn in listed] == ["get_current_weather", "get_time"]
    assert listed[0]["parameters"]["required"] == ["location"]
    # a named tool_choice passes that function alone
    req = openai.ChatCompletionRequest(messages=[{"role": "user", "content": "Time?"}], tools=TOOLS,
                                       tool_choice={"type": "function", "function": {"name": "get_time"}})
    inputs, _gen, use_fn, _n = engine_base.process_chat_completion_request(req, "r1", rt, 4096)
    text = rt.tokenizer.decode([int(t) for t in inputs[0]])
    assert use_fn and '"name":"get_time"' in text.replace(" ", "") and "get_current_weather" not in text
    # tool_choice "none", or no tools: no function string, the placeholder disappears
    for kw in (dict(tools=TOOLS, tool_choice="none"), {}):
        req = openai.ChatCompletionRequest(messages=[{"role": "user", "content": "Hi"}], **kw)
        inputs, _gen, use_fn, _n = engine_base.process_chat_completion_request(req, "r2", rt, 4096)
        text = rt.tokenizer.decode([int(t) for t in inputs[0]])
        assert not use_fn and "get_time" not in text and "{function_string}" not in text


def test_invalid_tool_choices_are_bad_requests():
    rt = _runtime("gorilla")
    for choice in ({"type": "function", "function": {"name": "missing"}}, {"type": "retrieval"},
                   {"type": "function"}):
        req = openai.ChatCompletionRequest(messages=[{"role": "user", "content": "x"}], tools=TOOLS, tool_choice=choice)
        with pytest.raises(BadRequestError):
            engine_base.process_chat_completion_request(req, "r", rt, 4096)
    import pydantic

    with pytest.raises(pydantic.ValidationError):  # only "none", "auto" or a function object pass the schema
        openai.ChatCompletionRequest(messages=[{"role": "user", "content": "x"}], tools=TOOLS, tool_choice="required")


def test_non_streaming_response_carries_tool_calls():
    """The accumulator of a non-streaming chat request: texts that parse as calls come back as ``tool_calls`` with
    ``content = None``; otherwise the text is returned."""
    from mlc_llm_b200.serve.engine import _Accumulator

    class Item:
        def __init__(self, index, text, finish):
            self.index, self.delta_text, self.finish_reason = index, text, finish
            self.delta_logprob_json_strs, self.usage_json = [], None

    acc = _Accumulator(1)
    acc.add([Item(0, "[get_current_weather(", None), Item(0, "location='Paris')]", "stop")])
    acc.usage_json = json.dumps({"prompt_tokens": 5, "completion_tokens": 9, "total_tokens": 14})
    resp = acc.chat_response("id0", "m", use_fn=True)
    choice = resp.choices[0]
    assert choice.finish_reason == "tool_calls" and choice.message.content is None
    assert choice.message.tool_calls[0].function.name == "get_current_weather"
    assert choice.message.tool_calls[0].function.arguments == {"location": "Paris"}
    plain = _Accumulator(1)
    plain.add([Item(0, "It is sunny.", "stop")])
    plain.usage_json = acc.usage_json
    resp = plain.chat_response("id1", "m", use_fn=True)
    assert resp.choices[0].finish_reason == "stop" and resp.choices[0].message.content == "It is sunny."
