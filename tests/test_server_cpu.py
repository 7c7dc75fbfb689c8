"""REST server over a tiny random model on CPU: OpenAI endpoints, SSE framing, metrics, debug."""
import json
import socket

import pytest
import requests

from mlc_llm_b200.serve.server import PopenServer

MODEL = "random://tiny-llama?quant=q0f32&seed=3"


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def server():
    srv = PopenServer(MODEL, "cpu", mode="local", port=_port(), enable_debug=True, enable_tracing=True,
                      api_key="sekret")
    srv.start(timeout=180)
    yield srv
    srv.terminate()


H = {"Authorization": "Bearer sekret"}


def test_models_and_auth(server):
    r = requests.get(server.base_url + "/v1/models", headers=H, timeout=30)
    assert r.status_code == 200 and r.json()["data"][0]["id"] == MODEL
    assert requests.get(server.base_url + "/v1/models", timeout=30).status_code == 401


def test_completion_and_usage(server):
    body = {"model": MODEL, "prompt": [5, 6, 7, 8, 9], "max_tokens": 6, "temperature": 0.0,
            "debug_config": {"ignore_eos": True}}
    r = requests.post(server.base_url + "/v1/completions", json=body, headers=H, timeout=120)
    assert r.status_code == 200, r.text
    out = r.json()
    assert out["object"] == "text_completion"
    assert out["usage"]["prompt_tokens"] == 5 and out["usage"]["completion_tokens"] == 6
    assert out["choices"][0]["finish_reason"] == "length"
    # same request again is deterministic
    r2 = requests.post(server.base_url + "/v1/completions", json=body, headers=H, timeout=120)
    assert r2.json()["choices"][0]["text"] == out["choices"][0]["text"]


def test_chat_stream_sse(server):
    body = {"model": MODEL, "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 5,
            "stream": True, "stream_options": {"include_usage": True}, "n": 2, "seed": 1}
    with requests.post(server.base_url + "/v1/chat/completions", json=body, headers=H, stream=True,
                       timeout=120) as r:
        assert r.status_code == 200
        assert r.headers["content-type"].startswith("text/event-stream")
        lines = [ln.decode() for ln in r.iter_lines() if ln]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(ln[len("data: "):]) for ln in lines[:-1]]
    assert all(c["object"] == "chat.completion.chunk" for c in chunks)
    finished = {ch["index"] for c in chunks for ch in c["choices"] if ch["finish_reason"]}
    assert finished == {0, 1}
    assert chunks[-1]["usage"]["completion_tokens"] > 0 and chunks[-1]["choices"] == []


def test_client_disconnects_abort_their_requests(server):
    """Streams that the client closes after two events, beside streams read to the end: the server aborts the
    abandoned generations (their tokens stop being produced: the completion counter settles far below what they
    asked for) and keeps serving."""
    import concurrent.futures as cf
    import time

    def metric(name):
        text = requests.get(server.base_url + "/metrics", timeout=30).text
        return float(next(ln.split()[-1] for ln in text.splitlines() if ln.startswith(name)))

    before = metric("completion_tokens_sum")

    def stream(i):
        body = {"model": MODEL, "prompt": f"request {i}", "max_tokens": 2000 if i % 2 else 12, "stream": True,
                "temperature": 0.0, "debug_config": {"ignore_eos": True}}
        seen = 0
        with requests.post(server.base_url + "/v1/completions", json=body, headers=H, stream=True, timeout=120) as r:
            assert r.status_code == 200
            for ln in r.iter_lines():
                if not ln:
                    continue
                seen += 1
                if i % 2 and seen == 2:
                    return "left"               # leaving the block closes the connection
                if ln == b"data: [DONE]":
                    return "done"
        return "eof"

    with cf.ThreadPoolExecutor(6) as pool:
        results = list(pool.map(stream, range(6)))
    assert results == ["done", "left"] * 3
    settled, last = None, -1.0
    for _ in range(60):                         # the aborts land within a few engine steps
        now = metric("completion_tokens_sum")
        if now == last:
            settled = now
            break
        last = now
        time.sleep(0.5)
    assert settled is not None and settled - before < 3 * 12 + 3 * 400
    r = requests.post(server.base_url + "/v1/completions", headers=H, timeout=60,
                      json={"model": MODEL, "prompt": "still there?", "max_tokens": 3})
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 3


def test_bad_request_is_400(server):
    body = {"model": MODEL, "messages": [{"role": "user", "content": "x"}], "max_tokens": 4, "temperature": -1}
    r = requests.post(server.base_url + "/v1/chat/completions", json=body, headers=H, timeout=60)
    assert r.status_code in (400, 422)


def test_metrics_and_debug(server):
    r = requests.get(server.base_url + "/metrics", timeout=30)
    assert r.status_code == 200 and "prefill_tokens_sum" in r.text
    r = requests.post(server.base_url + "/debug/dump_event_trace", json={"model": MODEL}, timeout=30)
    assert r.status_code == 200 and isinstance(r.json(), (list, dict))
    r = requests.post(server.base_url + "/debug/dump_engine_metrics", json={"model": MODEL}, timeout=30)
    assert r.status_code == 200 and "engine_prefill_time_sum" in r.json()
    r = requests.post(server.base_url + "/debug/reset_engine", json={"model": MODEL}, timeout=30)
    assert r.status_code == 200


def test_json_mode_over_rest(server):
    """response_format with a JSON schema: the grammar constrains decoding (jump-forward by default) and
    the usage block reports the forced tokens."""
    schema = json.dumps({"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"]})
    body = {"model": MODEL, "messages": [{"role": "user", "content": "say yes"}], "max_tokens": 24,
            "temperature": 0.0, "response_format": {"type": "json_object", "schema": schema}}
    r = requests.post(server.base_url + "/v1/chat/completions", json=body, headers=H, timeout=120)
    assert r.status_code == 200, r.text
    out = r.json()
    text = out["choices"][0]["message"]["content"]
    assert text.lstrip().startswith("{")   # the grammar admits white space after the brace
    if out["choices"][0]["finish_reason"] == "stop":
        assert json.loads(text)["ok"] in (True, False)
    assert "jump_forward_tokens" in out["usage"]["extra"]


def test_image_request_over_rest():
    """A LLaVA-type model behind the REST server takes `image_url` content parts (data URLs)."""
    import base64
    import io

    import numpy as np
    from PIL import Image

    model = "random://tiny-llava?quant=q0f32&seed=2"
    srv = PopenServer(model, "cpu", mode="local", port=_port())
    srv.start(timeout=180)
    try:
        img = Image.fromarray((np.random.default_rng(0).random((30, 30, 3)) * 255).astype(np.uint8))
        buf = io.BytesIO()
        img.save(buf, format="PNG")
        url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
        mk = lambda content: {"model": model, "messages": [{"role": "user", "content": content}],
                              "max_tokens": 4, "temperature": 0.0}
        plain = requests.post(srv.base_url + "/v1/chat/completions", json=mk("describe"), timeout=120).json()
        with_img = requests.post(srv.base_url + "/v1/chat/completions", timeout=120, json=mk(
            [{"type": "text", "text": "describe"}, {"type": "image_url", "image_url": {"url": url}}])).json()
        assert with_img["usage"]["prompt_tokens"] == plain["usage"]["prompt_tokens"] + 4 + 1
        assert with_img["usage"]["completion_tokens"] == 4
    finally:
        srv.terminate()
