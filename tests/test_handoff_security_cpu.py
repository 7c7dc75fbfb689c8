"""The KV hand-off descriptor and the debug options are untrusted input on a server: a forged or
altered descriptor, a slot outside the pool, and debug fields on a non-debug server must all be
refused before they reach the engine or a kernel."""
import base64
import json
import os
import pickle
import socket

import numpy as np
import pytest
import requests
import torch

from mlc_llm_b200.serve import kv_handoff
from mlc_llm_b200.serve.executor import ModelExecutor
from mlc_llm_b200.serve.server import PopenServer

MODEL = "random://tiny-llama?quant=q0f32&seed=3"


class _Holder:
    pass


def _executor(fill: float) -> ModelExecutor:
    m = _Holder()
    m.kv_pages = torch.full((2, 4, 2, 2, 16, 8), fill, dtype=torch.float32)
    ex = ModelExecutor.__new__(ModelExecutor)
    ex.models, ex.device, ex.comm = [m], torch.device("cpu"), None
    return ex


def test_signed_payload_round_trip_copies_rows():
    a, b = _executor(0.0), _executor(-1.0)
    a.models[0].kv_pages.copy_(torch.randn_like(a.models[0].kv_pages))
    meta = kv_handoff.encode_payload(b.kv_export(0), [5, 63], 0, 2)
    a.send_kv(0, np.asarray([1, 17], dtype=np.int32), meta)
    src, dst = a.models[0].kv_pages, b.models[0].kv_pages
    assert torch.equal(dst[:, 0, :, :, 5, :], src[:, 0, :, :, 1, :])
    assert torch.equal(dst[:, 3, :, :, 15, :], src[:, 1, :, :, 1, :])


class _Boom:
    """Unpickling this would create the marker file; the descriptor parser must never get that far."""

    def __init__(self, path):
        self.path = path

    def __reduce__(self):
        return (open, (self.path, "w"))


def test_forged_descriptors_are_rejected_without_running_anything(tmp_path):
    a, b = _executor(0.0), _executor(-1.0)
    marker = str(tmp_path / "pwned")
    pool = b.kv_export(0)
    legacy = dict(pool, ipc=base64.b64encode(pickle.dumps(_Boom(marker))).decode())
    cases = [
        # the pre-schema format: a pickled callable next to the pool description
        base64.b64encode(json.dumps({"pool": base64.b64encode(json.dumps(legacy).encode()).decode(),
                                     "slots": [1, 2]}).encode()).decode(),
        # right shape of payload, no signature
        base64.b64encode(json.dumps({"pool": pool, "slots": [1, 2], "begin": 0, "end": 2}).encode()).decode(),
        # signed by somebody else
        base64.b64encode(json.dumps({"pool": pool, "slots": [1, 2], "begin": 0, "end": 2,
                                     "mac": "0" * 64}).encode()).decode(),
        "not base64 at all!",
        base64.b64encode(b"[1, 2, 3]").decode(),
    ]
    for meta in cases:
        with pytest.raises(kv_handoff.HandoffError):
            a.send_kv(0, np.asarray([1, 2], dtype=np.int32), meta)
    # a valid payload altered after signing (slots moved) no longer verifies
    good = json.loads(base64.b64decode(kv_handoff.encode_payload(pool, [1, 2], 0, 2)))
    good["slots"] = [1, 3]
    with pytest.raises(kv_handoff.HandoffError):
        a.send_kv(0, np.asarray([1, 2], dtype=np.int32), base64.b64encode(json.dumps(good).encode()).decode())
    assert not os.path.exists(marker)
    assert bool((b.models[0].kv_pages == -1.0).all())


@pytest.mark.parametrize("dst,src", [([64, 1], [0, 1]), ([-1, 1], [0, 1]), ([0, 1], [0, 64]), ([0, 1], [-3, 1]),
                                     ([0, 1, 2], [0, 1])])
def test_slots_outside_the_pools_never_reach_a_copy(dst, src):
    a, b = _executor(0.5), _executor(-1.0)
    meta = kv_handoff.encode_payload(b.kv_export(0), dst, 0, len(dst))
    with pytest.raises(kv_handoff.HandoffError):
        a.send_kv(0, np.asarray(src, dtype=np.int32), meta)
    assert bool((b.models[0].kv_pages == -1.0).all())


def test_descriptor_of_another_layout_is_rejected():
    a, b = _executor(0.0), _executor(-1.0)
    pool = dict(b.kv_export(0), shape=[2, 400, 2, 2, 16, 8])   # claims 100x the pages it has
    with pytest.raises(kv_handoff.HandoffError):
        a.send_kv(0, np.asarray([1], dtype=np.int32), kv_handoff.encode_payload(pool, [5000], 0, 1))


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def plain_server():
    srv = PopenServer(MODEL, "cpu", mode="local", port=_port(), enable_debug=False, api_key="sekret")
    srv.start(timeout=180)
    yield srv
    srv.terminate()


H = {"Authorization": "Bearer sekret"}


def test_debug_options_are_ignored_without_enable_debug(plain_server):
    base = {"model": MODEL, "prompt": [5, 6, 7, 8, 9], "max_tokens": 6, "temperature": 0.0}
    want = requests.post(plain_server.base_url + "/v1/completions", json=base, headers=H, timeout=120).json()
    assert want["usage"].get("extra") is None
    # disagg_config with a hostile descriptor, ignore_eos: all dropped, the
    # request is served as the plain one
    body = dict(base, debug_config={
        "ignore_eos": True,
        "disagg_config": {"kind": "remote_send", "kv_window_begin": 0, "kv_window_end": 4,
                          "kv_append_metadata": base64.b64encode(b"{}").decode(), "dst_group_offset": 0}})
    r = requests.post(plain_server.base_url + "/v1/completions", json=body, headers=H, timeout=120)
    assert r.status_code == 200, r.text
    got = r.json()
    assert got["choices"][0]["text"] == want["choices"][0]["text"]
    assert got["usage"]["completion_tokens"] == want["usage"]["completion_tokens"]
    assert got["usage"].get("extra") is None
    chat = {"model": MODEL, "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0.0,
            "debug_config": {"ignore_eos": True, "pinned_system_prompt": True}}
    r = requests.post(plain_server.base_url + "/v1/chat/completions", json=chat, headers=H, timeout=120)
    assert r.status_code == 200 and r.json()["usage"].get("extra") is None
    assert r.json()["usage"]["completion_tokens"] > 0


def test_microserving_routes_need_the_api_key(plain_server):
    body = {"model": MODEL, "prompt": [5, 6, 7], "end": -1}
    assert requests.post(plain_server.base_url + "/microserving/prep_recv", json=body, timeout=30).status_code == 401
    assert requests.get(plain_server.base_url + "/debug/dump_event_trace", headers=H, timeout=30).status_code == 404
