"""Disaggregated prefill / decode on two GPUs: two server processes behind the router; the prefill
engine writes KV rows into the decode engine's pool through a CUDA IPC mapping (peer stores)."""
import asyncio
import socket

import numpy as np
import pytest
import torch

from mlc_llm_b200.protocol import openai_api_protocol as openai
from mlc_llm_b200.router import Router
from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.engine import MLCEngine

pytestmark = pytest.mark.gpu
MODEL = "random://tiny-llama-gpu?quant=q0f16&seed=5"


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_disagg_hand_off_between_gpus_in_process():
    """Prefill engine on GPU 0, decode engine on GPU 1 (one process): the decode engine's result must
    equal its own result when the same prefix comes from its prefix cache, i.e. the received KV rows
    are as good as locally computed ones (same kernels consume them either way)."""
    from mlc_llm_b200.serve.entrypoints.microserving_entrypoints import prep_recv_response

    rng = np.random.default_rng(0)
    prompts = [rng.integers(10, 31000, n).tolist() for n in (90, 33)]
    cfg = dict(mode="server", max_num_sequence=4, max_total_sequence_length=2048)
    p_eng = MLCEngine(MODEL, "cuda:0", engine_config=EngineConfig(prefix_cache_mode="disable", **cfg))
    d_eng = MLCEngine(MODEL, "cuda:1", engine_config=EngineConfig(prefix_cache_mode="disable", **cfg))
    ref = MLCEngine(MODEL, "cuda:1", engine_config=EngineConfig(prefix_cache_mode="radix", **cfg))
    try:
        for i, prompt in enumerate(prompts):
            greedy = dict(max_tokens=8, temperature=0.0)
            # reference: warm the prefix cache with all but the last token, then run the full prompt
            ref.completions.create(prompt=prompt[:-1] + [7], debug_config={"ignore_eos": True}, **greedy)
            want = ref.completions.create(prompt=prompt, debug_config={"ignore_eos": True}, **greedy)
            rid = f"disagg-{i}"
            prep = d_eng.completions.create(prompt=prompt, max_tokens=1, request_id=rid, debug_config={
                "disagg_config": {"kind": "prepare_receive", "kv_window_begin": 0, "kv_window_end": -1}})
            meta = prep_recv_response(d_eng, prep)
            end = len(prompt) - 1
            p_eng.completions.create(prompt=prompt, max_tokens=1, request_id=rid, debug_config={
                "disagg_config": {"kind": "remote_send", "kv_window_begin": meta.prefix_matched_length,
                                  "kv_window_end": end, "kv_append_metadata": meta.kv_append_metadata,
                                  "dst_group_offset": 1}})
            got = d_eng.completions.create(prompt=prompt, request_id=rid, debug_config={
                "ignore_eos": True, "disagg_config": {"kind": "start_generation", "kv_window_begin": end}}, **greedy)
            assert got.usage.extra["prefill_tokens"] == 1
            assert got.choices[0].text == want.choices[0].text
    finally:
        for e in (p_eng, d_eng, ref):
            e.terminate()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_router_disagg_across_processes():
    """Two server processes behind the router in disaggregated mode: the three-step protocol runs
    over HTTP and the KV rows cross process and GPU boundaries through a CUDA IPC mapping."""
    rng = np.random.default_rng(0)
    prompts = [rng.integers(10, 31000, n).tolist() for n in (90, 33)]
    router = Router(MODEL, hosts=["127.0.0.1"] * 2, ports=[_port(), _port()], num_gpus=[1, 1],
                    router_mode="disagg", device="cuda", server_start_timeout=300)
    try:
        async def one(i, p):
            req = openai.CompletionRequest(model=MODEL, prompt=p, max_tokens=8, temperature=0.0, stream=False,
                                           debug_config={"ignore_eos": True})
            out = []
            async for chunk in router.handle_completion(req, f"disagg-{i}"):
                assert chunk is not None
                out.append(chunk)
            return out[-1]

        async def main():
            return [await one(i, p) for i, p in enumerate(prompts)]

        for p, resp in zip(prompts, asyncio.run(main())):
            assert resp.usage.prompt_tokens == len(p) and resp.usage.completion_tokens == 8
            assert resp.usage.extra["prefill_tokens"] == 1   # the decode endpoint computed only the last token
            assert resp.choices[0].finish_reason == "length"
    finally:
        router.terminate()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_kv_slot_copy_between_gpus():
    """The hand-off kernel alone: rows of chosen slots travel from a pool on GPU 0 to other slots of
    a pool on GPU 1 (peer stores); everything else in the destination stays untouched."""
    from mlc_llm_b200.models import config as mc
    from mlc_llm_b200.models.presets import MODEL_PRESETS
    from mlc_llm_b200.serve.executor import ModelExecutor

    class Holder:
        pass

    def fake_model(dev, fill):
        m = Holder()
        m.kv_pages = torch.full((2, 8, 2, 2, 16, 128), fill, dtype=torch.float16, device=dev)
        return m

    src_dev, dst_dev = torch.device("cuda", 0), torch.device("cuda", 1)
    a, b = fake_model(src_dev, 0.0), fake_model(dst_dev, -1.0)
    a.kv_pages.copy_(torch.randn_like(a.kv_pages))
    ex_a, ex_b = ModelExecutor.__new__(ModelExecutor), ModelExecutor.__new__(ModelExecutor)
    for ex, m, d in ((ex_a, a, src_dev), (ex_b, b, dst_dev)):
        ex.models, ex.device, ex.comm = [m], d, None
    from mlc_llm_b200.serve import kv_handoff
    src_slots = np.asarray([3, 17, 18, 40, 127], dtype=np.int32)
    dst_slots = [64, 5, 6, 99, 0]
    meta = kv_handoff.encode_payload(ex_b.kv_export(0), dst_slots, 0, len(dst_slots))
    ex_a.send_kv(0, src_slots, meta)
    torch.cuda.synchronize(dst_dev)
    got, want = b.kv_pages.cpu(), a.kv_pages.cpu()
    for s, d in zip(src_slots.tolist(), dst_slots):
        assert torch.equal(got[:, d // 16, :, :, d % 16, :], want[:, s // 16, :, :, s % 16, :])
    untouched = torch.ones(8 * 16, dtype=torch.bool)
    untouched[dst_slots] = False
    rest = got.permute(1, 4, 0, 2, 3, 5).reshape(8 * 16, -1)[untouched]
    assert bool((rest == -1.0).all())
