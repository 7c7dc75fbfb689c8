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
def test_router_disagg_matches_single_engine():
    rng = np.random.default_rng(0)
    prompts = [rng.integers(10, 31000, n).tolist() for n in (90, 33)]
    plain = MLCEngine(MODEL, "cuda:0", engine_config=EngineConfig(mode="local"))
    try:
        want = [plain.completions.create(prompt=p, max_tokens=8, temperature=0.0,
                                         debug_config={"ignore_eos": True}).choices[0].text for p in prompts]
    finally:
        plain.terminate()
    router = Router(MODEL, hosts=["127.0.0.1"] * 2, ports=[_port(), _port()], num_gpus=[1, 1],
                    router_mode="disagg", device="cuda", server_start_timeout=300)
    try:
        async def one(i, p):
            req = openai.CompletionRequest(model=MODEL, prompt=p, max_tokens=8, temperature=0.0, stream=False,
                                           debug_config={"ignore_eos": True})
            text = ""
            async for chunk in router.handle_completion(req, f"disagg-{i}"):
                assert chunk is not None
                text += "".join(c.text for c in chunk.choices)
            return text

        async def main():
            return [await one(i, p) for i, p in enumerate(prompts)]

        got = asyncio.run(main())
        agree = np.mean([a == b for a, b in zip(got, want)])
        assert agree == 1.0, (got, want)
    finally:
        router.terminate()
