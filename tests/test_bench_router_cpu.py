"""Load generator and round-robin router against CPU server processes with a tiny random model."""
import asyncio
import socket

import pytest

from mlc_llm_b200.bench.__main__ import build_parser, run
from mlc_llm_b200.protocol import openai_api_protocol as openai
from mlc_llm_b200.router import Router
from mlc_llm_b200.serve.server import PopenServer

MODEL = "random://tiny-llama?quant=q0f32&seed=3"


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_load_generator_fixed_concurrency(tmp_path):
    port = _port()
    srv = PopenServer(MODEL, "cpu", mode="server", port=port)
    srv.start(timeout=180)
    try:
        out = tmp_path / "bench.csv"
        args = build_parser().parse_args([
            "--tokenizer", MODEL, "--num-gpus", "1", "--num-requests", "6", "--num-warmup-requests", "2",
            "--num-concurrent-requests", "3", "--input-len", "24", "--output-len", "8", "--ignore-eos",
            "--temperature", "0", "--host", "127.0.0.1", "--port", str(port), "--include-server-metrics",
            "--disable-tqdm", "--output", str(out)])
        reports = run(args)
        rep = reports[0]
        assert rep["num_completed_requests"] == 6 and rep["num_failed_requests"] == 0
        assert rep["output_tokens"]["mean"] == 8 and rep["input_tokens"]["mean"] == 24
        assert rep["output_token_throughput"] > 0
        assert rep["time_to_first_token_s"]["quantiles"]["p50"] > 0
        assert rep["time_per_output_token_s"]["mean"] > 0
        assert out.exists() and "output_token_throughput" in out.read_text().splitlines()[0]
    finally:
        srv.terminate()


def test_router_round_robin_balances_two_endpoints():
    ports = [_port(), _port()]
    router = Router(MODEL, hosts=["127.0.0.1"] * 2, ports=ports, num_gpus=[1, 1], router_mode="round-robin",
                    device="cpu", server_start_timeout=240)
    try:
        picked = []
        orig = router._pick_endpoint

        def spy(ids):
            i = orig(ids)
            picked.append(i)
            return i

        router._pick_endpoint = spy

        async def one(i):
            req = openai.CompletionRequest(model=MODEL, prompt=[5, 6, 7, 8 + i], max_tokens=4, temperature=0.0,
                                           stream=bool(i % 2), debug_config={"ignore_eos": True})
            texts = []
            async for chunk in router.handle_completion(req, f"r{i}"):
                assert chunk is not None
                texts.append("".join(c.text for c in chunk.choices))
            return "".join(texts)

        async def main():
            return await asyncio.gather(*[one(i) for i in range(4)])

        outs = asyncio.run(main())
        assert len(outs) == 4 and all(isinstance(o, str) for o in outs)
        assert set(picked) == {0, 1}  # concurrent requests are spread over both endpoints
        assert router.num_running_requests == [0, 0]
    finally:
        router.terminate()
