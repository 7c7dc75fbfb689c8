"""Failure handling without touching a device: an exception inside an engine step fails the requests in
flight and leaves the engine usable; a tensor-parallel worker that goes away between steps surfaces on rank 0
as an error within the process-group timeout instead of a hang."""
import json
import os
import subprocess
import sys
import time

import numpy as np
import pytest

from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.engine import MLCEngine

HERE = os.path.dirname(os.path.abspath(__file__))
MODEL = "random://tiny-llama?quant=q0f32&seed=11"


def test_exception_in_a_step_fails_requests_and_engine_recovers():
    eng = MLCEngine(MODEL, "cpu", mode="server",
                    engine_config=EngineConfig(max_num_sequence=4, prefill_chunk_size=64, max_total_sequence_length=1024))
    try:
        ex = eng.runtime.executor
        orig, orig_launch = ex.forward_sample, ex.forward_sample_launch
        calls = {"n": 0}

        def flaky(*a, **k):
            calls["n"] += 1
            if calls["n"] == 3:
                raise RuntimeError("injected failure in the model call")
            return orig(*a, **k)

        def flaky_launch(*a, **k):   # decode steps whose result is read one step later
            calls["n"] += 1
            if calls["n"] == 3:
                raise RuntimeError("injected failure in the model call")
            return orig_launch(*a, **k)

        ex.forward_sample, ex.forward_sample_launch = flaky, flaky_launch
        rng = np.random.default_rng(0)
        prompts = [rng.integers(10, 31000, 12).tolist() for _ in range(3)]
        res = eng.generate_many(prompts, {"max_tokens": 8, "temperature": 0.0, "debug_config": {"ignore_eos": True}})
        assert all(r["finish_reason"] == "error" for r in res)
        # the engine thread survived: a later request completes normally
        ok = eng.completions.create(prompt=prompts[0], max_tokens=5, temperature=0.0, debug_config={"ignore_eos": True})
        assert ok.choices[0].finish_reason == "length" and ok.usage.completion_tokens == 5
        # streaming consumers see the error too
        calls["n"] = 0
        reasons = []
        for chunk in eng.chat.completions.create(messages=[{"role": "user", "content": "hello there"}], max_tokens=8,
                                                 temperature=0.0, stream=True):
            reasons += [c.finish_reason for c in chunk.choices if c.finish_reason]
        assert reasons == ["error"]
    finally:
        eng.terminate()


def test_worker_rank_leaving_between_steps_is_an_error_not_a_hang():
    """Two gloo ranks; rank 1 exits (cleanly, between steps) after a few forward calls.  Rank 0's next step
    broadcast fails or times out within the group's timeout and the run ends with an error."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29571", os.path.join(HERE, "dist_worker.py"),
           MODEL.replace("seed=11", "seed=5"), "cpu"]
    env = dict(os.environ, OMP_NUM_THREADS="2", MLCB_TEST_WORKER_EXIT_AFTER="3", MLCB_TEST_COMM_TIMEOUT_S="20")
    t0 = time.time()
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    elapsed = time.time() - t0
    assert elapsed < 200
    lines = [l for l in out.stdout.splitlines() if l.startswith("FAILURE ")]
    assert lines, (out.stdout[-1500:], out.stderr[-1500:])
    info = json.loads(lines[-1][len("FAILURE "):])
    assert info["rank"] == 0 and info["error"]
