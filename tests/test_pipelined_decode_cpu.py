"""Deferred-read ("pipelined") decode steps: the engine queues step n + 1 before it has read step n's
tokens.  Whatever the requests do (stop at an end-of-sequence token, at a stop string, at their length
limit, get aborted, sample with a seed, fork into several choices), the output must be exactly what the
synchronous engine produces, and the pipelined path must actually have run."""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

MODEL = "random://tiny-llama?quant=q0f32&seed=11"


def _engine():
    return SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(
        mode="server", max_num_sequence=16, max_total_sequence_length=4096, prefill_chunk_size=256,
        prefix_cache_mode="disable"))


def _workload():
    rng = np.random.default_rng(5)
    prompts = [rng.integers(10, 31000, n).tolist() for n in (17, 5, 40, 9, 23, 3)]
    cfgs = [
        {"max_tokens": 24, "temperature": 0.0},                                   # may stop at EOS
        {"max_tokens": 7, "temperature": 0.0, "debug_config": {"ignore_eos": True}},
        {"max_tokens": 30, "temperature": 0.9, "top_p": 0.8, "seed": 3, "debug_config": {"ignore_eos": True}},
        {"max_tokens": 12, "temperature": 0.7, "seed": 9, "n": 3, "debug_config": {"ignore_eos": True}},
        {"max_tokens": 20, "temperature": 0.0, "logprobs": True, "top_logprobs": 2,
         "debug_config": {"ignore_eos": True}},
        {"max_tokens": 1, "temperature": 0.0},
    ]
    return prompts, cfgs


def _run(engine):
    prompts, cfgs = _workload()
    _, tokens = engine.generate(prompts, cfgs)
    return tokens, json.loads(engine.debug_stats())


def test_pipelined_outputs_equal_synchronous_outputs():
    eng = _engine()
    got, stats = _run(eng)
    assert stats["num_pipelined_decode_steps"] > 10, stats
    # the same workload in a process whose engine never defers a read
    code = textwrap.dedent("""
        import json, sys
        sys.path.insert(0, %r)
        from tests.test_pipelined_decode_cpu import _engine, _run
        tokens, stats = _run(_engine())
        print(json.dumps({"tokens": tokens, "pipelined": stats["num_pipelined_decode_steps"]}))
    """ % os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env = dict(os.environ, MLCB_PIPELINED_DECODE="0")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    ref = json.loads(out.stdout.strip().splitlines()[-1])
    assert ref["pipelined"] == 0
    assert got == ref["tokens"]
    assert [len(c) for c in got[1]] == [7] and [len(c) for c in got[3]] == [12, 12, 12] and len(got[5][0]) == 1


def test_stop_token_mid_stream_drops_the_extra_token():
    """A request that ends at a stop token was scheduled once more before the engine saw the token:
    that token must not reach the output and the other requests must not notice."""
    eng = _engine()
    rng = np.random.default_rng(1)
    prompt = rng.integers(10, 31000, 12).tolist()
    _, free = eng.generate([prompt], {"max_tokens": 16, "temperature": 0.0, "debug_config": {"ignore_eos": True}})
    stop_at = free[0][0][5]                      # the 6th generated token becomes a stop token
    first = free[0][0].index(stop_at)
    other = rng.integers(10, 31000, 8).tolist()
    _, alone = eng.generate([other], {"max_tokens": 16, "temperature": 0.0, "debug_config": {"ignore_eos": True}})
    before = json.loads(eng.debug_stats())["num_dropped_pipelined_tokens"]
    _, both = eng.generate([prompt, other], [
        {"max_tokens": 16, "temperature": 0.0, "stop_token_ids": [stop_at], "debug_config": {"ignore_eos": True}},
        {"max_tokens": 16, "temperature": 0.0, "debug_config": {"ignore_eos": True}}])
    assert both[0][0] == free[0][0][:first]       # the stop token itself is not part of the output
    assert both[1][0] == alone[0][0]
    assert json.loads(eng.debug_stats())["num_dropped_pipelined_tokens"] == before + 1


def test_abort_while_a_step_is_unread():
    eng = _engine()
    rng = np.random.default_rng(2)
    a, b = rng.integers(10, 31000, 9).tolist(), rng.integers(10, 31000, 14).tolist()
    cfg = {"max_tokens": 12, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    _, alone = eng.generate([b], cfg)
    eng.add_request("victim", [a], cfg)
    eng.add_request("keeper", [b], cfg)
    for _ in range(4):
        eng.step()
    eng.abort_request("victim")                   # its row of the unread step is dropped on arrival
    tokens = []
    while not eng.empty():
        eng.step()
    for out in eng.take_outputs():
        if out["request_id"] == "keeper":
            tokens.extend(out["group_delta_token_ids"][0])
        else:
            assert out["request_id"] == "victim"
    assert tokens == alone[0][0]


def test_new_request_joins_between_pipelined_steps():
    eng = _engine()
    rng = np.random.default_rng(3)
    a, b = rng.integers(10, 31000, 11).tolist(), rng.integers(10, 31000, 6).tolist()
    cfg = {"max_tokens": 14, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    _, ref = eng.generate([a, b], cfg)
    eng.add_request("first", [a], cfg)
    for _ in range(5):
        eng.step()
    eng.add_request("second", [b], cfg)           # forces the unread step to be settled, then a prefill
    got = {"first": [], "second": []}
    while not eng.empty():
        eng.step()
    for out in eng.take_outputs():
        got[out["request_id"]].extend(out["group_delta_token_ids"][0])
    assert got["first"] == ref[0][0] and got["second"] == ref[1][0]
