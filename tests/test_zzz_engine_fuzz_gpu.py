"""Randomised engine schedules on the GPU: the workload of ``test_engine_fuzz_cpu`` (staggered arrivals, shared
prefixes, parallel samples, aborts) through the CUDA paths that a fixed batch never reaches together: graph buckets
with stand-in sequences, the tensor-core attention plan of mixed prefill / decode steps, deferred-read decode steps,
draft trees and windows. The oracle is the same prompt run alone on the same GPU; fp16 near-ties may move a late
token, so agreement is required of the first token of every request and of most tokens overall."""
import json
import os

import numpy as np
import pytest
import torch

from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

from test_engine_fuzz_cpu import GREEDY, _workload

pytestmark = pytest.mark.gpu

DEVICE = os.environ.get("MLCB_FUZZ_DEVICE", "cuda")
QUANT = "q0f16" if DEVICE == "cuda" else "q0f32"
MODEL = f"random://tiny-llama-gpu?quant={QUANT}&seed=11"
DRAFT = f"random://tiny-llama-gpu?quant={QUANT}&seed=2"

CONFIGS = {
    "radix_buckets": dict(max_num_sequence=16, max_total_sequence_length=4096, prefill_chunk_size=64,
                          prefix_cache_mode="radix"),
    "tight_pool": dict(max_num_sequence=6, max_total_sequence_length=200, prefill_chunk_size=32,
                       prefix_cache_mode="disable", _gen=(60, 110)),
    "draft_tree": dict(max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64,
                       prefix_cache_mode="radix", speculative_mode="small_draft", spec_draft_length=2,
                       spec_tree_width=2, additional_models=[DRAFT]),
    "window_sink": dict(max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=32,
                        prefix_cache_mode="disable", sliding_window_size=64, attention_sink_size=4, _gen=(30, 90)),
}

_ALONE = {}


def _alone(prompt, max_tokens, window):
    key = (tuple(prompt), max_tokens, window)
    if key not in _ALONE:
        if ("eng", window) not in _ALONE:
            _ALONE[("eng", window)] = SyncMLCEngine(MODEL, DEVICE, engine_config=EngineConfig(
                mode="server", max_num_sequence=4, max_total_sequence_length=4096, prefill_chunk_size=256,
                prefix_cache_mode="disable", **dict(window)))
        _, toks = _ALONE[("eng", window)].generate([prompt], dict(GREEDY, max_tokens=max_tokens))
        _ALONE[key] = toks[0][0]
    return _ALONE[key]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_random_schedules_on_the_gpu(name):
    got, finished = {}, {}

    def on_outputs(outs):
        for out in outs:
            rid, singles = out.unpack()
            for j, s in enumerate(singles):
                if s.request_final_usage_json_str is not None:
                    continue
                got.setdefault((rid, j), []).extend(s.delta_token_ids)
                if s.finish_reason is not None:
                    finished[(rid, j)] = s.finish_reason

    cfg = dict(CONFIGS[name])
    gen = cfg.pop("_gen", (2, 14))
    eng = SyncMLCEngine(MODEL, DEVICE, engine_config=EngineConfig(mode="server", **cfg),
                        request_stream_callback=on_outputs)
    reqs = _workload(3, count=16, gen=gen)
    for r in reqs:
        r["extra"] = {}
    pending = sorted(reqs, key=lambda r: r["arrive"])
    live_since, aborted, step = {}, set(), 0
    while pending or not eng.empty():
        while pending and pending[0]["arrive"] <= step:
            r = pending.pop(0)
            eng.add_request(r["id"], [np.asarray(r["prompt"], dtype=np.int32)],
                            dict(GREEDY, max_tokens=r["max_tokens"], n=r["n"]))
            live_since[r["id"]] = step
        for r in reqs:
            if (r["abort_after"] is not None and r["id"] in live_since and r["id"] not in aborted
                    and step - live_since[r["id"]] >= r["abort_after"]
                    and not all((r["id"], j) in finished for j in range(r["n"]))):
                eng.abort_request(r["id"])
                aborted.add(r["id"])
        eng.step()
        step += 1
        assert step < 5000, "the engine does not drain"
    if DEVICE == "cuda":
        from mlc_llm_b200.ops import _lib

        _lib.check_status(torch.device("cuda"))
    limit = int(eng.engine_config.max_single_sequence_length)
    window = tuple((k, cfg[k]) for k in ("sliding_window_size", "attention_sink_size") if k in cfg)
    same = total = 0
    for r in reqs:
        want = _alone(r["prompt"], r["max_tokens"], window)[: max(0, limit - len(r["prompt"]))]
        for j in range(r["n"]):
            have = got.get((r["id"], j), [])
            if r["id"] in aborted and (r["id"], j) not in finished:
                assert len(have) <= len(want)
                want = want[: len(have)]
            else:
                assert len(have) == len(want), (name, r["id"], j, finished.get((r["id"], j)))
            if want:
                assert have[0] == want[0], (name, r["id"], j, "first token")
            same += sum(int(a == b) for a, b in zip(have, want))
            total += len(want)
    assert same >= 0.7 * total, (name, same, total)
    stats = json.loads(eng.debug_stats())
    assert stats["num_running"] == 0 and stats["num_waiting"] == 0
