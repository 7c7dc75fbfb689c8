"""Randomised engine runs on CPU: requests arrive at random steps, share prompt prefixes, ask for one or two
samples, some are aborted mid-flight, the KV pool is tight enough to force preemption. Whatever the schedule,
every finished request must carry the greedy tokens of the same prompt run alone, an aborted one a prefix of them,
and the engine must end empty with its pages back (prefix-cache entries aside)."""
import json

import numpy as np
import pytest

from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

MODEL = "random://tiny-llama?quant=q0f32&seed=11"
DRAFT = "random://tiny-llama?quant=q0f32&seed=2"
GREEDY = {"temperature": 0.0, "debug_config": {"ignore_eos": True}}


def _workload(seed, count=12, gen=(2, 14)):
    rng = np.random.default_rng(seed)
    stems = [rng.integers(10, 31000, int(n)).tolist() for n in (24, 40)]
    reqs = []
    for i in range(count):
        stem = stems[int(rng.integers(0, 2))] if rng.random() < 0.6 else []
        tail = rng.integers(10, 31000, int(rng.integers(3, 45))).tolist()
        reqs.append({"id": f"q{i}", "prompt": stem + tail, "max_tokens": int(rng.integers(*gen)),
                     "n": 2 if rng.random() < 0.2 else 1, "arrive": int(rng.integers(0, 12)),
                     "abort_after": int(rng.integers(1, 6)) if rng.random() < 0.25 else None})
    # logit processing that depends on what the request has generated so far (drawn after everything else, so the
    # schedules above stay what they were)
    extras = [{}, {}, {"repetition_penalty": 1.3}, {"frequency_penalty": 0.6, "presence_penalty": 0.4},
              {"logit_bias": {str(int(t)): 6.0 for t in rng.integers(10, 31000, 3)}}]
    for r in reqs:
        r["extra"] = extras[int(rng.integers(0, len(extras)))]
    return reqs


_ALONE = {}


def _alone(prompt, max_tokens, window=(), model=MODEL, extra=None):
    """Greedy tokens of one prompt on an engine of its own (``window``: the sliding-window settings, which change
    what a token sees and so belong to the oracle too)."""
    extra = extra or {}
    key = (tuple(prompt), max_tokens, window, model, json.dumps(extra, sort_keys=True))
    window = window + (("_model", model),) if model != MODEL else window
    if key not in _ALONE:
        if ("eng", window) not in _ALONE:
            _ALONE[("eng", window)] = SyncMLCEngine(model, "cpu", engine_config=EngineConfig(
                mode="server", max_num_sequence=4, max_total_sequence_length=2048, prefill_chunk_size=256,
                prefix_cache_mode="disable", **{k: v for k, v in window if k != "_model"}))
        _, toks = _ALONE[("eng", window)].generate([prompt], dict(GREEDY, max_tokens=max_tokens, **extra))
        _ALONE[key] = toks[0][0]
    return _ALONE[key]


CONFIGS = {
    "tight_kv_radix": dict(max_num_sequence=6, max_total_sequence_length=300, prefill_chunk_size=32,
                           prefix_cache_mode="radix"),
    # long outputs in a small pool: admitted sequences outgrow it, the engine preempts and re-prefills
    "preempting": dict(max_num_sequence=6, max_total_sequence_length=160, prefill_chunk_size=32,
                       prefix_cache_mode="disable", _gen=(80, 140)),
    "preempting_radix_draft": dict(max_num_sequence=6, max_total_sequence_length=160, prefill_chunk_size=32,
                                   prefix_cache_mode="radix", speculative_mode="small_draft", spec_draft_length=2,
                                   additional_models=[DRAFT], _gen=(80, 140)),
    # a window of 40 positions behind 4 sink positions: pages fall out of the window while sequences run
    "window_sink": dict(max_num_sequence=6, max_total_sequence_length=1024, prefill_chunk_size=32,
                        prefix_cache_mode="disable", sliding_window_size=40, attention_sink_size=4, _gen=(20, 60)),
    "window_radix_draft": dict(max_num_sequence=6, max_total_sequence_length=1024, prefill_chunk_size=32,
                               prefix_cache_mode="radix", sliding_window_size=40, attention_sink_size=4,
                               speculative_mode="small_draft", spec_draft_length=2, additional_models=[DRAFT],
                               _gen=(20, 60)),
    "window_tight": dict(max_num_sequence=6, max_total_sequence_length=160, prefill_chunk_size=32,
                         prefix_cache_mode="disable", sliding_window_size=48, attention_sink_size=0,
                         _gen=(60, 110)),
    "eagle_tree_radix": dict(max_num_sequence=6, max_total_sequence_length=1024, prefill_chunk_size=48,
                             prefix_cache_mode="radix", speculative_mode="eagle", spec_draft_length=2,
                             spec_tree_width=2, additional_models=["random://tiny-eagle?quant=q0f32&seed=3"]),
    "medusa_tight": dict(max_num_sequence=4, max_total_sequence_length=400, prefill_chunk_size=32,
                         prefix_cache_mode="disable", speculative_mode="medusa", spec_draft_length=3,
                         additional_models=["random://tiny-medusa?quant=q0f32&seed=4"]),
    # recurrent-state families: a sequence's state is found by its id, a preempted sequence starts over
    "rwkv6_tight": dict(_model="random://tiny-rwkv6?quant=q0f32&seed=5", max_num_sequence=4,
                        max_total_sequence_length=1024, prefill_chunk_size=32),
    "qwen35_hybrid_state": dict(_model="random://tiny-qwen35?quant=q0f32&seed=5", max_num_sequence=5,
                                max_total_sequence_length=1024, prefill_chunk_size=32, _gen=(4, 30)),
    # compressed latent cache (one row per token for all heads) against the expanded-cache oracle
    "deepseek_latent_radix": dict(_model="random://tiny-deepseek-v2?quant=q0f32&seed=5&mla_cache=latent",
                                  _oracle="random://tiny-deepseek-v2?quant=q0f32&seed=5", max_num_sequence=6,
                                  max_total_sequence_length=400, prefill_chunk_size=32, prefix_cache_mode="radix"),
    "qwen35_tight": dict(_model="random://tiny-qwen35?quant=q0f32&seed=5", max_num_sequence=6,
                         max_total_sequence_length=160, prefill_chunk_size=32, _gen=(60, 110)),
    "hybrid_prefill": dict(max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=48,
                           prefix_cache_mode="radix", prefill_mode="hybrid"),
    "draft_tree_radix": dict(max_num_sequence=6, max_total_sequence_length=1024, prefill_chunk_size=64,
                             prefix_cache_mode="radix", speculative_mode="small_draft", spec_draft_length=2,
                             spec_tree_width=2, additional_models=[DRAFT]),
    "draft_chain_tight": dict(max_num_sequence=4, max_total_sequence_length=400, prefill_chunk_size=32,
                              prefix_cache_mode="disable", speculative_mode="small_draft", spec_draft_length=3,
                              additional_models=[DRAFT]),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("seed", [0, 1])
def test_random_schedules_keep_every_request_exact(name, seed):
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
    model = cfg.pop("_model", MODEL)
    oracle = cfg.pop("_oracle", model)
    eng = SyncMLCEngine(model, "cpu", engine_config=EngineConfig(mode="server", **cfg),
                        request_stream_callback=on_outputs)
    reqs = _workload(seed, gen=gen)
    pending = sorted(reqs, key=lambda r: r["arrive"])
    live_since, aborted = {}, set()
    step = 0
    while pending or not eng.empty():
        while pending and pending[0]["arrive"] <= step:
            r = pending.pop(0)
            eng.add_request(r["id"], [np.asarray(r["prompt"], dtype=np.int32)],
                            dict(GREEDY, max_tokens=r["max_tokens"], n=r["n"], **r["extra"]))
            live_since[r["id"]] = step
        for r in reqs:
            if (r["abort_after"] is not None and r["id"] in live_since and r["id"] not in aborted
                    and step - live_since[r["id"]] >= r["abort_after"]
                    and not all((r["id"], j) in finished for j in range(r["n"]))):
                eng.abort_request(r["id"])
                aborted.add(r["id"])
        eng.step()
        step += 1
        assert step < 3000, "the engine does not drain"
    limit = int(eng.engine_config.max_single_sequence_length)
    window = tuple((k, cfg[k]) for k in ("sliding_window_size", "attention_sink_size") if k in cfg)
    for r in reqs:
        # a sequence ends with "length" at the engine's single-sequence limit as well as at max_tokens
        want = _alone(r["prompt"], r["max_tokens"], window, oracle, r["extra"])[: max(0, limit - len(r["prompt"]))]
        for j in range(r["n"]):
            have = got.get((r["id"], j), [])
            if r["id"] in aborted and (r["id"], j) not in finished:
                assert have == want[: len(have)], (name, r["id"], j, "aborted")
            else:
                assert have == want, (name, r["id"], j, finished.get((r["id"], j)))
                assert finished[(r["id"], j)] == "length"
    stats = json.loads(eng.debug_stats())
    assert stats["num_running"] == 0 and stats["num_waiting"] == 0
    if name.startswith("preempting") and seed == 0:
        assert stats["num_preemptions"] >= 1  # this schedule is known to outgrow the pool
    # sequences are gone: what is still allocated belongs to prefix-cache entries kept for reuse
    if CONFIGS[name].get("prefix_cache_mode") == "disable":
        assert stats["kv_total_sequence_length"] == 0
    eng.reset()
    assert json.loads(eng.debug_stats())["kv_total_sequence_length"] == 0


@pytest.mark.parametrize("recycling", [1, 8])
@pytest.mark.parametrize("draft", [False, True])
def test_multi_round_conversations_reuse_their_own_history(recycling, draft):
    """Four interleaved conversations of three rounds: a round's prompt is the previous prompt, the previous answer
    and new tokens, so the radix cache can continue the finished sequence (or, once recycled away, cannot). With
    room for one or for eight recycled sequences, with and without a draft model, answers equal the uncached ones
    and hits show up as prefill tokens saved."""
    rng = np.random.default_rng(4)
    kw = dict(max_num_sequence=6, max_total_sequence_length=2048, prefill_chunk_size=48, prefix_cache_mode="radix",
              prefix_cache_max_num_recycling_seqs=recycling)
    if draft:
        kw.update(speculative_mode="small_draft", spec_draft_length=2, additional_models=[DRAFT])
    eng = SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(mode="server", **kw))
    convs = [rng.integers(10, 31000, int(n)).tolist() for n in (30, 12, 55, 21)]
    fed = 0
    for rnd in range(3):
        prompts = [list(c) for c in convs]
        _, toks = eng.generate(prompts, dict(GREEDY, max_tokens=9))
        fed += sum(len(p) for p in prompts)
        for i, c in enumerate(convs):
            assert toks[i][0] == _alone(prompts[i], 9), (rnd, i)
            convs[i] = c + toks[i][0] + rng.integers(10, 31000, int(rng.integers(2, 9))).tolist()
    m = eng.metrics()
    prefilled = int(m.get("prefill_tokens_sum", m.get("sum_engine_prefill_tokens", -1)))
    if prefilled >= 0:
        assert prefilled < fed                   # later rounds did not recompute all of their history
        if recycling == 8:
            assert prefilled < 0.7 * fed


def test_preempted_hybrid_state_sequences_start_over():
    """Qwen3.5 (paged attention layers beside a recurrent state) in a pool its sequences outgrow: a preempted
    sequence is prefilled again from position 0, which must also reset its recurrent state."""
    model = "random://tiny-qwen35?quant=q0f32&seed=5"
    rng = np.random.default_rng(0)
    prompts = [rng.integers(10, 31000, int(rng.integers(20, 60))).tolist() for _ in range(6)]
    gen = dict(GREEDY, max_tokens=120)
    roomy = SyncMLCEngine(model, "cpu", engine_config=EngineConfig(
        mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64))
    _, want = roomy.generate(prompts, gen)
    tight = SyncMLCEngine(model, "cpu", engine_config=EngineConfig(
        mode="server", max_num_sequence=6, max_total_sequence_length=224, prefill_chunk_size=64))
    _, got = tight.generate(prompts, gen)
    assert [t[0] for t in got] == [t[0] for t in want]
    assert json.loads(tight.debug_stats())["num_preemptions"] >= 1


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_nested_prefixes_under_eviction(seed):
    """Twenty requests over three nested stems (A, A+B, A+B+C) and unrelated prompts, in a pool that cannot keep
    everything cached: the radix cache forks, extends, recycles and evicts while requests run, one system prompt
    is pinned. Every answer equals the uncached one."""
    rng = np.random.default_rng(100 + seed)
    a = rng.integers(10, 31000, 22).tolist()
    b = a + rng.integers(10, 31000, 17).tolist()
    c = b + rng.integers(10, 31000, 26).tolist()
    stems = [[], a, b, c]
    eng_got = {}

    def on_outputs(outs):
        for out in outs:
            rid, singles = out.unpack()
            if singles[0].request_final_usage_json_str is None:
                eng_got.setdefault(rid, []).extend(singles[0].delta_token_ids)

    eng = SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(
        mode="server", max_num_sequence=5, max_total_sequence_length=420, prefill_chunk_size=32,
        prefix_cache_mode="radix", prefix_cache_max_num_recycling_seqs=2), request_stream_callback=on_outputs)
    reqs = []
    for i in range(20):
        stem = stems[int(rng.integers(0, 4))]
        cut = len(stem) if rng.random() < 0.7 else int(rng.integers(0, len(stem) + 1))   # sometimes mid-stem
        prompt = stem[:cut] + rng.integers(10, 31000, int(rng.integers(1, 30))).tolist()
        reqs.append((f"p{i}", prompt, int(rng.integers(2, 20)), int(rng.integers(0, 25))))
    pending = sorted(reqs, key=lambda r: r[3])
    step = 0
    while pending or not eng.empty():
        while pending and pending[0][3] <= step:
            rid, prompt, max_tokens, _ = pending.pop(0)
            debug = dict(GREEDY["debug_config"], pinned_system_prompt=(rid == "p0"))
            eng.add_request(rid, [np.asarray(prompt, dtype=np.int32)],
                            dict(GREEDY, max_tokens=max_tokens, debug_config=debug))
        eng.step()
        step += 1
        assert step < 4000
    for rid, prompt, max_tokens, _ in reqs:
        assert eng_got.get(rid, []) == _alone(prompt, max_tokens), rid
    stats = json.loads(eng.debug_stats())
    assert stats["num_running"] == 0 and stats["num_waiting"] == 0


def test_json_mode_survives_preemption():
    """Schema-constrained requests in a pool they outgrow: a preempted request is prefilled again with the tokens
    it had produced, and its grammar state must still stand where those tokens left it."""
    rng = np.random.default_rng(7)
    prompts = [rng.integers(10, 31000, int(n)).tolist() for n in (25, 40, 31, 52, 18, 44)]
    schema = json.dumps({"type": "object", "properties": {"a": {"type": "array", "items": {"type": "integer"}}},
                         "required": ["a"]})
    gen = {"temperature": 0.0, "max_tokens": 100, "response_format": {"type": "json_object", "schema": schema}}
    base = dict(mode="server", prefill_chunk_size=32, prefix_cache_mode="disable")
    roomy = SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(max_num_sequence=8,
                                                                   max_total_sequence_length=2048, **base))
    _, want = roomy.generate(prompts, gen)
    tight = SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(max_num_sequence=6,
                                                                   max_total_sequence_length=224, **base))
    _, got = tight.generate(prompts, gen)
    assert [t[0] for t in got] == [t[0] for t in want]
    assert json.loads(tight.debug_stats())["num_preemptions"] >= 1
