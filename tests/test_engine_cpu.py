"""Engine behaviour on CPU with a tiny random model: scheduling (chunked / hybrid prefill, preemption),
prefix cache, parallel sampling, stop conditions, logprobs, speculative decoding, the mock echo model,
metrics and the public MLCEngine / AsyncMLCEngine surface."""
import asyncio
import json

import numpy as np
import pytest

from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.engine import AsyncMLCEngine, MLCEngine
from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

MODEL = "random://tiny-llama?quant=q0f32&seed=11"
GREEDY = {"temperature": 0.0, "debug_config": {"ignore_eos": True}}


def _prompts(n, lo=20, hi=60, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(10, 31000, int(rng.integers(lo, hi))).tolist() for _ in range(n)]


def _engine(**kw):
    cfg = EngineConfig(mode="server", max_num_sequence=kw.pop("max_num_sequence", 8),
                       max_total_sequence_length=kw.pop("max_total_sequence_length", 2048),
                       prefill_chunk_size=kw.pop("prefill_chunk_size", 64), **kw)
    return SyncMLCEngine(MODEL, "cpu", engine_config=cfg)


@pytest.fixture(scope="module")
def reference_outputs():
    eng = _engine(prefix_cache_mode="disable")
    prompts = _prompts(6)
    _, toks = eng.generate(prompts, dict(GREEDY, max_tokens=12))
    return prompts, [t[0] for t in toks]


def test_batched_generation_is_independent_of_batching(reference_outputs):
    prompts, want = reference_outputs
    # one at a time
    eng = _engine(prefix_cache_mode="disable", max_num_sequence=1)
    for p, w in zip(prompts[:3], want[:3]):
        _, toks = eng.generate([p], dict(GREEDY, max_tokens=12))
        assert toks[0][0] == w
    # chunked prefill with a chunk smaller than the prompts
    eng = _engine(prefix_cache_mode="disable", prefill_chunk_size=16, prefill_mode="chunked")
    _, toks = eng.generate(prompts, dict(GREEDY, max_tokens=12))
    assert [t[0] for t in toks] == want


def test_preemption_under_kv_pressure_keeps_outputs(reference_outputs):
    prompts, _ = reference_outputs
    roomy = _engine(prefix_cache_mode="disable")
    _, want = roomy.generate(prompts, dict(GREEDY, max_tokens=120))
    # the admitted sequences outgrow the cache while decoding: the engine must preempt and re-prefill
    eng = _engine(prefix_cache_mode="disable", max_total_sequence_length=224, max_num_sequence=6)
    _, toks = eng.generate(prompts, dict(GREEDY, max_tokens=120))
    assert [t[0] for t in toks] == [t[0] for t in want]
    stats = json.loads(eng.debug_stats())
    assert stats.get("num_preemptions", 0) >= 1


def test_prefix_cache_skips_shared_prefix():
    eng = _engine(prefix_cache_mode="radix")
    shared = _prompts(1, 96, 97, seed=3)[0]
    p1, p2 = shared + [11, 12, 13], shared + [21, 22]
    _, a = eng.generate([p1], dict(GREEDY, max_tokens=4))
    m1 = eng.metrics()
    _, b = eng.generate([p2], dict(GREEDY, max_tokens=4))
    m2 = eng.metrics()
    prefilled_second = m2["prefill_tokens_sum"] - m1["prefill_tokens_sum"]
    assert m1["prefill_tokens_sum"] == len(p1)
    assert prefilled_second <= len(p2) - 90  # the shared 96 tokens are not recomputed
    # and the result equals a run without the cache
    cold = _engine(prefix_cache_mode="disable")
    _, c = cold.generate([p2], dict(GREEDY, max_tokens=4))
    assert b[0][0] == c[0][0]


def test_parallel_sampling_n_and_seed():
    eng = _engine()
    p = _prompts(1, seed=5)
    cfg = {"n": 3, "temperature": 1.0, "top_p": 0.95, "seed": 123, "max_tokens": 8,
           "debug_config": {"ignore_eos": True}}
    _, a = eng.generate(p, cfg)
    _, b = eng.generate(p, cfg)
    assert len(a[0]) == 3 and a == b                      # same seed -> same three continuations
    assert len({tuple(x) for x in a[0]}) > 1              # the three branches differ from each other
    _, c = eng.generate(p, dict(cfg, seed=124))
    assert c != a


def test_stop_conditions_and_logprobs():
    eng = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(mode="local"))
    try:
        prompt = _prompts(1, seed=9)[0]
        base = eng.completions.create(prompt=prompt, max_tokens=10, temperature=0.0,
                                      debug_config={"ignore_eos": True}, logprobs=True, top_logprobs=3)
        ch = base.choices[0]
        assert ch.finish_reason == "length" and base.usage.completion_tokens == 10
        lp = ch.logprobs.content
        assert len(lp) == 10 and all(len(x.top_logprobs) == 3 for x in lp)
        # the legacy completions layout: ``logprobs=<number of alternatives>`` gives parallel lists
        legacy = eng.completions.create(prompt=prompt, max_tokens=10, temperature=0.0,
                                        debug_config={"ignore_eos": True}, logprobs=2).choices[0]
        assert legacy.text == ch.text
        ll = legacy.logprobs
        assert ll.tokens == [x.token for x in lp] and len(ll.token_logprobs) == 10
        assert all(abs(a - x.logprob) < 1e-5 for a, x in zip(ll.token_logprobs, lp))
        assert all(len(t) <= 2 and tok in t for t, tok in zip(ll.top_logprobs, ll.tokens))  # greedy: the token is top-1
        assert ll.text_offset[0] == 0 and ll.text_offset[1] == len(ll.tokens[0])
        assert all(x.logprob <= 0 and abs(x.logprob - x.top_logprobs[0].logprob) < 1e-4 for x in lp)  # greedy = top-1
        # stop string: generation ends before the text that contains it, finish_reason "stop"
        text = ch.text
        cut = text[len(text) // 2: len(text) // 2 + 3]
        if cut.strip():
            r = eng.completions.create(prompt=prompt, max_tokens=10, temperature=0.0, stop=[cut],
                                       debug_config={"ignore_eos": True})
            assert r.choices[0].finish_reason == "stop" and cut not in r.choices[0].text
            assert text.startswith(r.choices[0].text)
        # echo + streaming
        chunks = list(eng.completions.create(prompt=prompt, max_tokens=5, temperature=0.0, stream=True, echo=True,
                                             debug_config={"ignore_eos": True},
                                             stream_options={"include_usage": True}))
        assert chunks[-1].usage.completion_tokens == 5 and not chunks[-1].choices
        # logit_bias forces a token
        forced = eng.completions.create(prompt=prompt, max_tokens=3, temperature=0.0, logit_bias={777: 100},
                                        debug_config={"ignore_eos": True})
        assert forced.usage.completion_tokens == 3
        m = eng.metrics()
        assert m["completion_tokens_sum"] >= 18 and "engine_decode_time_sum" in m.metrics
        assert "completion_tokens_sum" in m.prometheus_text()
    finally:
        eng.terminate()


def test_async_engine_concurrent_streams_and_abort():
    eng = AsyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(mode="server", max_num_sequence=8,
                                                                  max_total_sequence_length=2048))

    async def run():
        async def one(i, n_tok):
            out = []
            stream = await eng.completions.create(prompt=_prompts(1, seed=20 + i)[0], max_tokens=n_tok,
                                                  temperature=0.0, stream=True, debug_config={"ignore_eos": True})
            async for chunk in stream:
                out.append(chunk)
            return out

        results = await asyncio.gather(*[one(i, 6 + i) for i in range(4)])
        for i, chunks in enumerate(results):
            finals = [c for c in chunks for ch in c.choices if ch.finish_reason]
            assert len(finals) == 1
        # abort: cancel a long request mid-stream; the engine must stay usable
        stream = await eng.completions.create(prompt=_prompts(1, seed=30)[0], max_tokens=400, temperature=0.0,
                                              stream=True, request_id="victim", debug_config={"ignore_eos": True})
        got = 0
        async for _ in stream:
            got += 1
            if got == 3:
                await eng.abort("victim")
                break
        await stream.aclose()
        again = await eng.completions.create(prompt=[5, 6, 7], max_tokens=4, temperature=0.0,
                                             debug_config={"ignore_eos": True})
        assert again.usage.completion_tokens == 4

    try:
        asyncio.run(run())
    finally:
        eng.terminate()


def test_speculative_decoding_small_draft_matches_plain_greedy(reference_outputs):
    prompts, want = reference_outputs
    cfg = EngineConfig(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64,
                       prefix_cache_mode="disable", speculative_mode="small_draft", spec_draft_length=3,
                       additional_models=["random://tiny-llama?quant=q0f32&seed=12&num_hidden_layers=1"])
    eng = SyncMLCEngine(MODEL, "cpu", engine_config=cfg)
    _, toks = eng.generate(prompts[:4], dict(GREEDY, max_tokens=12))
    # greedy verification only ever emits the target model's argmax tokens
    assert [t[0] for t in toks] == want[:4]
    m = eng.metrics()
    assert m["spec_decode"]["draft_count"][0] > 0 if isinstance(m.get("spec_decode"), dict) else True
    # a draft identical to the target is always accepted: fewer verify steps than tokens
    cfg2 = EngineConfig(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64,
                        prefix_cache_mode="disable", speculative_mode="small_draft", spec_draft_length=3,
                        additional_models=[MODEL])
    eng2 = SyncMLCEngine(MODEL, "cpu", engine_config=cfg2)
    _, toks2 = eng2.generate(prompts[:2], dict(GREEDY, max_tokens=12))
    assert [t[0] for t in toks2] == want[:2]
    stats = json.loads(eng2.debug_stats())
    assert stats["num_verify_steps"] * 2 <= 12 + 4


def test_mock_echo_model_runs_engine_without_a_model():
    eng = MLCEngine(MODEL, "cpu", model_lib="mock://echo", engine_config=EngineConfig(mode="local"))
    try:
        r = eng.completions.create(prompt=[101, 102, 103, 104], max_tokens=4)
        assert r.usage.prompt_tokens == 4 and r.usage.completion_tokens == 4
        assert r.choices[0].text == eng.tokenizer.decode([101, 102, 103, 104])
        chunks = list(eng.chat.completions.create(messages=[{"role": "user", "content": "abc"}], max_tokens=3,
                                                  stream=True))
        assert any(ch.finish_reason for c in chunks for ch in c.choices)
    finally:
        eng.terminate()


def test_request_validation_errors():
    eng = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(mode="local", max_single_sequence_length=64))
    try:
        with pytest.raises(Exception):
            eng.completions.create(prompt=list(range(10, 200)), max_tokens=4)  # longer than the limit
        with pytest.raises(Exception):
            eng.completions.create(prompt=[1, 2, 3], max_tokens=4, temperature=-0.5)
        ok = eng.completions.create(prompt=[1, 2, 3], max_tokens=2)
        assert ok.usage.completion_tokens <= 2
    finally:
        eng.terminate()


def test_json_ffi_engine_matches_python_engine():
    """The native JSON front end (template + tokenizer + detokenizer in C++) gives the same text as
    the Python protocol path."""
    from mlc_llm_b200.json_ffi import JSONFFIEngine

    msgs = [{"role": "user", "content": "hello there"}]
    ffi = JSONFFIEngine(MODEL, "cpu", engine_config=EngineConfig(mode="local"))
    try:
        chunks = list(ffi.chat.completions.create(messages=msgs, max_tokens=8, temperature=0.0,
                                                  stream_options={"include_usage": True}))
        text = "".join(ch.delta.content or "" for c in chunks for ch in c.choices)
        assert chunks[-1].usage is not None and chunks[-1].usage.completion_tokens <= 8
        assert any(ch.finish_reason for c in chunks for ch in c.choices)
        with pytest.raises(ValueError):
            list(ffi.chat.completions.create(messages=msgs, max_tokens=4, temperature=-3))
        ffi._test_reset()
        again = "".join(ch.delta.content or "" for c in ffi.chat.completions.create(
            messages=msgs, max_tokens=8, temperature=0.0) for ch in c.choices)
        assert again == text
    finally:
        ffi.terminate()
    py = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(mode="local"))
    try:
        r = py.chat.completions.create(messages=msgs, max_tokens=8, temperature=0.0)
        assert r.choices[0].message.content == text
    finally:
        py.terminate()


def test_disaggregated_prefill_decode_hand_off():
    """Two engines of one process act as prefill (P) and decode (D) endpoints: D reserves KV and
    reports its prefix-cache hit, P prefills and copies the KV rows into D's pool, D prefills only the
    last prompt token and decodes. The output must equal a plain run, and D must not recompute."""
    from mlc_llm_b200.serve.entrypoints.microserving_entrypoints import prep_recv_response

    cfg = dict(mode="server", max_num_sequence=4, max_total_sequence_length=1024, prefill_chunk_size=64)
    plain = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**cfg))
    p_eng = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**cfg))
    d_eng = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**cfg))
    try:
        prompt = _prompts(1, 70, 71, seed=41)[0]
        want = plain.completions.create(prompt=prompt, max_tokens=10, temperature=0.0,
                                        debug_config={"ignore_eos": True})

        def run(prompt, rid):
            prep = d_eng.completions.create(prompt=prompt, max_tokens=1, request_id=rid, debug_config={
                "disagg_config": {"kind": "prepare_receive", "kv_window_begin": 0, "kv_window_end": -1}})
            meta = prep_recv_response(d_eng, prep)
            end = len(prompt) - 1
            assert meta.prefix_matched_length <= end
            if meta.prefix_matched_length < end:
                p_eng.completions.create(prompt=prompt, max_tokens=1, request_id=rid, debug_config={
                    "disagg_config": {"kind": "remote_send", "kv_window_begin": meta.prefix_matched_length,
                                      "kv_window_end": end, "kv_append_metadata": meta.kv_append_metadata,
                                      "dst_group_offset": 0}})
            before = d_eng.metrics()["prefill_tokens_sum"]
            out = d_eng.completions.create(prompt=prompt, max_tokens=10, temperature=0.0, request_id=rid,
                                           debug_config={"ignore_eos": True, "disagg_config": {
                                               "kind": "start_generation", "kv_window_begin": end}})
            return out, meta.prefix_matched_length, d_eng.metrics()["prefill_tokens_sum"] - before

        got, matched, d_prefilled = run(prompt, "disagg-1")
        assert got.choices[0].text == want.choices[0].text and matched == 0
        assert d_prefilled == 1 and got.usage.prompt_tokens == len(prompt)   # D computed only the last token
        # a second request sharing 64 tokens hits D's prefix cache: P sends only the remainder
        prompt2 = prompt[:64] + _prompts(1, 12, 13, seed=42)[0]
        want2 = plain.completions.create(prompt=prompt2, max_tokens=10, temperature=0.0,
                                         debug_config={"ignore_eos": True})
        got2, matched2, _ = run(prompt2, "disagg-2")
        assert got2.choices[0].text == want2.choices[0].text and matched2 >= 48
    finally:
        for e in (plain, p_eng, d_eng):
            e.terminate()


def test_json_mode_jump_forward_skips_decode_steps_and_keeps_the_text():
    """Grammar-constrained output with and without jump-forward decoding: the forced parts of the JSON
    (keys, punctuation) are appended without a decode step each, several requests at once, and the
    text is what token-by-token constrained decoding produces (greedy)."""
    pytest.importorskip("xgrammar")
    schema = json.dumps({"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                                           "tags": {"type": "array", "items": {"type": "string"}}},
                         "required": ["name", "age", "tags"]})
    prompts = _prompts(3, seed=3)
    out = {}
    for mode in ("constraint", "jump_forward"):
        eng = _engine(prefix_cache_mode="radix")
        cfg = {"max_tokens": 48, "temperature": 0.0, "response_format": {"type": "json_object", "schema": schema},
               "debug_config": {"grammar_execution_mode": mode}}
        texts, toks = eng.generate(prompts, cfg)
        stats = json.loads(eng.debug_stats())
        out[mode] = ([t[0] for t in texts], stats["num_decode_steps"], stats["num_prefill_steps"])
        assert all(t[0].startswith("{") for t in texts)
        # the sequences' KV was returned: nothing leaks through the roll-back / re-prefill path
        assert stats["num_running"] == 0
    assert out["jump_forward"][0] == out["constraint"][0]
    assert out["jump_forward"][1] < out["constraint"][1]
    assert out["jump_forward"][2] > out["constraint"][2]


def test_speculative_decoding_with_draft_trees(reference_outputs):
    """spec_tree_width > 1: every draft round gives each leaf several children; verification walks the
    tree.  Greedy output stays the target model's, also when lower-ranked children carry no draft
    probability; an identical draft model has its first child accepted at every level."""
    prompts, want = reference_outputs
    for draft, width, length in (("random://tiny-llama?quant=q0f32&seed=12&num_hidden_layers=1", 2, 3),
                                 (MODEL, 2, 3), (MODEL, 3, 2)):
        cfg = EngineConfig(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64,
                           prefix_cache_mode="disable", speculative_mode="small_draft", spec_draft_length=length,
                           spec_tree_width=width, additional_models=[draft])
        eng = SyncMLCEngine(MODEL, "cpu", engine_config=cfg)
        _, toks = eng.generate(prompts[:4], dict(GREEDY, max_tokens=12))
        assert [t[0] for t in toks] == want[:4], (draft, width, length)
        stats = json.loads(eng.debug_stats())
        assert stats["num_running"] == 0
        if draft == MODEL:
            assert stats["num_verify_steps"] <= -(-11 // (length + 1)) + 1
    # sampling (temperature > 0) runs through the same path
    cfg = EngineConfig(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64,
                       prefix_cache_mode="disable", speculative_mode="small_draft", spec_draft_length=2,
                       spec_tree_width=2, additional_models=[MODEL])
    eng = SyncMLCEngine(MODEL, "cpu", engine_config=cfg)
    _, toks = eng.generate(prompts[:2], {"max_tokens": 10, "temperature": 0.8, "top_p": 0.95, "seed": 3,
                                         "debug_config": {"ignore_eos": True}})
    assert all(len(t[0]) == 10 for t in toks)


def test_verify_tree_rejects_candidates_without_probability():
    """A child whose token has zero probability under both distributions must not be accepted (0 >= 0)."""
    import torch

    from mlc_llm_b200.ops import reference as ref

    vocab = 6
    model = torch.zeros(3, vocab)
    model[0, 4] = 1.0            # after the root the target wants token 4
    draft = torch.zeros(3, vocab)
    draft[1, 2] = 1.0            # both children share the draft distribution: all mass on token 2
    draft[2, 2] = 1.0
    tokens = torch.tensor([0, 2, 3])          # row 1: token 2 (draft argmax), row 2: token 3 (q == 0, p == 0)
    first_child = torch.tensor([1, -1, -1])
    next_sibling = torch.tensor([-1, 2, -1])
    uniform = torch.tensor([0.0, 0.5, 0.5])
    parent = torch.tensor([0])
    ref.verify_tree(draft, tokens, model, first_child, next_sibling, uniform, parent)
    assert int(parent[0]) == 0   # nothing accepted; the residual stays on token 4
    assert float(model[0, 4]) == 1.0


def test_generate_many_gathers_outputs_natively():
    """``generate_many`` lets the native stream-back thread gather each request's outputs (tokens,
    detokenised text, grammar-forced text in order) and delivers one merged result per request; the text
    equals what the streaming API returns."""
    eng = MLCEngine(MODEL, "cpu", mode="server",
                    engine_config=EngineConfig(max_num_sequence=8, prefill_chunk_size=64, max_total_sequence_length=2048))
    try:
        prompts = _prompts(5, seed=9)
        cfg = dict(GREEDY, max_tokens=9)
        res = eng.generate_many(prompts, cfg)
        assert [r["finish_reason"] for r in res] == ["length"] * 5
        assert all(r["usage"]["completion_tokens"] == 9 for r in res)
        for p, r in zip(prompts[:2], res[:2]):
            one = eng.completions.create(prompt=p, max_tokens=9, temperature=0.0, debug_config={"ignore_eos": True})
            assert one.choices[0].text == r["text"]
        # JSON mode: forced text arrives as strings between token runs; the merged text keeps the order
        schema = json.dumps({"type": "object", "properties": {"name": {"type": "string"}}, "required": ["name"]})
        jcfg = {"max_tokens": 24, "temperature": 0.0, "response_format": {"type": "json_object", "schema": schema}}
        merged = eng.generate_many(prompts[:2], jcfg)
        for p, r in zip(prompts[:2], merged):
            one = eng.completions.create(prompt=p, **jcfg)
            assert one.choices[0].text == r["text"]
        assert eng.generate_many([], cfg) == []
    finally:
        eng.terminate()


def test_request_objects_drive_the_step_loop(reference_outputs):
    """``create_request`` / ``add_request(request)`` / ``step`` with a stream callback that unpacks the
    outputs, as a caller of the low-level synchronous engine does."""
    from mlc_llm_b200.serve import data

    prompts, want = reference_outputs
    got = {}

    def on_outputs(outs):
        for out in outs:
            rid, singles = out.unpack()
            if singles[0].request_final_usage_json_str is None:
                got.setdefault(rid, []).extend(singles[0].delta_token_ids)

    cfg = EngineConfig(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64,
                       prefix_cache_mode="disable")
    eng = SyncMLCEngine(MODEL, "cpu", engine_config=cfg, request_stream_callback=on_outputs)
    for i in range(2):
        req = eng.create_request(f"r{i}", data.TokenData(prompts[i]), dict(GREEDY, max_tokens=12))
        eng.add_request(req)
    while not eng.empty():
        eng.step()
    assert [got["r0"], got["r1"]] == want[:2]


def test_declined_deferred_step_keeps_the_fork_page_copies():
    """Parallel samples fork the prompt's sequence; the copy of its last partial page rides on the next plan.
    When that plan is a deferred-read decode step the backend declines (pipeline stages, draft heads, recurrent
    models do), the engine pops the step and plans again: the copies must ride on the new plan."""
    prompt = _prompts(1, lo=40, hi=41, seed=9)[0]       # 40 tokens: two full pages and eight rows of a third
    _, want = _engine(prefix_cache_mode="disable").generate([prompt], dict(GREEDY, max_tokens=6))
    eng = _engine(prefix_cache_mode="disable")
    ex = eng.runtime.executor
    seen = {"declined": [], "sync": []}
    orig = ex._forward_sample

    def sync(model_id, plan, token_ids, embed_handles, sp):
        seen["sync"].append(list(map(int, plan["page_copies"])))
        return orig(model_id, plan, token_ids, embed_handles, sp)

    def launch(model_id, plan, token_ids, token_src, sp):
        seen["declined"].append(list(map(int, plan["page_copies"])))
        return False

    ex._forward_sample, ex.forward_sample_launch = sync, launch
    _, got = eng.generate([prompt], dict(GREEDY, max_tokens=6, n=2))
    assert got[0] == [want[0][0], want[0][0]]
    assert len(seen["declined"]) == 1 and len(seen["declined"][0]) == 4     # two (source, destination) pairs
    assert seen["declined"][0] in seen["sync"]


def test_concurrent_disaggregated_hand_offs_and_plain_requests():
    """Four client threads drive eight requests against one prefill and one decode engine: six go through
    prepare_receive / remote_send / start_generation (half of them share a 48-token stem, so the decode side's
    prefix cache shortens what is sent), two are ordinary requests to the decode engine in between. Every text
    equals the plain engine's."""
    import concurrent.futures as cf

    from mlc_llm_b200.serve.entrypoints.microserving_entrypoints import prep_recv_response

    cfg = dict(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64)
    plain = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**cfg))
    p_eng = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**cfg))
    d_eng = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**cfg))
    rng = np.random.default_rng(5)
    stem = rng.integers(10, 31000, 48).tolist()
    prompts = [(stem if i % 2 else []) + rng.integers(10, 31000, int(rng.integers(5, 70))).tolist() for i in range(8)]
    greedy = dict(max_tokens=10, temperature=0.0)

    def run(i):
        prompt, rid = prompts[i], f"dis-{i}"
        if i % 4 == 3:
            return d_eng.completions.create(prompt=prompt, debug_config={"ignore_eos": True}, **greedy).choices[0].text
        prep = d_eng.completions.create(prompt=prompt, max_tokens=1, request_id=rid, debug_config={
            "disagg_config": {"kind": "prepare_receive", "kv_window_begin": 0, "kv_window_end": -1}})
        meta = prep_recv_response(d_eng, prep)
        end = len(prompt) - 1
        if meta.prefix_matched_length < end:
            p_eng.completions.create(prompt=prompt, max_tokens=1, request_id=rid, debug_config={
                "disagg_config": {"kind": "remote_send", "kv_window_begin": meta.prefix_matched_length,
                                  "kv_window_end": end, "kv_append_metadata": meta.kv_append_metadata,
                                  "dst_group_offset": 0}})
        out = d_eng.completions.create(prompt=prompt, request_id=rid, debug_config={
            "ignore_eos": True, "disagg_config": {"kind": "start_generation", "kv_window_begin": end}}, **greedy)
        return out.choices[0].text

    try:
        want = [plain.completions.create(prompt=p, debug_config={"ignore_eos": True}, **greedy).choices[0].text
                for p in prompts]
        with cf.ThreadPoolExecutor(4) as pool:
            got = list(pool.map(run, range(len(prompts))))
        assert got == want
    finally:
        for e in (plain, p_eng, d_eng):
            e.terminate()


def test_async_streams_with_random_cancellations():
    """Sixteen concurrent streams; a third of them are aborted after a random number of chunks (some right away,
    some through cancellation of the consuming task). The survivors' texts equal what the same prompts give one
    by one, and the engine answers a fresh request afterwards."""
    rng = np.random.default_rng(77)
    prompts = _prompts(16, seed=50)
    lengths = [int(rng.integers(4, 30)) for _ in prompts]
    kill_after = [int(rng.integers(0, 5)) if rng.random() < 0.33 else None for _ in prompts]
    eng = AsyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(mode="server", max_num_sequence=6,
                                                                  max_total_sequence_length=1024,
                                                                  prefill_chunk_size=48))
    greedy = dict(temperature=0.0, debug_config={"ignore_eos": True})

    async def run():
        async def one(i):
            text, chunks = "", 0
            stream = await eng.completions.create(prompt=prompts[i], max_tokens=lengths[i], stream=True,
                                                  request_id=f"s{i}", **greedy)
            async for chunk in stream:
                text += "".join(ch.text for ch in chunk.choices)
                chunks += 1
                if kill_after[i] is not None and chunks > kill_after[i]:
                    await eng.abort(f"s{i}")
                    break
            await stream.aclose()
            return text

        tasks = [asyncio.ensure_future(one(i)) for i in range(len(prompts))]
        await asyncio.sleep(0.05)
        tasks[3].cancel()                      # a consumer that simply goes away
        results = await asyncio.gather(*tasks, return_exceptions=True)
        await eng.abort("s3")
        alone = []
        for i in range(len(prompts)):
            out = await eng.completions.create(prompt=prompts[i], max_tokens=lengths[i], **greedy)
            alone.append(out.choices[0].text)
        return results, alone

    try:
        results, alone = asyncio.run(asyncio.wait_for(run(), timeout=240))
    finally:
        eng.terminate()
    for i, (got, want) in enumerate(zip(results, alone)):
        if i == 3:
            continue
        assert isinstance(got, str), (i, got)
        if kill_after[i] is None:
            assert got == want, i
        else:
            assert want.startswith(got), i


@pytest.mark.parametrize("spec", [dict(spec_draft_length=4), dict(spec_draft_length=3, spec_tree_width=2)])
def test_fully_accepted_drafts_stop_where_plain_decoding_stops(spec, reference_outputs):
    """A draft model with the target's own weights: every proposal is accepted, so several tokens are committed per
    verification. A stop token or the length limit that falls inside such a run must end the request at the same
    token as one-by-one decoding."""
    prompts, _ = reference_outputs
    prompts = prompts[:3]
    plain = _engine(prefix_cache_mode="disable")
    eng = _engine(prefix_cache_mode="disable", speculative_mode="small_draft", additional_models=[MODEL], **spec)
    _, full = plain.generate(prompts, dict(GREEDY, max_tokens=20))
    for i, p in enumerate(prompts):
        for cut in (5, 6, 7, 11):
            gen = dict(GREEDY, max_tokens=20, stop_token_ids=[int(full[i][0][cut])])
            assert eng.generate([p], gen)[1][0][0] == plain.generate([p], gen)[1][0][0], (i, cut)
    for max_tokens in (1, 2, 3, 5, 6, 7):
        gen = dict(GREEDY, max_tokens=max_tokens)
        assert [t[0] for t in eng.generate(prompts, gen)[1]] == [t[0][:max_tokens] for t in full]
    stats = json.loads(eng.debug_stats())
    assert stats["num_verify_steps"] > 0
