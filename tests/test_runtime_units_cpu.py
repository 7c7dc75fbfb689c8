"""Unit tests of the native runtime pieces and the artifact code (no model, no GPU)."""
import json

import numpy as np
import pytest
import torch

from mlc_llm_b200 import _core
from mlc_llm_b200 import quantization as Q
from mlc_llm_b200.conversation_template import ConvTemplateRegistry
from mlc_llm_b200.loader.tensor_cache import TensorCache, dump_tensor_cache
from mlc_llm_b200.protocol import openai_api_protocol as openai
from mlc_llm_b200.protocol.conversation_protocol import Conversation
from mlc_llm_b200.tokenizers import StopStrHandler, TextStreamer, Tokenizer


# ------------------------------------------------------------------ KV manager
def test_kv_manager_append_fork_cow_popn():
    kv = _core.KVManager(32, 16, 8)
    kv.add_sequence(0)
    plan = kv.begin_forward([0], [20])
    assert list(plan["positions"]) == list(range(20))
    assert kv.sequence_length(0) == 20 and len(kv.sequence_pages(0)) == 2
    slots = np.asarray(plan["slots"])
    pages = kv.sequence_pages(0)
    assert list(slots[:16] // 16) == [pages[0]] * 16 and list(slots[16:] // 16) == [pages[1]] * 4
    # fork shares the full pages; the partial last page gets a private copy, emitted with the next plan
    free_before = kv.num_available_pages()
    kv.fork_sequence(0, 1)
    child_pages = kv.sequence_pages(1)
    assert child_pages[0] == pages[0] and child_pages[1] != pages[1]
    assert kv.num_available_pages() == free_before - 1
    plan = kv.begin_forward([1], [1])
    copies = np.asarray(plan["page_copies"]).reshape(-1, 2)
    assert copies.tolist() == [[pages[1], child_pages[1]]]
    assert kv.sequence_length(1) == 21 and kv.sequence_length(0) == 20
    # the parent keeps appending into its own page without a copy
    plan = kv.begin_forward([0], [1])
    assert len(plan["page_copies"]) == 0
    kv.popn(1, 6)
    assert kv.sequence_length(1) == 15 and len(kv.sequence_pages(1)) == 1
    kv.remove_sequence(1)
    kv.remove_sequence(0)
    assert kv.num_available_pages() == 32 and kv.num_sequences() == 0


def test_kv_manager_batch_plan_layout_and_exhaustion():
    kv = _core.KVManager(4, 16, 8)
    for i in range(2):
        kv.add_sequence(i)
    plan = kv.begin_forward([0, 1], [3, 18])
    assert list(plan["q_indptr"]) == [0, 3, 21]
    assert list(plan["q_seq"]) == [0] * 3 + [1] * 18
    assert list(plan["q_kvlen"])[:3] == [1, 2, 3] and list(plan["q_kvlen"])[-1] == 18
    assert list(plan["page_indptr"]) == [0, 1, 3]
    assert kv.num_available_pages() == 1
    assert kv.pages_needed(0, 13) == 0 and kv.pages_needed(0, 14) == 1 and kv.pages_needed(1, 15) == 1
    with pytest.raises(Exception):
        kv.begin_forward([0, 1], [40, 40])


def test_kv_manager_tree_append_and_commit():
    kv = _core.KVManager(16, 16, 4)
    kv.add_sequence(0)
    kv.begin_forward([0], [5])
    # verify step: root + chain of 3 draft tokens, all appended speculatively
    plan = kv.begin_forward([0], [4], tree_parents=[-1, 0, 1, 2])
    assert list(plan["positions"]) == [5, 6, 7, 8]
    assert len(plan["tree_mask"]) == 4
    # keep root + the first two draft nodes
    moves = kv.commit_tree_nodes(0, 4, [0, 1, 2])
    assert kv.sequence_length(0) == 8 and list(moves) == []  # a chain prefix is already in place
    # branching tree: root, two children of the root, a grandchild under the second child
    plan = kv.begin_forward([0], [4], tree_parents=[-1, 0, 0, 2])
    assert list(plan["positions"]) == [8, 9, 9, 10]
    moves = kv.commit_tree_nodes(0, 4, [0, 2, 3])
    assert kv.sequence_length(0) == 11
    # accepted nodes 2 and 3 sat in slots 2 and 3 of the append and move down to slots 1 and 2
    assert len(moves) == 4


def test_kv_manager_sliding_window_releases_pages():
    kv = _core.KVManager(64, 16, 4)
    kv.add_sequence(0)
    kv.enable_sliding_window(0, 32, 4)
    for _ in range(10):
        plan = kv.begin_forward([0], [16])
    assert kv.sequence_length(0) == 160
    live = [p for p in kv.sequence_pages(0) if p >= 0]
    assert len(live) <= 5 and kv.num_available_pages() >= 64 - 5  # sink page + window pages, not 10
    assert len(plan["q_kvstart"]) == 16


def test_kv_manager_window_keeps_what_the_first_token_of_a_chunk_sees():
    """A chunk longer than the window: its first token still attends `window` positions back, so only pages
    below that may go when the chunk is appended."""
    kv = _core.KVManager(64, 16, 4)
    kv.add_sequence(0)
    kv.enable_sliding_window(0, 32, 0)
    kv.begin_forward([0], [64])
    plan = kv.begin_forward([0], [64])          # positions 64..127
    pages = kv.sequence_pages(0)
    first_start = int(plan["q_kvstart"][0])     # 64 + 1 - 32 = 33
    assert first_start == 33
    assert all(p >= 0 for p in pages[first_start // 16:])   # page 2 (positions 32..47) onwards are live
    assert pages[0] < 0 and pages[1] < 0                    # positions 0..31 are dead for every token
    plan = kv.begin_forward([0], [1])           # position 128: sees 97..128
    pages = kv.sequence_pages(0)
    assert all(p < 0 for p in pages[:6]) and all(p >= 0 for p in pages[6:])


def test_kv_manager_forks_of_a_windowed_sequence_inherit_the_window():
    """Parallel samples of a windowed sequence: the child shares the live pages (reference counts), carries the
    holes of the dropped ones, keeps the window for its own tokens, and both can be removed in any order. A fork
    at a position whose window reaches into dropped pages is refused."""
    import pytest as _pytest

    kv = _core.KVManager(64, 16, 8)
    kv.add_sequence(0)
    kv.enable_sliding_window(0, 32, 0)
    kv.begin_forward([0], [100])
    kv.begin_forward([0], [1])                   # position 100 sees 69..100: pages 0..3 (positions 0..63) are gone
    parent_pages = kv.sequence_pages(0)
    assert all(p < 0 for p in parent_pages[:4]) and all(p >= 0 for p in parent_pages[4:])
    free_before = kv.num_available_pages()
    kv.fork_sequence(0, 1, -1)
    child_pages = kv.sequence_pages(1)
    assert child_pages[:6] == parent_pages[:6] and child_pages[6] != parent_pages[6]   # last partial page copied
    assert kv.num_available_pages() == free_before - 1
    plan = kv.begin_forward([1], [1])            # the child's token at position 101 sees 70..101
    assert int(plan["q_kvstart"][0]) == 70
    for _ in range(40):
        kv.begin_forward([1], [1])
    assert all(p < 0 for p in kv.sequence_pages(1)[:6])          # the child's window moved on by itself
    assert all(p >= 0 for p in kv.sequence_pages(0)[4:])         # the parent still holds what it sees
    with _pytest.raises(RuntimeError):
        kv.fork_sequence(0, 2, 80)               # a token at position 80 would see 49..80: page 3 is gone
    kv.fork_sequence(0, 3, 96)                   # position 96 sees 65..96: all there
    kv.remove_sequence(0)
    kv.remove_sequence(1)
    kv.remove_sequence(3)
    assert kv.num_available_pages() == 64


# ------------------------------------------------------------------ prefix cache
def test_prefix_cache_reuse_fork_and_recycle():
    removed = []
    pc = _core.PrefixCache(True, 2, removed.append)
    m = pc.insert_sequence(0, list(range(100)))
    assert m.prefilled_offset == 0 and m.forked_seq_id == -1 and m.reused_seq_id == -1
    pc.extend_sequence(0, list(range(100)))  # tokens enter the tree once they are prefilled
    # same prefix, different tail: fork from the live sequence
    tail = list(range(60)) + [7, 7, 7]
    m = pc.insert_sequence(1, tail)
    assert m.forked_seq_id == 0 and m.prefilled_offset == 60
    pc.extend_sequence(1, tail[60:])
    pc.recycle_sequence(0, True)
    assert pc.num_recycling() == 1 and not removed
    # a recycled sequence matching >= 90% of its length is reused as is (tail popped)
    reuse = list(range(95)) + [1, 2]
    m = pc.insert_sequence(2, reuse)
    assert m.reused_seq_id == 0 and m.reused_seq_pop_last_tokens == 5 and m.prefilled_offset == 95
    assert pc.num_recycling() == 0
    pc.extend_sequence(0, reuse[95:])  # the caller keeps using the reused id
    # recycling beyond the limit evicts the least recently used
    for sid in (0, 1):
        pc.recycle_sequence(sid, True)
    pc.insert_sequence(3, [900, 901])
    pc.extend_sequence(3, [900, 901])
    pc.recycle_sequence(3, True)
    assert pc.num_recycling() == 2 and len(removed) == 1
    assert pc.try_free_memory() and len(removed) == 2


def test_prefix_cache_disabled_never_matches():
    pc = _core.PrefixCache(False, 0, None)
    pc.insert_sequence(0, [1, 2, 3])
    m = pc.insert_sequence(1, [1, 2, 3])
    assert m.prefilled_offset == 0 and m.forked_seq_id == -1


# ------------------------------------------------------------------ configs
def test_generation_config_validation_and_defaults():
    g = _core.GenerationConfig.from_json(json.dumps({"temperature": 0.5, "top_p": 0.9, "n": 2, "max_tokens": 7}))
    d = json.loads(g.as_json())
    assert d["temperature"] == 0.5 and d["n"] == 2 and g.max_tokens == 7
    defaults = json.dumps({"temperature": 0.3, "top_p": 0.8, "repetition_penalty": 1.1})
    d = json.loads(_core.GenerationConfig.from_json("{}", defaults).as_json())
    assert d["temperature"] == pytest.approx(0.3) and d["top_p"] == pytest.approx(0.8)
    for bad in ({"temperature": -1}, {"top_p": 1.5}, {"frequency_penalty": 3}, {"n": 0}, {"top_logprobs": 9},
                {"logit_bias": {"5": 200}}, {"repetition_penalty": 0}):
        with pytest.raises(Exception):
            _core.GenerationConfig.from_json(json.dumps(bad))


def test_engine_config_inference_modes():
    model = {"params_bytes": 4 << 30, "num_layers": 32, "num_qo_heads": 32, "num_kv_heads": 8, "head_dim": 128,
             "vocab_size": 128256, "context_window_size": 8192, "prefill_chunk_size": 8192, "max_batch_size": 128}
    out = {}
    for mode in ("local", "interactive", "server"):
        r = _core.infer_capacity(json.dumps({"mode": mode}), [model], 180 << 30)
        out[mode] = json.loads(r["config_json"])
        assert r["num_pages"] * 16 >= out[mode]["max_total_sequence_length"]
        assert abs(r["kv_bytes_per_token"] - 2 * 32 * 8 * 128 * 2) < 4  # KV rows + page-table bookkeeping
    assert out["interactive"]["max_num_sequence"] == 1
    assert out["local"]["max_num_sequence"] == 4
    assert out["server"]["max_num_sequence"] >= 128
    assert out["server"]["max_total_sequence_length"] > out["local"]["max_total_sequence_length"]
    # explicit values are kept; impossible requests are rejected
    r = _core.infer_capacity(json.dumps({"mode": "server", "max_num_sequence": 9, "max_total_sequence_length": 4096}),
                             [model], 180 << 30)
    c = json.loads(r["config_json"])
    assert c["max_num_sequence"] == 9 and c["max_total_sequence_length"] == 4096
    with pytest.raises(Exception):
        _core.infer_capacity(json.dumps({"mode": "server"}), [model], 2 << 30)
    rt = json.loads(_core.engine_config_roundtrip(json.dumps({"mode": "server", "prefix_cache_mode": "disable",
                                                              "speculative_mode": "small_draft"})))
    assert rt["prefix_cache_mode"] == "disable" and rt["speculative_mode"] == "small_draft"


# ------------------------------------------------------------------ CPU sampler
def test_cpu_sampler_top_p_and_verify():
    p = np.asarray([0.5, 0.3, 0.15, 0.05], dtype=np.float32)
    assert _core.cpu_sample_top_p(p, 1.0, 0.0)[0] == 0
    assert _core.cpu_sample_top_p(p, 1.0, 0.79)[0] == 1
    assert _core.cpu_sample_top_p(p, 1.0, 0.99)[0] == 3
    # top_p 0.6 keeps {0, 1}: renormalised 0.625 / 0.375
    tok, prob = _core.cpu_sample_top_p(p, 0.6, 0.7)
    assert tok == 1 and prob == pytest.approx(0.3, abs=1e-5)  # reported on the unrenormalised distribution
    q = p.copy()
    _core.cpu_renormalize_top_p(q, 0.6)
    assert q[2] == 0 and q[3] == 0 and q.sum() == pytest.approx(1.0)
    # chain verification: draft token accepted when u < min(1, p/q), else resample from max(p - q, 0)
    model = np.asarray([[0.1, 0.9, 0.0], [0.6, 0.2, 0.2], [0.3, 0.3, 0.4]], dtype=np.float32)
    draft = np.asarray([[0.5, 0.5, 0.0], [0.1, 0.8, 0.1]], dtype=np.float32)
    accepted, final = _core.cpu_verify_chain(model.copy(), draft, [1, 1], [0.5, 0.9], 0.0)
    assert accepted == 1          # second draft token: p/q = 0.25 < 0.9 -> rejected
    assert final == 0             # residual max(p - q, 0) = [0.5, 0, 0.1] -> u = 0 picks token 0
    accepted, final = _core.cpu_verify_chain(model.copy(), draft, [1, 1], [0.5, 0.1], 0.99)
    assert accepted == 2 and final == 2  # all accepted: bonus token from the last row


# ------------------------------------------------------------------ tokenizer glue
def test_text_streamer_handles_split_utf8_and_stop_strings():
    tok = Tokenizer.synthetic(1000)
    ids = tok.encode("héllo wörld ✓ done")
    st = TextStreamer(tok)
    pieces = [st.put([i]) for i in ids] + [st.finish()]
    assert "".join(pieces) == tok.decode(ids)
    assert all("�" not in p for p in pieces[:-1])
    handler = StopStrHandler(["wör"], tok)
    out = []
    for i in ids:
        out.extend(handler.put(i))
        if handler.stop_triggered:
            break
    assert handler.stop_triggered
    assert tok.decode(out) == "héllo "


def test_tokenizer_info_detection():
    info = json.loads(_core.detect_tokenizer_info(json.dumps(
        {"decoder": {"type": "ByteLevel"}, "normalizer": None, "model": {"type": "BPE"}})))
    assert info["token_postproc_method"] == "byte_level"
    info = json.loads(_core.detect_tokenizer_info(json.dumps(
        {"decoder": {"type": "Sequence", "decoders": [{"type": "Replace"}, {"type": "ByteFallback"}]},
         "normalizer": {"type": "Prepend", "prepend": "▁"}, "model": {"type": "BPE"}})))
    assert info["token_postproc_method"] == "byte_fallback" and info["prepend_space_in_encode"]
    assert _core.post_process_token("<0x41>", "byte_fallback") == b"A"
    assert _core.post_process_token("▁hi", "byte_fallback") == b" hi"
    assert _core.post_process_token("Ġhi", "byte_level") == b" hi"


def test_tokenizer_continuation_encode_and_prefix_mask():
    """Helpers of jump-forward decoding: encoding a continuation without the SentencePiece-style
    leading space, and the mask of tokens that are prefixes of other tokens."""
    vocab = ["<unk>", "<0x01>", "▁", "a", "ab", "▁ab", "c", "abc"]

    def encode(text):  # greedy longest match over the post-processed bytes, space prepended
        table = {"\x01": 1, " ": 2, "a": 3, "ab": 4, " ab": 5, "c": 6, "abc": 7}
        text = " " + text
        out = []
        while text:
            for n in range(len(text), 0, -1):
                if text[:n] in table:
                    out.append(table[text[:n]])
                    text = text[n:]
                    break
            else:
                text = text[1:]
        return out

    info = {"token_postproc_method": "byte_fallback", "prepend_space_in_encode": True,
            "strip_space_in_decode": False}
    tok = _core.Tokenizer(vocab, json.dumps(info), encode, [])
    assert tok.encode("ab") == [5]                    # " ab"
    assert tok.encode_no_prepend_space("abc") == [7]  # no leading space this time
    mask = tok.prefix_token_mask()
    assert mask[3] and mask[4] and not mask[7] and not mask[6]  # "a" < "ab" < "abc"; "c", "abc" are not
    assert mask[2]                                    # " " is a prefix of " ab"


# ------------------------------------------------------------------ event trace
def test_event_trace_recorder_chrome_json():
    rec = _core.EventTraceRecorder()
    rec.add_event("req-1", "start prefill")
    rec.add_event("req-1", "finish prefill")
    rec.add_event_batch(["req-1", "req-2"], "decode")
    events = json.loads(rec.dump_json())
    names = [e["name"] for e in events]
    assert len(events) == 4 and "decode" in "".join(names)
    assert all({"ts", "ph", "pid"} <= set(e) for e in events)
    # a start/finish pair becomes a begin/end pair on the request's own track
    phases = [e["ph"] for e in events if e["name"].endswith("prefill")]
    assert phases == ["B", "E"]
    rec.clear()
    assert json.loads(rec.dump_json()) == []


# ------------------------------------------------------------------ conversation templates
def test_conversation_templates_python_and_native_agree():
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"},
            {"role": "assistant", "content": "Hello."}, {"role": "user", "content": "Bye"}]
    for name in ("llama-3", "chatml", "llama-2", "mistral_default", "gemma_instruction", "phi-3", "qwen2",
                 "deepseek", "LM"):
        conv = ConvTemplateRegistry.get_conv_template(name)
        assert conv is not None, name
        c = Conversation.from_json_dict(conv.to_json_dict())
        c.messages = []
        for m in msgs:
            if m["role"] == "system":
                c.system_message = m["content"]
            else:
                c.messages.append((m["role"], m["content"]))
        c.messages.append(("assistant", None))
        py = "".join(p for p in c.as_prompt() if isinstance(p, str))
        native = _core.conv_template_render(json.dumps(conv.to_json_dict()), json.dumps(msgs))
        assert py == native, name
    llama3 = ConvTemplateRegistry.get_conv_template("llama-3")
    out = _core.conv_template_render(json.dumps(llama3.to_json_dict()), json.dumps(msgs[1:2]))
    assert out.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n") and "Hi<|eot_id|>" in out
    assert len(ConvTemplateRegistry.names()) >= 45


# ------------------------------------------------------------------ protocol
def test_openai_protocol_validation():
    req = openai.ChatCompletionRequest(messages=[{"role": "user", "content": "x"}], logprobs=True, top_logprobs=3)
    assert req.top_logprobs == 3
    legacy = openai.CompletionRequest(prompt="x", logprobs=4)       # legacy completions form: a count
    assert legacy.logprobs is True and legacy.top_logprobs == 4 and legacy.legacy_logprobs
    plain = openai.CompletionRequest(prompt="x")
    assert plain.logprobs is False and not plain.legacy_logprobs
    assert openai.CompletionRequest(prompt="x", logprobs=True, top_logprobs=2).legacy_logprobs is False
    with pytest.raises(ValueError):
        openai.CompletionRequest(prompt="x", logprobs=6)             # at most five alternatives
    with pytest.raises(Exception):
        openai.ChatCompletionRequest(messages=[{"role": "user", "content": "x"}], top_logprobs=3)  # needs logprobs
    with pytest.raises(Exception):
        openai.ChatCompletionRequest(messages=[{"role": "user", "content": "x"}], logprobs=True, top_logprobs=30)
    with pytest.raises(Exception):
        openai.ChatCompletionRequest(messages=[{"role": "system", "content": "a"}, {"role": "system", "content": "b"},
                                               {"role": "user", "content": "x"}]).check_message_validity()
    r = openai.CompletionRequest(prompt=[1, 2, 3], response_format={"type": "json_object", "schema": "{}"})
    assert r.response_format.json_schema == "{}"
    with pytest.raises(Exception):
        openai.CompletionRequest(prompt="x", response_format={"type": "yaml"})


# ------------------------------------------------------------------ artifacts
@pytest.mark.parametrize("name", ["q4f16_1", "q4f16_0", "q3f16_1", "q4bf16_1", "q4f32_1"])
def test_group_quantization_round_trip(name):
    q = Q.get(name)
    torch.manual_seed(0)
    w = torch.randn(64, 160) * 0.1
    qw, qs = Q.group_quantize(w, q)
    assert qw.dtype == torch.int32 and qw.shape[0] == 64
    back = Q.group_dequantize(qw, qs, q, k=160).float()
    step = w.abs().amax() / q.max_int
    assert (back - w).abs().max() <= step * 0.6 + 1e-3
    if q.bits == 4 and q.group_size == 32:
        assert qw.shape[1] == 160 // 8 and qs.shape == (64, 5)
        # device nibble order is a pure permutation of the packed words
        assert torch.equal(Q.from_device_layout_q4(Q.to_device_layout_q4(qw)), qw)


def test_fp8_block_scale_round_trip():
    w = torch.randn(256, 384) * 0.05
    qw, sc = Q.fp8_block_quantize(w, (128, 128), "float8_e4m3fn")
    assert qw.dtype == torch.float8_e4m3fn and sc.shape == (2, 3)
    back = Q.fp8_block_dequantize(qw, sc, (128, 128)).float()
    assert (back - w).abs().max() < 0.07 * w.abs().max()


def test_tensor_cache_round_trip_and_md5(tmp_path):
    torch.manual_seed(1)
    tensors = {"a.weight": torch.randn(300, 70).half(), "b.q_weight": torch.randint(-2**31, 2**31 - 1, (64, 9), dtype=torch.int64).to(torch.int32),
               "c.scale": torch.randn(7).bfloat16(), "d.bias": torch.randn(33), "e.fp8": torch.randn(16, 16).to(torch.float8_e4m3fn)}
    doc = dump_tensor_cache(iter(tensors.items()), str(tmp_path), shard_bytes=32 * 1024)
    assert len(doc["records"]) >= 2 and doc["metadata"]["ParamSize"] == sum(t.numel() for t in tensors.values())
    cache = TensorCache(str(tmp_path), verify_md5=True)
    got = dict(iter(cache))
    assert set(got) == set(tensors)
    for k in ("a.weight", "b.q_weight", "c.scale"):
        assert torch.equal(got[k], tensors[k])
    assert torch.equal(got["e.fp8"].view(torch.uint8), tensors["e.fp8"].view(torch.uint8))
    # float32 is stored as bf16 ("f32-to-bf16", round to nearest even) and widened on load
    assert torch.equal(got["d.bias"], tensors["d.bias"].bfloat16().float())
    shard = tmp_path / doc["records"][0]["dataPath"]
    data = bytearray(shard.read_bytes())
    data[0] ^= 0xFF
    shard.write_bytes(bytes(data))
    with pytest.raises(ValueError):
        list(TensorCache(str(tmp_path), verify_md5=True))


def test_tensor_cache_bf16_rounding_and_updated_totals(tmp_path):
    from mlc_llm_b200.loader.tensor_cache import update_tensor_cache

    # values exactly between two bf16 neighbours (ties go to the even mantissa), just above and just
    # below the midpoint, negative ones, and the specials
    bits = torch.tensor([0x3F808000, 0x3F818000, 0x3F808001, 0x3F807FFF, 0xBF808000 - (1 << 32), 0x7F800000,
                         0x7F7FFFFF, 0x00000001, 0x80000000 - (1 << 32)], dtype=torch.int64).to(torch.int32)
    vals = bits.view(torch.float32)
    nan = torch.tensor([float("nan")])
    dump_tensor_cache(iter({"x": vals, "n": nan}.items()), str(tmp_path))
    got = dict(iter(TensorCache(str(tmp_path))))
    want = vals.bfloat16().float()
    assert torch.equal(got["x"].view(torch.int32), want.view(torch.int32))
    assert got["x"][0].item() == 1.0 and got["x"][1].view(torch.int32).item() == 0x3F820000   # ties to even
    assert bool(torch.isnan(got["n"]).all())
    doc = update_tensor_cache(iter({"x": torch.randn(40), "extra": torch.ones(3, 5).half()}.items()), str(tmp_path))
    live = dict(iter(TensorCache(str(tmp_path))))
    assert doc["metadata"]["ParamSize"] == sum(t.numel() for t in live.values()) == 40 + 15 + 1
    assert doc["metadata"]["ParamBytes"] == 40 * 2 + 15 * 2 + 2


def test_reference_module_paths_and_stream_output_unpack():
    """Names a user of the reference imports: module paths, request objects, stream-output unpacking."""
    from mlc_llm_b200.serve import data
    from mlc_llm_b200.serve.engine import AsyncChat, Chat  # noqa: F401
    from mlc_llm_b200.serve.event_trace_recorder import EventTraceRecorder
    from mlc_llm_b200.serve.radix_tree import PagedRadixTree
    from mlc_llm_b200.serve.request import Request
    from mlc_llm_b200.tokenizers.streamer import StopStrHandler, TextStreamer  # noqa: F401
    from mlc_llm_b200.tokenizers.tokenizers import Tokenizer  # noqa: F401

    tree = PagedRadixTree()
    tree.add(0)
    tree.extend(0, [1, 2, 3])
    assert tree.match([1, 2, 9])[0] == 2 and tree.get_length(0) == 3
    rec = EventTraceRecorder()
    rec.add_event("r0", "start")
    assert "r0" in rec.dump_json()
    req = Request("r0", [data.TokenData([1, 2])], {"max_tokens": 2})
    assert req.inputs[0].token_ids == [1, 2]
    out = data.RequestStreamOutput({"request_id": "r0", "group_delta_token_ids": [[4], [5, 6]],
                                    "group_delta_logprob_json_strs": [[], []], "group_finish_reason": [None, "stop"],
                                    "group_extra_prefix_string": ["", "x"], "request_final_usage_json_str": None})
    rid, singles = out.unpack()
    assert rid == "r0" and [s.delta_token_ids for s in singles] == [[4], [5, 6]]
    assert singles[1].finish_reason == "stop" and singles[1].extra_prefix_string == "x"
    last = data.RequestStreamOutput({"request_id": "r0", "group_delta_token_ids": [], "group_delta_logprob_json_strs": [],
                                     "group_finish_reason": [], "group_extra_prefix_string": [],
                                     "request_final_usage_json_str": "{}"})
    assert last.unpack()[1][0].request_final_usage_json_str == "{}"
    cfg = {"model_config": {"vision_config": {"image_size": 336, "patch_size": 14}}}
    assert data.ImageData.get_embed_size(cfg) == 576 and data.ImageData.get_input_size(cfg) == 336


def test_q4_tile_records_decode_to_the_dequantised_weight():
    """The GPU GEMM's int4 tile records, decoded on the host exactly as the kernel's dequant threads do
    (two 16-byte nibble words and one scale pair per row and K block; nibble q under exponent 0x6400 is
    1024 + q, under 0x5400 it is 64 + q), give back ``(q - 7) * scale``."""
    import numpy as np

    from mlc_llm_b200 import quantization as Q

    torch.manual_seed(3)
    quant = Q.get("q4f16_1")
    n, k = 200, 192                       # rows pad to 256: two row blocks, three K blocks
    w = (torch.randn(n, k) * 0.05).half()
    qw, qs = Q.group_quantize(w, quant)
    want = Q.group_dequantize(qw, qs, quant, k=k).float().numpy()
    tiles = Q.to_tiled_q4(Q.to_device_layout_q4(qw), qs)
    assert tuple(tiles.shape) == (2, 3, Q.Q4_TILE_BYTES) and tiles.dtype == torch.uint8
    raw = tiles.numpy()
    got = np.zeros((256, k), dtype=np.float32)
    for nb in range(2):
        for kb in range(3):
            rec = raw[nb, kb]
            nib = rec[:4096].view(np.uint32).reshape(2, 128, 4)
            scl = rec[4096:].view(np.float16).reshape(128, 2)
            for half in range(2):
                x = nib[half].astype(np.uint32)                    # [128 rows, 4 words]
                y = x >> np.uint32(8)
                v = np.stack([(x & 0x000F000F) | 0x64006400, (x & 0x00F000F0) | 0x54005400,
                              (y & 0x000F000F) | 0x64006400, (y & 0x00F000F0) | 0x54005400], axis=-1)
                h = v.astype(np.uint32).view(np.float16).reshape(128, 4, 4, 2).astype(np.float32)
                h[:, :, 0::2, :] -= 1031.0
                h[:, :, 1::2, :] -= 71.0
                vals = h.reshape(128, 32) * scl[:, half:half + 1].astype(np.float32)
                got[nb * 128:(nb + 1) * 128, kb * 64 + half * 32: kb * 64 + half * 32 + 32] = vals
    assert np.array_equal(got[:n].astype(np.float16), want.astype(np.float16))
    assert not got[n:].any()               # padding rows decode to zero


def test_awq_checkpoint_tensors_expand_to_the_dense_weight(tmp_path):
    """AutoAWQ layout (packed columns in the order 0 2 4 6 1 3 5 7 per word, per-group zero points): the
    loader offers ``<layer>.weight`` for a (qweight, qzeros, scales) triple."""
    from safetensors.torch import save_file

    from mlc_llm_b200 import quantization as Q
    from mlc_llm_b200.loader.huggingface_loader import HFCheckpoint

    torch.manual_seed(9)
    k, n, g = 256, 64, 128
    q = torch.randint(0, 16, (k, n))
    z = torch.randint(0, 16, (k // g, n))
    s = (torch.rand(k // g, n) * 0.02 + 0.001).half()
    want = ((q.float() - z.repeat_interleave(g, 0).float()) * s.float().repeat_interleave(g, 0)).t().half()
    qweight, qzeros = Q.awq_pack(q), Q.awq_pack(z)
    # spot-check the nibble order: output column 1 of a word sits in bits 16..19
    assert ((int(qweight[0, 0]) & 0xFFFFFFFF) >> 16) & 0xF == int(q[0, 1])
    assert torch.equal(Q.awq_dequantize(qweight, qzeros, s), want)
    save_file({"model.layers.0.mlp.down_proj.qweight": qweight, "model.layers.0.mlp.down_proj.qzeros": qzeros,
               "model.layers.0.mlp.down_proj.scales": s, "model.norm.weight": torch.ones(n).half()},
              str(tmp_path / "model.safetensors"))
    ck = HFCheckpoint(str(tmp_path))
    assert torch.equal(ck.get("model.layers.0.mlp.down_proj.weight"), want)
    assert torch.equal(ck.get("model.norm.weight"), torch.ones(n).half())
    with pytest.raises(ValueError):
        Q.get("q4f16_ft")
    assert Q.get("q4f16_autoawq").kind == "no-quant"


def test_decode_batches_are_padded_to_graph_buckets():
    """Stand-in sequences appended to a pure decode step: consistent index arrays, nothing written to the
    cache (slot -1), one readable token each."""
    import numpy as np

    from mlc_llm_b200.serve.executor import graph_bucket, pad_decode_arrays

    assert [graph_bucket(n) for n in range(1, 10)] == [1, 2, 4, 4, 8, 8, 8, 8, 16]
    assert graph_bucket(33) == 48 and graph_bucket(256) == 256 and graph_bucket(257) == 272
    n = 5
    i32 = np.int32
    arrays = {
        "token_ids": np.arange(10, 10 + n, dtype=i32), "positions": np.array([7, 3, 20, 1, 16], i32),
        "slots": np.array([23, 35, 68, 81, 96], i32), "q_seq": np.arange(n, dtype=i32),
        "q_kvlen": np.array([8, 4, 21, 2, 17], i32), "page_indptr": np.array([0, 1, 2, 4, 5, 7], i32),
        "page_indices": np.array([1, 2, 3, 4, 5, 6, 7], i32), "q_indptr": np.arange(n + 1, dtype=i32),
        "seq_lens": np.array([8, 4, 21, 2, 17], i32), "append_lens": np.ones(n, i32),
        "token_src": np.array([0, -1, 2, 3, -1], i32),
    }
    before = {k: v.copy() for k, v in arrays.items()}
    pad_decode_arrays(arrays, graph_bucket(n))
    for k, v in before.items():
        assert (arrays[k][: v.size] == v).all() and arrays[k].dtype == i32
    assert arrays["token_ids"].size == 8 and arrays["q_indptr"].tolist() == list(range(9))
    assert arrays["slots"][n:].tolist() == [-1] * 3 and arrays["token_src"][n:].tolist() == [-1] * 3
    assert arrays["page_indptr"].tolist() == [0, 1, 2, 4, 5, 7, 8, 9, 10]
    assert arrays["page_indices"].size == 10 and arrays["q_kvlen"][n:].tolist() == [1, 1, 1]
    assert arrays["q_seq"].tolist() == list(range(8))
    pad_decode_arrays(arrays, 8)  # already at the bucket: unchanged
    assert arrays["token_ids"].size == 8


def test_recurrent_state_capacity_inference():
    """Batch size, token capacity and snapshot count of a recurrent-state model from the memory left beside the
    weights; a per-sequence length limit is refused."""
    import json

    import pytest

    from mlc_llm_b200 import _core

    info = {"params_bytes": 3 << 30, "num_layers": 24, "vocab_size": 65536, "prefill_chunk_size": 8192,
            "max_batch_size": 80, "hidden_size": 2048, "rnn_state_bytes_per_sequence": 24 * (2 * 2048 * 2 + 32 * 64 * 64 * 4)}

    def infer(total, **cfg):
        base = {"kv_state_kind": "rnn_state", "mode": "local", "gpu_memory_utilization": 0.85}
        base.update(cfg)
        res = _core.infer_capacity(json.dumps(base), [info], int(total))
        return json.loads(res["config_json"]), res

    c, res = infer(16 << 30)
    assert c["max_num_sequence"] == 4 and c["prefill_chunk_size"] == 4096 and c["max_total_sequence_length"] == 32768
    per_snapshot = 4 * info["rnn_state_bytes_per_sequence"]
    assert 0 < c["max_history_size"] <= ((16 << 30) * 0.85 - (3 << 30)) / per_snapshot
    assert c["max_history_size"] > ((16 << 30) * 0.85 - (3 << 30)) / per_snapshot * 0.8
    assert "recurrent state" in res["report"] and res["kv_bytes_per_token"] == 0
    c, _ = infer(16 << 30, mode="interactive", max_history_size=3)
    assert c["max_num_sequence"] == 1 and c["max_history_size"] == 3
    c, _ = infer(16 << 30, mode="server", max_num_sequence=64, max_total_sequence_length=100000)
    assert c["max_num_sequence"] == 64 and c["max_total_sequence_length"] == 100000
    with pytest.raises(Exception, match="max_single_sequence_length"):
        infer(16 << 30, max_single_sequence_length=4096)
    with pytest.raises(Exception, match="Insufficient GPU memory"):
        infer(3 << 30)


def test_split_plan_cuts_a_forward_at_a_sequence_boundary():
    """Both halves are self-contained plans (rebased indices), page copies go with the first, the logit rows are
    divided by sequence and the second half keeps the sampling parameters of every row."""
    import numpy as np

    from mlc_llm_b200 import _core
    from mlc_llm_b200.serve.executor import split_plan

    kv = _core.KVManager(64, 16, 8)
    for i in range(3):
        kv.add_sequence(i)
    lens = [20, 7, 33]
    plan = dict(kv.begin_forward([0, 1, 2], lens))
    plan["max_seq_len"] = 33
    toks = np.arange(60, dtype=np.int32)
    sp = {"logit_token_index": np.array([19, 26, 59], np.int32), "temperature": np.array([0.0, 0.5, 1.0], np.float32),
          "top_p": np.ones(3, np.float32), "uniform": np.zeros(3, np.float32), "top_k": np.zeros(3, np.int32),
          "penalties": np.zeros(0, np.float32), "pen_row": np.zeros(0, np.int32), "pen_token": np.zeros(0, np.int32),
          "pen_count": np.zeros(0, np.int32), "bias_row": np.zeros(0, np.int32), "bias_token": np.zeros(0, np.int32),
          "bias_value": np.zeros(0, np.float32), "mask_rows": np.zeros(0, np.int32), "mask_bits": np.zeros(0, np.int32),
          "prob_slots": np.zeros(0, np.int32), "num_top_logprobs": 0}
    (pa, ta, sa), (pb, tb, sb) = split_plan(plan, toks, sp, 2)
    assert ta.tolist() == list(range(27)) and tb.tolist() == list(range(27, 60))
    assert pa["q_indptr"].tolist() == [0, 20, 27] and pb["q_indptr"].tolist() == [0, 33]
    assert pa["q_seq"].tolist() == [0] * 20 + [1] * 7 and pb["q_seq"].tolist() == [0] * 33
    full_pi, full_pages = np.asarray(plan["page_indptr"]), np.asarray(plan["page_indices"])
    assert pa["page_indptr"].tolist() == full_pi[:3].tolist()
    assert pb["page_indptr"].tolist() == (full_pi[2:] - full_pi[2]).tolist()
    assert np.concatenate([pa["page_indices"], pb["page_indices"]]).tolist() == full_pages.tolist()
    assert np.concatenate([pa["slots"], pb["slots"]]).tolist() == np.asarray(plan["slots"]).tolist()
    assert pa["max_seq_len"] == 20 and pb["max_seq_len"] == 33
    assert sa["logit_token_index"].tolist() == [19, 26] and sb["logit_token_index"].tolist() == [32]
    assert len(sa["temperature"]) == 0 and sb["temperature"].tolist() == [0.0, 0.5, 1.0]
    assert len(pb["page_copies"]) == 0


def test_detect_weight_formats(tmp_path):
    """``--source-format awq`` names the container the AWQ triples sit in; a missing container is an error."""
    import pytest as _pytest

    from mlc_llm_b200.support.auto_config import detect_weight

    (tmp_path / "config.json").write_text("{}")
    with _pytest.raises(ValueError):
        detect_weight(str(tmp_path), str(tmp_path / "config.json"), "awq")
    (tmp_path / "model.safetensors").write_bytes(b"")
    assert detect_weight(str(tmp_path), str(tmp_path / "config.json"), "awq") == (str(tmp_path), "huggingface-safetensor")
    assert detect_weight("auto", str(tmp_path / "config.json"), "auto") == (str(tmp_path), "huggingface-safetensor")


def test_text_streamer_and_stop_strings_on_random_unicode():
    """Random strings of one- to four-byte characters, fed to the streamer in random bursts: the pieces join to
    the plain decoding and no piece before the end holds a replacement character. A stop string cut at a random
    place of the text stops the handler there, however the text is split into tokens."""
    rng = np.random.default_rng(0)
    tok = Tokenizer.synthetic(1000)
    alphabet = list("abc xyz.,") + list("éüñß") + list("✓€漢字") + list("😀🚀")
    for _ in range(60):
        text = "".join(alphabet[int(i)] for i in rng.integers(0, len(alphabet), int(rng.integers(1, 40))))
        ids = tok.encode(text)
        st = TextStreamer(tok)
        pieces, at = [], 0
        while at < len(ids):
            n = int(rng.integers(1, 5))
            pieces.append(st.put(ids[at:at + n]))
            at += n
        assert all("�" not in p for p in pieces)
        pieces.append(st.finish())
        assert "".join(pieces) == tok.decode(ids) == text
        if len(text) < 4:
            continue
        a = int(rng.integers(1, len(text) - 1))
        b = int(rng.integers(a + 1, min(len(text), a + 6) + 1))
        stop = text[a:b]
        handler = StopStrHandler([stop], tok)
        out = []
        for i in ids:
            out.extend(handler.put(i))
            if handler.stop_triggered:
                break
        assert handler.stop_triggered, (text, stop)
        assert tok.decode(out) == text[: text.index(stop)], (text, stop)


def test_every_template_renders_alike_in_python_and_native_code():
    """All registered templates, random conversations (with and without a system message, one to four turns, a
    list-of-text-parts content now and then): the Python renderer and the C++ one of the JSON FFI engine give the
    same prompt."""
    rng = np.random.default_rng(3)
    words = ["Hi", "Tell me more.", "Why?", "ok", "Summarise: a b c", "1 + 1 = ?", "Danke schön ✓", ""]
    checked = 0
    for name in ConvTemplateRegistry.names():
        conv = ConvTemplateRegistry.get_conv_template(name)
        for _ in range(4):
            msgs = []
            if rng.random() < 0.5:
                msgs.append({"role": "system", "content": "You are terse."})
            turns = int(rng.integers(1, 5))
            for t in range(turns):
                text = words[int(rng.integers(0, len(words)))]
                content = [{"type": "text", "text": text}] if rng.random() < 0.2 else text
                msgs.append({"role": "user", "content": content})
                if t + 1 < turns:
                    msgs.append({"role": "assistant", "content": words[int(rng.integers(0, len(words) - 1))]})
            c = Conversation.from_json_dict(conv.to_json_dict())
            c.messages = []
            for m in msgs:
                if m["role"] == "system":
                    c.system_message = m["content"]
                else:
                    c.messages.append((m["role"], m["content"]))
            c.messages.append(("assistant", None))
            try:
                py = "".join(p for p in c.as_prompt() if isinstance(p, str))
            except ValueError:
                continue                      # a template without that role
            native = _core.conv_template_render(json.dumps(conv.to_json_dict()), json.dumps(msgs))
            assert py == native, (name, msgs)
            checked += 1
    assert checked >= 150
