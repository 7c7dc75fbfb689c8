"""Qwen3.5 hybrid (gated delta-rule layers + gated softmax attention) against HuggingFace transformers,
and its recurrent state across chunked prefill, batched decode and the serving engine."""
import json

import numpy as np
import pytest
import torch

from mlc_llm_b200 import _core
from mlc_llm_b200 import quantization as Q
from mlc_llm_b200.models import config as mc
from mlc_llm_b200.models import loader
from mlc_llm_b200.models.qwen35 import Qwen35Model, gated_delta_step
from mlc_llm_b200.models.transformer import BatchInfo

transformers = pytest.importorskip("transformers")

HF_CFG = dict(hidden_size=64, intermediate_size=112, num_hidden_layers=4, num_attention_heads=4,
              num_key_value_heads=2, head_dim=32, vocab_size=160, max_position_embeddings=128,
              linear_key_head_dim=16, linear_value_head_dim=24, linear_num_key_heads=2, linear_num_value_heads=4,
              linear_conv_kernel_dim=4, full_attention_interval=4, rms_norm_eps=1e-6, pad_token_id=0,
              layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"])


def _batch(plan, seq_ids, starts):
    t = lambda k: torch.from_numpy(np.asarray(plan[k])).to(torch.int32)
    b = BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                  page_indptr=t("page_indptr"), page_indices=t("page_indices"), num_tokens=len(plan["positions"]))
    b.seq_ids = np.asarray(seq_ids)
    b.q_indptr = np.asarray(plan["q_indptr"])
    b.start_positions = np.asarray(starts)
    return b


def _build(tmp_path):
    if not hasattr(transformers, "Qwen3_5TextConfig"):
        pytest.skip("transformers has no Qwen3.5")
    torch.manual_seed(0)
    hf_cfg = transformers.Qwen3_5TextConfig(**HF_CFG)
    hf = transformers.Qwen3_5ForCausalLM(hf_cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)
    hf.save_pretrained(tmp_path, safe_serialization=True)
    raw = json.load(open(tmp_path / "config.json"))
    cfg = mc.from_dict(raw["model_type"], raw)
    assert cfg.layer_attn_kinds == ["linear", "linear", "linear", "mha"] and cfg.rotary_dim == 8
    quant = Q.get("q0f32")
    store = loader.load_hf_params(str(tmp_path), cfg, quant, torch.device("cpu"))
    model = Qwen35Model(cfg, quant, store, torch.device("cpu"))
    model.create_kv_cache(32, 16)
    assert model.kv_pages.shape[0] == 1  # only the attention layer owns pages
    return hf, model


def test_qwen35_logits_match_transformers(tmp_path):
    hf, model = _build(tmp_path)
    kv = _core.KVManager(32, 16, 4)
    kv.add_sequence(0)
    toks = torch.randint(0, 160, (23,))
    with torch.no_grad():
        want = hf(toks[None]).logits[0].float()
    # prefill in two chunks (the convolution window and the recurrent state carry over), then two decode steps
    done = 0
    got = []
    for n in (13, 8, 1, 1):
        plan = kv.begin_forward([0], [n])
        h = model.forward(model.embed(toks[done:done + n].to(torch.int32)), _batch(plan, [0], [done]))
        got.append(model.logits(h, torch.arange(n, dtype=torch.int32)).float())
        done += n
    got = torch.cat(got)
    assert (got - want).abs().max() < 2e-3, (got - want).abs().max()


def test_qwen35_batched_decode_equals_separate_sequences(tmp_path):
    _, model = _build(tmp_path)
    kv = _core.KVManager(32, 16, 4)
    toks = [torch.randint(0, 160, (9,)), torch.randint(0, 160, (6,))]
    for s in (0, 1):
        kv.add_sequence(s)
    # both prompts in one ragged prefill, then one batched decode step
    plan = kv.begin_forward([0, 1], [8, 5])
    x = torch.cat([toks[0][:8], toks[1][:5]]).to(torch.int32)
    model.forward(model.embed(x), _batch(plan, [0, 1], [0, 0]))
    plan = kv.begin_forward([0, 1], [1, 1])
    x = torch.stack([toks[0][8], toks[1][5]]).to(torch.int32)
    h = model.forward(model.embed(x), _batch(plan, [0, 1], [8, 5]))
    both = model.logits(h, None).float()
    # the same sequences one at a time, as fresh ids
    for j, s in enumerate((2, 3)):
        kv.add_sequence(s)
        n = len(toks[j]) - 1
        plan = kv.begin_forward([s], [n])
        model.forward(model.embed(toks[j][:n].to(torch.int32)), _batch(plan, [s], [0]))
        plan = kv.begin_forward([s], [1])
        h = model.forward(model.embed(toks[j][n:].to(torch.int32)), _batch(plan, [s], [n]))
        alone = model.logits(h, None).float()
        assert (alone[0] - both[j]).abs().max() < 1e-4


def test_gated_delta_step_is_the_delta_rule():
    """With no decay and full write strength the state stores v under a unit key exactly."""
    state = torch.zeros(1, 1, 4, 3)
    k = torch.tensor([[[1.0, 0, 0, 0]]])
    v = torch.tensor([[[1.0, 2.0, 3.0]]])
    zero, one = torch.zeros(1, 1), torch.ones(1, 1)
    out = gated_delta_step(state, k, k, v, zero, one)
    assert torch.allclose(out, v)
    # writing a new value under the same key replaces the old one; decay halves what is stored first
    v2 = torch.tensor([[[0.0, 1.0, 0.0]]])
    out = gated_delta_step(state, k, k, v2, torch.log(torch.tensor([[0.5]])), one)
    assert torch.allclose(out, v2)
    out = gated_delta_step(state, k, k, v2, zero, torch.tensor([[0.0]]))  # nothing written
    assert torch.allclose(out, v2)


def test_qwen35_through_the_engine():
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.engine import MLCEngine

    eng = MLCEngine("random://tiny-qwen35?quant=q0f32&seed=3", "cpu", mode="server",
                    engine_config=EngineConfig(max_num_sequence=4, max_total_sequence_length=1024,
                                               prefill_chunk_size=16))
    try:
        prompt = "the quick brown fox jumps over the lazy dog and keeps running through the field"
        a = eng.completions.create(prompt=prompt, max_tokens=6, temperature=0.0)
        # the same prompt next to another request (ragged prefill + batched decode) gives the same text
        import concurrent.futures as cf
        with cf.ThreadPoolExecutor(2) as pool:
            f1 = pool.submit(eng.completions.create, prompt=prompt, max_tokens=6, temperature=0.0)
            f2 = pool.submit(eng.completions.create, prompt="something else entirely", max_tokens=6, temperature=0.0)
            b, _ = f1.result(), f2.result()
        assert a.choices[0].text == b.choices[0].text
        assert a.usage.completion_tokens == 6
    finally:
        eng.terminate()


def test_qwen35_gen_config_convert_and_generate(tmp_path):
    """HuggingFace checkpoint -> mlc-chat-config + converted weights -> engine; greedy tokens equal
    ``transformers``' (both the raw artifact and the compile metadata name the hybrid state)."""
    import os

    import tokenizers

    from mlc_llm_b200.cli import compile as cli_compile
    from mlc_llm_b200.cli import gen_config as cli_gen
    from mlc_llm_b200.interface.convert_weight import convert_weight
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.engine import MLCEngine

    if not hasattr(transformers, "Qwen3_5TextConfig"):
        pytest.skip("transformers has no Qwen3.5")
    src = tmp_path / "hf"
    src.mkdir()
    tok = tokenizers.Tokenizer(tokenizers.models.BPE(unk_token=None))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    trainer = tokenizers.trainers.BpeTrainer(vocab_size=300, special_tokens=["<s>", "</s>"],
                                             initial_alphabet=tokenizers.pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog", "hello world of models"] * 4, trainer)
    tok.save(str(src / "tokenizer.json"))
    torch.manual_seed(1)
    hf_cfg = transformers.Qwen3_5TextConfig(**dict(HF_CFG, vocab_size=tok.get_vocab_size(), bos_token_id=0,
                                                   eos_token_id=1))
    hf = transformers.Qwen3_5ForCausalLM(hf_cfg).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.mul_(6.0) if p.dim() > 1 else None
    hf.save_pretrained(src, safe_serialization=True)
    out = str(tmp_path / "mlc")
    cli_gen.main([str(src), "--quantization", "q0f32", "--conv-template", "LM", "--output", out])
    chat = json.load(open(os.path.join(out, "mlc-chat-config.json")))
    assert chat["model_type"] in ("qwen3_5_text", "qwen3_5")
    convert_weight(str(src), "q0f32", output=out, verbose=False, encode_format="raw")
    lib = str(tmp_path / "lib.json")
    cli_compile.main([out, "--output", lib])
    assert json.load(open(lib))["kv_state_kind"] == "hybrid"
    eng = MLCEngine(out, "cpu", engine_config=EngineConfig(mode="local"))
    try:
        prompt = tok.encode("the quick brown fox").ids
        want = hf.generate(torch.tensor([prompt]), max_new_tokens=8, do_sample=False, eos_token_id=None,
                           pad_token_id=0)[0, len(prompt):].tolist()
        resp = eng.completions.create(prompt=prompt, max_tokens=8, temperature=0.0, debug_config={"ignore_eos": True})
        assert resp.choices[0].text == tok.decode(want), resp
    finally:
        eng.terminate()


def test_chunked_recurrence_equals_the_token_loop():
    from mlc_llm_b200.models.qwen35 import gated_delta_chunk

    g0 = torch.Generator().manual_seed(0)
    n, h, dk, dv = 150, 3, 8, 5  # two full chunks and a ragged one
    q = torch.nn.functional.normalize(torch.randn(n, h, dk, generator=g0), dim=-1) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(n, h, dk, generator=g0), dim=-1)
    v = torch.randn(n, h, dv, generator=g0)
    g = -torch.rand(n, h, generator=g0) * 0.3
    beta = torch.rand(n, h, generator=g0)
    s0 = torch.randn(h, dk, dv, generator=g0)
    loop_state = s0.clone().unsqueeze(0)
    want = torch.stack([gated_delta_step(loop_state, q[t:t + 1], k[t:t + 1], v[t:t + 1], g[t:t + 1], beta[t:t + 1])[0]
                        for t in range(n)])
    state = s0.clone()
    got = gated_delta_chunk(state, q, k, v, g, beta, chunk=64)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), (got - want).abs().max()
    assert torch.allclose(state, loop_state[0], atol=1e-4, rtol=1e-4)


def test_state_slots_grow_and_recycle(tmp_path, monkeypatch):
    from mlc_llm_b200.models import qwen35

    monkeypatch.setattr(qwen35, "FIRST_SLOTS", 2)
    monkeypatch.setattr(qwen35, "STATE_SLOTS", 4)
    _, model = _build(tmp_path)
    model._ensure_state()
    assert model.capacity == 2
    slots = [model._slot(s, 0) for s in range(4)]
    assert sorted(slots) == [0, 1, 2, 3] and model.capacity == 4
    # a fifth sequence takes the slot of the least recently used one; continuing that one is an error
    assert model._slot(4, 0) == slots[0]
    with pytest.raises(RuntimeError):
        model._slot(0, 7)
    assert model._slot(1, 5) == slots[1]  # a live sequence keeps its slot
