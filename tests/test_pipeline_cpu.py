"""Offline pipeline on CPU: HuggingFace checkpoint -> gen_config -> convert_weight -> engine, checked
against ``transformers`` greedy generation; plus compile metadata, chat REPL and the direct
(unconverted) HuggingFace path."""
import json
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")
tokenizers = pytest.importorskip("tokenizers")

from mlc_llm_b200.cli import compile as cli_compile  # noqa: E402
from mlc_llm_b200.cli import convert_weight as cli_convert  # noqa: E402
from mlc_llm_b200.cli import gen_config as cli_gen  # noqa: E402
from mlc_llm_b200.interface.chat import ChatState  # noqa: E402
from mlc_llm_b200.loader.tensor_cache import TensorCache  # noqa: E402
from mlc_llm_b200.serve.config import EngineConfig  # noqa: E402
from mlc_llm_b200.serve.engine import MLCEngine  # noqa: E402

CORPUS = ["the quick brown fox jumps over the lazy dog", "hello world, this is a tiny tokenizer",
          "serving large language models on fast hardware", "what is the capital of France?",
          "numbers 0 1 2 3 4 5 6 7 8 9 and symbols !?.,;:"] * 4


@pytest.fixture(scope="module")
def hf_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("hf")
    tok = tokenizers.Tokenizer(tokenizers.models.BPE(unk_token=None))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    trainer = tokenizers.trainers.BpeTrainer(vocab_size=300, special_tokens=["<s>", "</s>", "<unk>"],
                                             initial_alphabet=tokenizers.pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(CORPUS, trainer)
    tok.save(str(d / "tokenizer.json"))
    vocab = tok.get_vocab_size()
    torch.manual_seed(1)
    cfg = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, vocab_size=vocab,
                                   max_position_embeddings=256, bos_token_id=0, eos_token_id=1)
    model = transformers.LlamaForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for p in model.parameters():  # larger weights -> confident argmax, stable under quantisation checks
            p.mul_(8.0) if p.dim() > 1 else None
    model.save_pretrained(d, safe_serialization=True)
    return str(d), model, tok


def test_gen_config_convert_and_generate(hf_dir, tmp_path):
    src, hf_model, tok = hf_dir
    out = str(tmp_path / "mlc")
    cli_gen.main([src, "--quantization", "q0f32", "--conv-template", "LM", "--output", out])
    chat = json.load(open(os.path.join(out, "mlc-chat-config.json")))
    assert chat["model_type"] == "llama" and chat["quantization"] == "q0f32"
    assert "tokenizer.json" in chat["tokenizer_files"] and os.path.exists(os.path.join(out, "tokenizer.json"))
    assert chat["conv_template"]["name"] == "LM" and chat["vocab_size"] == tok.get_vocab_size()
    from mlc_llm_b200.interface.convert_weight import convert_weight
    convert_weight(src, "q0f32", output=out, verbose=False, encode_format="raw")
    cache = TensorCache(out, verify_md5=True)
    assert "model.layers.0.self_attn.qkv_proj.weight" in cache.names()
    assert cache.metadata["ParamSize"] == len(cache.names())
    engine = MLCEngine(out, "cpu", engine_config=EngineConfig(mode="local"))
    try:
        prompt = tok.encode("the quick brown fox").ids
        want = hf_model.generate(torch.tensor([prompt]), max_new_tokens=8, do_sample=False,
                                 eos_token_id=None, pad_token_id=0)[0, len(prompt):].tolist()
        resp = engine.completions.create(prompt=prompt, max_tokens=8, temperature=0.0,
                                         debug_config={"ignore_eos": True})
        assert resp.choices[0].text == tok.decode(want)
        # text prompt goes through the real tokenizer and gives the same continuation
        resp2 = engine.completions.create(prompt="the quick brown fox", max_tokens=8, temperature=0.0,
                                          debug_config={"ignore_eos": True})
        prefix = list(engine.conv_template.system_prefix_token_ids or [])
        want2 = hf_model.generate(torch.tensor([prefix + prompt]), max_new_tokens=8, do_sample=False,
                                  eos_token_id=None, pad_token_id=0)[0, len(prefix) + len(prompt):].tolist()
        assert resp2.choices[0].text == tok.decode(want2)
        assert resp2.usage.prompt_tokens == len(prefix) + len(prompt)
        # chat REPL over the same engine
        lines = []
        state = ChatState(engine, write=lines.append)
        assert state.handle("/set temperature=0;max_tokens=4")
        assert state.handle("hello world")
        assert len(state.history) == 2 and state.history[1]["role"] == "assistant"
        assert state.handle("/stats") and "completion_tokens: 4" in "".join(lines)
        assert state.handle("/reset") and not state.history
        assert not state.handle("/exit")
    finally:
        engine.terminate()


def test_quantized_convert_and_compile_metadata(hf_dir, tmp_path):
    src, _, _ = hf_dir
    out = str(tmp_path / "mlc-q4")
    cli_gen.main([src, "--quantization", "q4f16_1", "--conv-template", "LM", "--output", out,
                  "--context-window-size", "128"])
    cli_convert.main([src, "--quantization", "q4f16_1", "--output", out, "--device", "cpu"])
    cache = TensorCache(out)
    names = cache.names()
    assert "model.layers.1.mlp.gate_up_proj.q_weight" in names and "model.layers.1.mlp.gate_up_proj.q_scale" in names
    qw = cache.get("model.layers.1.mlp.gate_up_proj.q_weight")
    assert qw.shape == (256, 64 // 8)
    assert 4.0 < cache.metadata["BitsPerParam"] < 6.5
    lib = str(tmp_path / "lib.json")
    cli_compile.main([out, "--output", lib])
    meta = json.load(open(lib))
    assert meta["quantization"] == "q4f16_1" and meta["context_window_size"] == 128
    assert meta["kv_cache"]["num_key_value_heads"] == 2
    engine = MLCEngine(out, "cpu", model_lib=lib, engine_config=EngineConfig(mode="local"))
    try:
        r = engine.chat.completions.create(messages=[{"role": "user", "content": "hello"}], max_tokens=5)
        assert r.usage.completion_tokens <= 5 and r.choices[0].message.role == "assistant"
    finally:
        engine.terminate()


def test_serve_unconverted_hf_directory(hf_dir):
    src, hf_model, tok = hf_dir
    os.environ["MLC_JIT_QUANTIZATION"] = "q0f32"
    try:
        engine = MLCEngine(src, "cpu", engine_config=EngineConfig(mode="local"))
    finally:
        del os.environ["MLC_JIT_QUANTIZATION"]
    try:
        prompt = tok.encode("hello world").ids
        want = hf_model.generate(torch.tensor([prompt]), max_new_tokens=6, do_sample=False,
                                 eos_token_id=None, pad_token_id=0)[0, len(prompt):].tolist()
        resp = engine.completions.create(prompt=prompt, max_tokens=6, temperature=0.0,
                                         debug_config={"ignore_eos": True})
        assert resp.choices[0].text == tok.decode(want)
    finally:
        engine.terminate()


def test_convert_weight_merges_a_lora_adapter(hf_dir, tmp_path):
    """``--lora-adapter``: the PEFT-format low-rank updates are merged (W += alpha / r * B @ A) into the
    tensors they target before q / k / v fusing; everything else is untouched."""
    from safetensors.torch import save_file

    src, hf_model, _ = hf_dir
    adapter = tmp_path / "adapter"
    adapter.mkdir()
    g = torch.Generator().manual_seed(3)
    r, alpha = 4, 8.0
    a_q, b_q = torch.randn(r, 64, generator=g) * 0.1, torch.randn(64, r, generator=g) * 0.1
    a_d, b_d = torch.randn(r, 128, generator=g) * 0.1, torch.randn(64, r, generator=g) * 0.1
    save_file({"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": a_q,
               "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": b_q,
               "base_model.model.model.layers.1.mlp.down_proj.lora_A.weight": a_d,
               "base_model.model.model.layers.1.mlp.down_proj.lora_B.weight": b_d},
              str(adapter / "adapter_model.safetensors"))
    (adapter / "adapter_config.json").write_text(json.dumps(
        {"peft_type": "LORA", "r": r, "lora_alpha": alpha, "target_modules": ["q_proj", "down_proj"]}))
    out = str(tmp_path / "merged")
    cli_convert.main([src, "--quantization", "q0f32", "--output", out, "--lora-adapter", str(adapter)])
    cache = TensorCache(out)
    sd = hf_model.state_dict()
    scale = alpha / r
    qkv = cache.get("model.layers.0.self_attn.qkv_proj.weight").float()
    want_q = sd["model.layers.0.self_attn.q_proj.weight"] + scale * (b_q @ a_q)
    assert torch.allclose(qkv[:64], want_q, atol=2e-2, rtol=1e-2)        # bf16 storage
    assert torch.allclose(qkv[64:96], sd["model.layers.0.self_attn.k_proj.weight"], atol=2e-2, rtol=1e-2)
    assert not torch.allclose(qkv[:64], sd["model.layers.0.self_attn.q_proj.weight"], atol=2e-2, rtol=1e-2)
    down = cache.get("model.layers.1.mlp.down_proj.weight").float()
    assert torch.allclose(down, sd["model.layers.1.mlp.down_proj.weight"] + scale * (b_d @ a_d), atol=2e-2,
                          rtol=1e-2)
    down0 = cache.get("model.layers.0.mlp.down_proj.weight").float()
    assert torch.allclose(down0, sd["model.layers.0.mlp.down_proj.weight"], atol=2e-2, rtol=1e-2)


def test_delivery_runs_only_what_the_log_lacks(hf_dir, tmp_path):
    """Continuous delivery: every (model, quantisation) pair of the spec that the log does not list is
    converted; a second run has nothing left to do; a changed conversation template only redoes the config."""
    from mlc_llm_b200.cli import delivery

    src, _, _ = hf_dir
    spec = {"tasks": [{"model_id": "tiny", "model": src, "conv_template": "LM", "quantization": ["q0f32"],
                       "overrides": {"q4f16_1": {"context_window_size": 128}}}],
            "default_quantization": ["q4f16_1"]}
    spec_path, log_path, out = tmp_path / "spec.json", tmp_path / "log.json", tmp_path / "out"
    spec_path.write_text(json.dumps(spec))
    delivery.main(["--spec", str(spec_path), "--log", str(log_path), "--output", str(out)])
    dirs = sorted(os.listdir(out))
    assert dirs == ["tiny-q0f32-MLC", "tiny-q4f16_1-MLC"]
    chat = json.load(open(out / "tiny-q4f16_1-MLC" / "mlc-chat-config.json"))
    assert chat["context_window_size"] == 128 and chat["quantization"] == "q4f16_1"
    assert "model.layers.0.self_attn.qkv_proj.q_weight" in TensorCache(str(out / "tiny-q4f16_1-MLC")).names()
    log = json.load(open(log_path))
    assert sorted(t["quantization"] for t in log["tasks"]) == ["q0f32", "q4f16_1"]
    diff = delivery.generate_model_delivery_diff(delivery.ModelDeliveryList.from_json(spec),
                                                 delivery.get_current_log(str(log_path)))
    assert diff.tasks == []
    spec["tasks"][0]["conv_template"] = "chatml"
    diff = delivery.generate_model_delivery_diff(delivery.ModelDeliveryList.from_json(spec),
                                                 delivery.get_current_log(str(log_path)))
    assert len(diff.tasks) == 2 and all(t.gen_config_only for t in diff.tasks)


def test_presharded_convert_gives_each_rank_its_slices(hf_dir, tmp_path):
    """``--preshard 2``: records ``<name>_shard-<rank>``; a rank loading them gets exactly what it would cut
    out of the unsharded artifact."""
    import torch as _torch

    from mlc_llm_b200 import quantization as Q
    from mlc_llm_b200.models import config as mcfg
    from mlc_llm_b200.models import loader

    src, _, _ = hf_dir
    plain, pre = str(tmp_path / "plain"), str(tmp_path / "pre")
    for out in (plain, pre):
        cli_gen.main([src, "--quantization", "q4f16_1", "--conv-template", "LM", "--output", out])
    cli_convert.main([src, "--quantization", "q4f16_1", "--output", plain, "--device", "cpu"])
    cli_convert.main([src, "--quantization", "q4f16_1", "--output", pre, "--device", "cpu", "--preshard", "2"])
    names = TensorCache(pre).names()
    assert "model.layers.0.self_attn.qkv_proj.q_weight_shard-1" in names
    assert "model.layers.0.input_layernorm.weight" in names        # replicated: written once
    chat = json.load(open(os.path.join(pre, "mlc-chat-config.json")))
    cfg = mcfg.from_dict(chat["model_type"], chat["model_config"])
    quant = Q.get("q4f16_1")
    for rank in (0, 1):
        a = loader.load_params(plain, cfg, quant, _torch.device("cpu"), 2, rank)
        b = loader.load_params(pre, cfg, quant, _torch.device("cpu"), 2, rank)
        assert set(a.linears) == set(b.linears) and set(a.tensors) == set(b.tensors)
        for k in a.linears:
            assert _torch.equal(a.linears[k].w, b.linears[k].w), k
            assert _torch.equal(a.linears[k].scale, b.linears[k].scale), k
        for k in a.tensors:
            assert _torch.equal(a.tensors[k], b.tensors[k]), k
