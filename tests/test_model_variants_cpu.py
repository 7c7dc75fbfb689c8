"""Architecture switches that have no HuggingFace counterpart installed: checked through algebraic
identities against the plain Llama forward."""
import math

import numpy as np
import pytest
import torch

from mlc_llm_b200 import _core
from mlc_llm_b200 import quantization as Q
from mlc_llm_b200.models import config as mc
from mlc_llm_b200.models import loader
from mlc_llm_b200.models.transformer import BatchInfo, DecoderModel

BASE = dict(hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, vocab_size=160, max_position_embeddings=128, rms_norm_eps=1e-5)


def _logits(model, toks):
    model.create_kv_cache(8, 16)
    kv = _core.KVManager(8, 16, 2)
    kv.add_sequence(0)
    plan = kv.begin_forward([0], [len(toks)])
    t = lambda k: torch.from_numpy(np.asarray(plan[k])).to(torch.int32)
    b = BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                  page_indptr=t("page_indptr"), page_indices=t("page_indices"), num_tokens=len(toks))
    h = model.forward(model.embed(torch.tensor(toks, dtype=torch.int32)), b)
    return model.logits(h, None).float()


def test_minicpm_scaling_equals_llama_with_rescaled_weights():
    """embedding x scale_emb, residual branches x scale_depth / sqrt(L), hidden / (hidden / dim_model_base)
    before the head: the same function as a Llama whose embedding, o_proj / down_proj and lm_head
    weights carry those factors."""
    quant = Q.get("q0f32")
    cpm = mc.from_dict("minicpm", dict(BASE, scale_emb=12, scale_depth=1.4, dim_model_base=16))
    assert cpm.embedding_scale == 12 and math.isclose(cpm.extra["residual_scale"], 1.4 / math.sqrt(2))
    assert math.isclose(cpm.extra["logit_scale"], 1 / 4)
    llama = mc.from_dict("llama", dict(BASE))
    store = loader.random_params(cpm, quant, 7, torch.device("cpu"), std=0.2)
    ref_store = loader.random_params(llama, quant, 7, torch.device("cpu"), std=0.2)
    rs = cpm.extra["residual_scale"]
    ref_store.tensors["model.embed_tokens.weight"] = ref_store.tensors["model.embed_tokens.weight"] * 12
    for i in range(2):
        for name in (f"model.layers.{i}.self_attn.o_proj", f"model.layers.{i}.mlp.down_proj"):
            ref_store.linears[name].w = ref_store.linears[name].w * rs
    ref_store.linears["lm_head"].w = ref_store.linears["lm_head"].w / 4
    toks = [3, 17, 42, 99, 5, 8]
    got = _logits(DecoderModel(cpm, quant, store, torch.device("cpu")), toks)
    want = _logits(DecoderModel(llama, quant, ref_store, torch.device("cpu")), toks)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), (got - want).abs().max()
    plain = _logits(DecoderModel(llama, quant, loader.random_params(llama, quant, 7, torch.device("cpu"), std=0.2),
                                 torch.device("cpu")), toks)
    assert not torch.allclose(got, plain, atol=1e-2)


def test_internlm_bias_and_orion_layernorm_switches():
    assert mc.from_dict("internlm", dict(BASE, bias=True)).attention_bias
    assert not mc.from_dict("internlm", dict(BASE, bias=False)).attention_bias
    assert mc.from_dict("orion", dict(BASE)).norm_type == "layernorm"


def test_chatglm3_checkpoint_layout_equals_glm(tmp_path):
    """A ChatGLM3-format checkpoint (fused ``query_key_value`` / ``dense_h_to_4h``, its own config keys)
    built from the tensors of a HuggingFace ``glm`` model must give the same logits as that model."""
    import json

    import pytest
    from safetensors.torch import save_file

    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "GlmConfig"):
        pytest.skip("transformers has no GLM")
    torch.manual_seed(0)
    hf_cfg = transformers.GlmConfig(hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, vocab_size=160, head_dim=16,
                                    max_position_embeddings=128, partial_rotary_factor=0.5, attention_bias=True,
                                    pad_token_id=0)
    hf = transformers.AutoModelForCausalLM.from_config(hf_cfg).float().eval()
    (tmp_path / "glm").mkdir()
    hf.save_pretrained(tmp_path / "glm", safe_serialization=True)
    sd = hf.state_dict()
    out = {"transformer.embedding.word_embeddings.weight": sd["model.embed_tokens.weight"],
           "transformer.encoder.final_layernorm.weight": sd["model.norm.weight"],
           "transformer.output_layer.weight": sd["lm_head.weight"]}
    for i in range(2):
        s, d = f"model.layers.{i}.", f"transformer.encoder.layers.{i}."
        out[d + "input_layernorm.weight"] = sd[s + "input_layernorm.weight"]
        out[d + "post_attention_layernorm.weight"] = sd[s + "post_attention_layernorm.weight"]
        for suffix in ("weight", "bias"):
            out[d + f"self_attention.query_key_value.{suffix}"] = torch.cat(
                [sd[s + f"self_attn.{n}_proj.{suffix}"] for n in "qkv"])
        out[d + "self_attention.dense.weight"] = sd[s + "self_attn.o_proj.weight"]
        out[d + "mlp.dense_h_to_4h.weight"] = sd[s + "mlp.gate_up_proj.weight"]
        out[d + "mlp.dense_4h_to_h.weight"] = sd[s + "mlp.down_proj.weight"]
    (tmp_path / "chatglm").mkdir()
    save_file({k: v.contiguous().clone() for k, v in out.items()}, str(tmp_path / "chatglm" / "model.safetensors"))
    chat_cfg = dict(model_type="chatglm", hidden_size=64, num_layers=2, num_attention_heads=4,
                    multi_query_attention=True, multi_query_group_num=2, kv_channels=16, ffn_hidden_size=112,
                    layernorm_epsilon=hf_cfg.rms_norm_eps, padded_vocab_size=160, seq_length=128,
                    add_qkv_bias=True, rope_ratio=1.0)
    quant = Q.get("q0f32")
    toks = [3, 17, 42, 99, 5, 8, 120]
    glm_cfg = mc.from_dict("glm", json.load(open(tmp_path / "glm" / "config.json")))
    want = _logits(DecoderModel(glm_cfg, quant, loader.load_hf_params(str(tmp_path / "glm"), glm_cfg, quant,
                                                                      torch.device("cpu")), torch.device("cpu")), toks)
    cfg = mc.from_dict("chatglm", chat_cfg)
    assert cfg.num_key_value_heads == 2 and cfg.head_dim == 16 and cfg.rotary_dim == 8 and cfg.attention_bias
    got = _logits(DecoderModel(cfg, quant, loader.load_hf_params(str(tmp_path / "chatglm"), cfg, quant,
                                                                 torch.device("cpu")), torch.device("cpu")), toks)
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()


def test_qwen1_checkpoint_layout_equals_qwen2(tmp_path):
    """First-generation Qwen checkpoint names (``c_attn``, ``w1`` / ``w2``, doubled ``intermediate_size``)
    built from a HuggingFace Qwen2 model (same math: q/k/v bias, SwiGLU) give the same logits."""
    import json

    import pytest
    from safetensors.torch import save_file

    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    hf_cfg = transformers.Qwen2Config(hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=4, vocab_size=160,
                                      max_position_embeddings=128, tie_word_embeddings=False)
    hf = transformers.AutoModelForCausalLM.from_config(hf_cfg).float().eval()
    (tmp_path / "q2").mkdir()
    hf.save_pretrained(tmp_path / "q2", safe_serialization=True)
    sd = hf.state_dict()
    out = {"transformer.wte.weight": sd["model.embed_tokens.weight"], "transformer.ln_f.weight": sd["model.norm.weight"],
           "lm_head.weight": sd["lm_head.weight"]}
    for i in range(2):
        s, d = f"model.layers.{i}.", f"transformer.h.{i}."
        out[d + "ln_1.weight"] = sd[s + "input_layernorm.weight"]
        out[d + "ln_2.weight"] = sd[s + "post_attention_layernorm.weight"]
        for suffix in ("weight", "bias"):
            out[d + f"attn.c_attn.{suffix}"] = torch.cat([sd[s + f"self_attn.{n}_proj.{suffix}"] for n in "qkv"])
        out[d + "attn.c_proj.weight"] = sd[s + "self_attn.o_proj.weight"]
        out[d + "mlp.w1.weight"] = sd[s + "mlp.up_proj.weight"]
        out[d + "mlp.w2.weight"] = sd[s + "mlp.gate_proj.weight"]
        out[d + "mlp.c_proj.weight"] = sd[s + "mlp.down_proj.weight"]
    (tmp_path / "q1").mkdir()
    save_file({k: v.contiguous().clone() for k, v in out.items()}, str(tmp_path / "q1" / "model.safetensors"))
    q1_cfg = dict(model_type="qwen", hidden_size=64, num_hidden_layers=2, num_attention_heads=4, kv_channels=16,
                  intermediate_size=224, layer_norm_epsilon=hf_cfg.rms_norm_eps, vocab_size=160, seq_length=128,
                  rotary_emb_base=json.load(open(tmp_path / "q2" / "config.json")).get("rope_theta", 10000.0))
    quant = Q.get("q0f32")
    toks = [3, 17, 42, 99, 5, 8, 120]
    c2 = mc.from_dict("qwen2", json.load(open(tmp_path / "q2" / "config.json")))
    c1 = mc.from_dict("qwen", q1_cfg)
    c1.rope_theta = c2.rope_theta
    assert c1.intermediate_size == 112 and c1.attention_bias
    want = _logits(DecoderModel(c2, quant, loader.load_hf_params(str(tmp_path / "q2"), c2, quant, torch.device("cpu")),
                                torch.device("cpu")), toks)
    got = _logits(DecoderModel(c1, quant, loader.load_hf_params(str(tmp_path / "q1"), c1, quant, torch.device("cpu")),
                               torch.device("cpu")), toks)
    assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()


@pytest.mark.parametrize("preset", ["tiny-deepseek-v2", "tiny-llava", "tiny-phi3v", "tiny-qwen35", "tiny-rwkv6",
                                    "tiny-eagle", "tiny-medusa"])
def test_gen_config_keeps_what_the_family_parser_needs(preset, tmp_path):
    """The model section written by gen_config parses back to the same configuration, family-specific
    settings (latent-attention ranks, vision section, recurrent geometry, draft-head sizes) included."""
    import json
    import os

    from mlc_llm_b200.interface.gen_config import gen_config
    from mlc_llm_b200.models import config as C
    from mlc_llm_b200.models.presets import MODEL_PRESETS

    src = tmp_path / "src"
    src.mkdir()
    json.dump(MODEL_PRESETS[preset], open(src / "config.json", "w"))
    out = str(tmp_path / "out")
    gen_config(str(src), "auto", "q0f16", "LM", None, None, None, None, None, None, None, 64, out)
    chat = json.load(open(os.path.join(out, "mlc-chat-config.json")))
    again = C.from_dict(chat["model_type"], chat["model_config"])
    first = C.from_dict(MODEL_PRESETS[preset]["model_type"], dict(MODEL_PRESETS[preset], max_batch_size=64))
    assert again.extra == first.extra
    a, b = again.asdict(), first.asdict()
    assert a == b, {k: (a[k], b[k]) for k in a if a[k] != b[k]}


def test_public_presets_parse_to_their_published_sizes():
    """Every named preset of a published checkpoint parses; parameter counts of a few well-known ones."""
    import math as _math

    from mlc_llm_b200.models.presets import MODEL_PRESETS
    from mlc_llm_b200.models.transformer import param_specs

    def billions(name):
        d = MODEL_PRESETS[name]
        cfg = mc.from_dict(d["model_type"], d)
        return sum(_math.prod(shape) for shape, _ in param_specs(cfg).values()) / 1e9

    assert abs(billions("llama2_7b") - 6.74) < 0.01
    assert abs(billions("llama3_1_8b") - 8.03) < 0.01
    assert abs(billions("mistral_7b") - 7.24) < 0.01
    assert abs(billions("Mixtral-8x7B-v0.1") - 46.7) < 0.05
    assert abs(billions("qwen2_7b") - 7.62) < 0.01
    assert abs(billions("deepseek_v2_lite") - 15.7) < 0.2
    assert 3.0 < billions("ministral3_3b_2512") < 4.0
    for name, d in MODEL_PRESETS.items():
        if d.get("model_type") == "bert":
            continue  # the embedding encoder has its own configuration class
        cfg = mc.from_dict(d["model_type"], d)
        assert cfg.hidden_size > 0 and cfg.num_hidden_layers >= 0, name
