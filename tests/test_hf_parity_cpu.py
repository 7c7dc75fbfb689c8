"""Model math against HuggingFace transformers: tiny random checkpoints of several architectures are
saved, read through the HuggingFace loader and run through the CPU reference ops; logits of a
prefill and of a following decode step must match ``transformers``."""
import numpy as np
import pytest
import torch

from mlc_llm_b200 import _core
from mlc_llm_b200 import quantization as Q
from mlc_llm_b200.models import config as mc
from mlc_llm_b200.models import loader
from mlc_llm_b200.models.transformer import BatchInfo, DecoderModel

transformers = pytest.importorskip("transformers")

BASE = dict(hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, vocab_size=160, max_position_embeddings=128)

CASES = {
    "llama": ("LlamaConfig", dict(BASE, rms_norm_eps=1e-5, rope_theta=10000.0)),
    "mistral": ("MistralConfig", dict(BASE, sliding_window=None)),
    "qwen2": ("Qwen2Config", dict(BASE)),
    "qwen3": ("Qwen3Config", dict(BASE, head_dim=32)),
    "gemma": ("GemmaConfig", dict(BASE, head_dim=16, hidden_activation="gelu_pytorch_tanh")),
    "gemma2": ("Gemma2Config", dict(BASE, head_dim=16, query_pre_attn_scalar=16, sliding_window=4096)),
    "phi3": ("Phi3Config", dict(BASE, pad_token_id=0)),
    "gpt2": ("GPT2Config", dict(n_embd=64, n_layer=2, n_head=4, vocab_size=160, n_positions=128)),
    "gpt_neox": ("GPTNeoXConfig", dict(hidden_size=64, intermediate_size=256, num_hidden_layers=2,
                                       num_attention_heads=4, vocab_size=160, max_position_embeddings=128,
                                       rotary_pct=0.25)),
    "gptj": ("GPTJConfig", dict(n_embd=64, n_layer=2, n_head=4, vocab_size=160, n_positions=128, rotary_dim=8)),
    "nemotron": ("NemotronConfig", dict(BASE, head_dim=16)),
    "olmo": ("OlmoConfig", dict(BASE)),
    "gpt_bigcode": ("GPTBigCodeConfig", dict(n_embd=64, n_layer=2, n_head=4, vocab_size=160, n_positions=128,
                                             multi_query=True)),
    "gemma3_text": ("Gemma3TextConfig", dict(BASE, head_dim=16, query_pre_attn_scalar=16, sliding_window=4096)),
    "deepseek_v2": ("DeepseekV2Config", dict(
        hidden_size=64, intermediate_size=112, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
        vocab_size=160, max_position_embeddings=128, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16,
        qk_rope_head_dim=16, v_head_dim=16, head_dim=16, n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=3,
        moe_intermediate_size=24, first_k_dense_replace=1, topk_method="greedy", n_group=4,
        topk_group=2, routed_scaling_factor=1.5, norm_topk_prob=False)),
    "glm": ("GlmConfig", dict(BASE, head_dim=16, partial_rotary_factor=0.5, attention_bias=True, pad_token_id=0)),
    "llama4_text": ("Llama4TextConfig", dict(
        hidden_size=64, intermediate_size=48, intermediate_size_mlp=112, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, vocab_size=160, max_position_embeddings=128, num_local_experts=4,
        num_experts_per_tok=1, interleave_moe_layer_step=2, use_qk_norm=True, attn_temperature_tuning=True,
        floor_scale=8, attn_scale=0.1, attention_chunk_size=8, rope_theta=10000.0, pad_token_id=0)),
    "mixtral": ("MixtralConfig", dict(BASE, num_local_experts=4, num_experts_per_tok=2)),
    "qwen2_moe": ("Qwen2MoeConfig", dict(BASE, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
                                         shared_expert_intermediate_size=80, decoder_sparse_step=1,
                                         mlp_only_layers=[])),
    "qwen3_moe": ("Qwen3MoeConfig", dict(BASE, head_dim=32, num_experts=4, num_experts_per_tok=2,
                                         moe_intermediate_size=48, decoder_sparse_step=1, mlp_only_layers=[],
                                         norm_topk_prob=True)),
    "starcoder2": ("Starcoder2Config", dict(BASE, use_bias=True)),
    "stablelm": ("StableLmConfig", dict(BASE)),
    "olmo2": ("Olmo2Config", dict(BASE)),
    "cohere": ("CohereConfig", dict(BASE)),
    "phi": ("PhiConfig", dict(BASE, num_key_value_heads=4)),
    # stretched-context rotary variants: YaRN (band-wise slow-down + cos/sin scale), LongRoPE (per-band
    # divisors, long set because the served window exceeds the trained one), YaRN with DeepSeek's softmax scale
    "llama_yarn": ("LlamaConfig", dict(BASE, rope_parameters={
        "rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 16, "rope_theta": 10000.0,
        "beta_fast": 32.0, "beta_slow": 1.0})),
    "phi3_longrope": ("Phi3Config", dict(BASE, pad_token_id=0, original_max_position_embeddings=16, rope_parameters={
        "rope_type": "longrope", "rope_theta": 10000.0, "short_factor": [1.0 + 0.05 * i for i in range(8)],
        "long_factor": [1.5 + 0.25 * i for i in range(8)]})),
    "ministral3": ("Ministral3Config", dict(BASE, head_dim=16, sliding_window=None, rope_parameters={
        "rope_type": "yarn", "factor": 16.0, "original_max_position_embeddings": 8, "rope_theta": 10000.0,
        "beta_fast": 32.0, "beta_slow": 1.0, "mscale": 1.0, "mscale_all_dim": 1.0, "llama_4_scaling_beta": 0.1})),
    "deepseek_v2_yarn": ("DeepseekV2Config", dict(
        hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
        vocab_size=160, max_position_embeddings=128, q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16,
        qk_rope_head_dim=16, v_head_dim=16, head_dim=16, n_routed_experts=4, n_shared_experts=1, num_experts_per_tok=2,
        moe_intermediate_size=24, first_k_dense_replace=1, topk_method="greedy", n_group=1, topk_group=1,
        routed_scaling_factor=1.0, norm_topk_prob=False, rope_parameters={
            "rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 16, "rope_theta": 10000.0,
            "beta_fast": 32.0, "beta_slow": 1.0, "mscale": 0.707, "mscale_all_dim": 0.707})),
}


def _batch(plan):
    t = lambda k: torch.from_numpy(np.asarray(plan[k])).to(torch.int32)
    return BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                     page_indptr=t("page_indptr"), page_indices=t("page_indices"),
                     num_tokens=len(plan["positions"]))


@pytest.mark.parametrize("name", sorted(CASES))
def test_logits_match_transformers(name, tmp_path):
    cls_name, kwargs = CASES[name]
    if not hasattr(transformers, cls_name):
        pytest.skip(f"transformers has no {cls_name}")
    torch.manual_seed(0)
    hf_cfg = getattr(transformers, cls_name)(**kwargs)
    hf = transformers.AutoModelForCausalLM.from_config(hf_cfg, attn_implementation="eager").float().eval()
    with torch.no_grad():  # default inits leave norms at 1 and biases at 0; perturb them so they matter
        for pname, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)
    hf.save_pretrained(tmp_path, safe_serialization=True)
    import json
    raw = json.load(open(tmp_path / "config.json"))
    cfg = mc.from_dict(raw["model_type"], raw)
    quant = Q.get("q0f32")
    store = loader.load_hf_params(str(tmp_path), cfg, quant, torch.device("cpu"))
    model = DecoderModel(cfg, quant, store, torch.device("cpu"))
    model.create_kv_cache(16, 16)
    kv = _core.KVManager(16, 16, 4)
    kv.add_sequence(0)
    toks = torch.randint(0, 160, (21,))
    with torch.no_grad():
        want = hf(toks[None]).logits[0].float()
    plan = kv.begin_forward([0], [20])
    h = model.forward(model.embed(toks[:20].to(torch.int32)), _batch(plan))
    got = model.logits(h, torch.arange(20, dtype=torch.int32)).float()
    assert (got - want[:20]).abs().max() < 2e-3, (got - want[:20]).abs().max()
    plan = kv.begin_forward([0], [1])
    h = model.forward(model.embed(toks[20:21].to(torch.int32)), _batch(plan))
    got1 = model.logits(h, None).float()
    assert (got1[0] - want[20]).abs().max() < 2e-3, (got1[0] - want[20]).abs().max()
