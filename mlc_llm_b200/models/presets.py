"""Named architecture presets (HuggingFace-style config dicts) used by ``gen_config`` and by the
random-weight benchmark / test models (reference: ``python/mlc_llm/model/model_preset.py``)."""

MODEL_PRESETS = {
    # 2-layer model for CPU plumbing tests
    "tiny-llama": {
        "model_type": "llama", "hidden_size": 256, "intermediate_size": 688, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 2048,
    },
    # speculative draft heads sized for tiny-llama: a one-block EAGLE head and three Medusa heads
    "tiny-eagle": {
        "model_type": "eagle", "hidden_size": 256, "intermediate_size": 688, "num_hidden_layers": 1,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 2048, "bias": True,
    },
    "tiny-medusa": {
        "model_type": "medusa", "hidden_size": 256, "vocab_size": 32000, "medusa_num_heads": 3,
        "medusa_num_layers": 1,
    },
    # tiny-llama with a 2-block CLIP tower: 28 x 28 images, four 14 x 14 patches
    "tiny-llava": {
        "model_type": "llava", "image_token_index": 31999, "vision_feature_layer": -2,
        "vision_feature_select_strategy": "default", "projector_hidden_act": "gelu",
        "text_config": {
            "model_type": "llama", "hidden_size": 256, "intermediate_size": 688, "num_hidden_layers": 2,
            "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 32000,
            "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 2048,
        },
        "vision_config": {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
                          "num_attention_heads": 4, "image_size": 28, "patch_size": 14,
                          "hidden_act": "quick_gelu", "layer_norm_eps": 1e-5},
    },
    # Qwen3.5-shaped hybrid: three gated delta-rule layers, then one gated softmax-attention layer
    "tiny-qwen35": {
        "model_type": "qwen3_5_text", "hidden_size": 256, "intermediate_size": 688, "num_hidden_layers": 4,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 32000,
        "rms_norm_eps": 1e-6, "rope_theta": 10000000.0, "partial_rotary_factor": 0.25,
        "max_position_embeddings": 4096, "linear_key_head_dim": 32, "linear_value_head_dim": 32,
        "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_conv_kernel_dim": 4,
        "full_attention_interval": 4,
    },
    # Phi-3-vision-shaped model: fused qkv / gate_up language model, CLIP tower read through the
    # high-definition tiling (28-pixel tiles of 2x2 patches, so each tile merges into one feature)
    "tiny-phi3v": {
        "model_type": "phi3_v", "hidden_size": 256, "intermediate_size": 688, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 4, "vocab_size": 32064, "rms_norm_eps": 1e-5,
        "rope_theta": 10000.0, "max_position_embeddings": 4096,
        "vision_config": {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
                          "num_attention_heads": 4, "image_size": 56, "patch_size": 14,
                          "hidden_act": "quick_gelu", "layer_norm_eps": 1e-5, "hd_num": 4},
    },
    # 3-layer DeepSeek-V2-shaped model: latent attention (128 + 64 wide heads), one dense layer, then
    # layers with 8 routed experts (4 groups) and 2 shared experts
    "tiny-deepseek-v2": {
        "model_type": "deepseek_v2", "hidden_size": 512, "intermediate_size": 1024, "num_hidden_layers": 3,
        "num_attention_heads": 4, "num_key_value_heads": 4, "vocab_size": 32000, "rms_norm_eps": 1e-6,
        "rope_theta": 10000.0, "max_position_embeddings": 4096, "q_lora_rank": None, "kv_lora_rank": 128,
        "qk_nope_head_dim": 128, "qk_rope_head_dim": 64, "v_head_dim": 128, "n_routed_experts": 8,
        "n_shared_experts": 2, "num_experts_per_tok": 2, "moe_intermediate_size": 256,
        "first_k_dense_replace": 1, "topk_method": "group_limited_greedy", "n_group": 4, "topk_group": 2,
        "routed_scaling_factor": 1.0, "norm_topk_prob": False,
    },
    # the same with the compressed cache: one [rotary key | latent] row per token instead of per-head keys / values
    "tiny-deepseek-v2-latent": {
        "model_type": "deepseek_v2", "hidden_size": 512, "intermediate_size": 1024, "num_hidden_layers": 3,
        "num_attention_heads": 4, "num_key_value_heads": 4, "vocab_size": 32000, "rms_norm_eps": 1e-6,
        "rope_theta": 10000.0, "max_position_embeddings": 4096, "q_lora_rank": None, "kv_lora_rank": 128,
        "qk_nope_head_dim": 128, "qk_rope_head_dim": 64, "v_head_dim": 128, "n_routed_experts": 8,
        "n_shared_experts": 2, "num_experts_per_tok": 2, "moe_intermediate_size": 256,
        "first_k_dense_replace": 1, "topk_method": "group_limited_greedy", "n_group": 4, "topk_group": 2,
        "routed_scaling_factor": 1.0, "norm_topk_prob": False, "mla_cache": "latent",
    },
    "tiny-rwkv5": {
        "model_type": "rwkv5", "hidden_size": 128, "num_hidden_layers": 2, "head_size": 32, "vocab_size": 32000,
        "layer_norm_epsilon": 1e-5, "rescale_every": 0,
    },
    "tiny-rwkv6": {
        "model_type": "rwkv6", "hidden_size": 128, "num_hidden_layers": 2, "head_size": 32, "vocab_size": 32000,
        "layer_norm_epsilon": 1e-5, "rescale_every": 0,
    },
    # GPU-friendly small model (head_dim 128, dimensions multiples of 128)
    "tiny-llama-gpu": {
        "model_type": "llama", "hidden_size": 512, "intermediate_size": 1024, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 4096,
    },
    # LayerNorm families (GPU numerics of the LayerNorm / plain-activation kernels at model level)
    "tiny-gpt2-gpu": {
        "model_type": "gpt2", "n_embd": 256, "n_head": 2, "n_layer": 2, "n_positions": 1024, "n_inner": 1024,
        "vocab_size": 32000, "layer_norm_epsilon": 1e-5,
    },
    "tiny-neox-gpu": {
        "model_type": "gpt_neox", "hidden_size": 256, "intermediate_size": 1024, "num_hidden_layers": 2,
        "num_attention_heads": 2, "vocab_size": 32000, "layer_norm_eps": 1e-5, "rotary_pct": 0.25,
        "rotary_emb_base": 10000, "max_position_embeddings": 2048, "use_parallel_residual": True,
    },
    "tiny-starcoder2-gpu": {
        "model_type": "starcoder2", "hidden_size": 256, "intermediate_size": 1024, "num_hidden_layers": 2,
        "num_attention_heads": 2, "num_key_value_heads": 1, "vocab_size": 32000, "norm_epsilon": 1e-5,
        "rope_theta": 10000.0, "max_position_embeddings": 2048,
    },
    # alternating sliding-window / full layers, attention and final logit soft-capping (masked attention paths)
    "tiny-gemma2-gpu": {
        "model_type": "gemma2", "hidden_size": 512, "intermediate_size": 1024, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 32000,
        "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 4096, "sliding_window": 48,
        "attn_logit_softcapping": 30.0, "final_logit_softcapping": 20.0, "query_pre_attn_scalar": 128,
    },
    # small models whose every sharded dimension divides by 8 (multi-rank tests up to 8 GPUs)
    "tiny-llama-tp8": {
        "model_type": "llama", "hidden_size": 1024, "intermediate_size": 2048, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 4096,
    },
    # one-block EAGLE head for tiny-llama-tp8
    "tiny-eagle-tp8": {
        "model_type": "eagle", "hidden_size": 1024, "intermediate_size": 2048, "num_hidden_layers": 1,
        "num_attention_heads": 8, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 4096, "bias": True,
    },
    "tiny-mixtral-tp8": {
        "model_type": "mixtral", "hidden_size": 1024, "intermediate_size": 1024, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 4096,
        "num_local_experts": 8, "num_experts_per_tok": 2,
    },
    "llama-3-8b": {
        "model_type": "llama", "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 8192,
    },
    "llama-3-70b": {
        "model_type": "llama", "hidden_size": 8192, "intermediate_size": 28672, "num_hidden_layers": 80,
        "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 8192,
    },
    # 2-layer Llama-3-shaped draft model for speculative decoding
    "llama-3-draft-2l": {
        "model_type": "llama", "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 2,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 8192,
    },
    "llama-2-7b": {
        "model_type": "llama", "hidden_size": 4096, "intermediate_size": 11008, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 32, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "max_position_embeddings": 4096,
    },
    "mistral-7b": {
        "model_type": "mistral", "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 8, "vocab_size": 32000, "rms_norm_eps": 1e-5,
        "rope_theta": 10000.0, "max_position_embeddings": 32768, "sliding_window": 4096,
    },
    "mixtral-8x7b": {
        "model_type": "mixtral", "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 8, "vocab_size": 32000, "rms_norm_eps": 1e-5,
        "rope_theta": 1000000.0, "max_position_embeddings": 32768, "num_local_experts": 8,
        "num_experts_per_tok": 2,
    },
    "tiny-mixtral": {
        "model_type": "mixtral", "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 2048,
        "num_local_experts": 4, "num_experts_per_tok": 2,
    },
    "tiny-mixtral-gpu": {
        "model_type": "mixtral", "hidden_size": 512, "intermediate_size": 1024, "num_hidden_layers": 2,
        "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 32000,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 4096,
        "num_local_experts": 8, "num_experts_per_tok": 2,
    },
    "qwen2-7b": {
        "model_type": "qwen2", "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
        "num_attention_heads": 28, "num_key_value_heads": 4, "vocab_size": 152064, "rms_norm_eps": 1e-6,
        "rope_theta": 1000000.0, "max_position_embeddings": 32768,
    },
    "qwen3-8b": {
        "model_type": "qwen3", "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 36,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936,
        "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 40960,
    },
    "gemma-2b": {
        "model_type": "gemma", "hidden_size": 2048, "intermediate_size": 16384, "num_hidden_layers": 18,
        "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 256, "vocab_size": 256000,
        "rms_norm_eps": 1e-6, "max_position_embeddings": 8192,
    },
    "gemma2-9b": {
        "model_type": "gemma2", "hidden_size": 3584, "intermediate_size": 14336, "num_hidden_layers": 42,
        "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 256, "vocab_size": 256000,
        "rms_norm_eps": 1e-6, "max_position_embeddings": 8192, "query_pre_attn_scalar": 256,
        "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "sliding_window": 4096,
    },
    "phi-3-mini": {
        "model_type": "phi3", "hidden_size": 3072, "intermediate_size": 8192, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 32, "vocab_size": 32064, "rms_norm_eps": 1e-5,
        "max_position_embeddings": 4096,
    },
    "phi-2": {
        "model_type": "phi", "hidden_size": 2560, "intermediate_size": 10240, "num_hidden_layers": 32,
        "num_attention_heads": 32, "vocab_size": 51200, "layer_norm_eps": 1e-5,
        "max_position_embeddings": 2048, "partial_rotary_factor": 0.4,
    },
    "gpt2": {
        "model_type": "gpt2", "n_embd": 768, "n_layer": 12, "n_head": 12, "vocab_size": 50257,
        "layer_norm_epsilon": 1e-5, "n_positions": 1024,
    },
    "gpt-neox-pythia-1b": {
        "model_type": "gpt_neox", "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
        "num_attention_heads": 8, "vocab_size": 50304, "layer_norm_eps": 1e-5,
        "max_position_embeddings": 2048, "rotary_pct": 0.25, "use_parallel_residual": True,
    },
    "qwen2-moe-a2.7b": {
        "model_type": "qwen2_moe", "hidden_size": 2048, "intermediate_size": 5632, "num_hidden_layers": 24,
        "num_attention_heads": 16, "num_key_value_heads": 16, "vocab_size": 151936, "rms_norm_eps": 1e-6,
        "num_experts": 60, "num_experts_per_tok": 4, "moe_intermediate_size": 1408,
        "shared_expert_intermediate_size": 5632, "max_position_embeddings": 8192,
    },
}


def _public_presets() -> dict:
    """Architecture hyper-parameters of published checkpoints under the names the reference's
    ``gen_config`` accepts (``python/mlc_llm/model/model_preset.py``: ``llama2_7b``, ``mistral_7b``,
    ``phi-3_5`` ...), kept as a data file next to this module."""
    import json  # pylint: disable=import-outside-toplevel
    import os  # pylint: disable=import-outside-toplevel

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "public_presets.json")
    if not os.path.isfile(path):
        return {}
    with open(path, encoding="utf-8") as f:
        return json.load(f)


for _name, _cfg in _public_presets().items():
    MODEL_PRESETS.setdefault(_name, _cfg)
