"""Image inputs: CLIP tower + LLaVA projector against HuggingFace transformers, pre-processing, and an
image request through the public chat API."""
import base64
import io
import json

import numpy as np
import pytest
import torch

from mlc_llm_b200 import _core
from mlc_llm_b200 import quantization as Q
from mlc_llm_b200.models import config as mc
from mlc_llm_b200.models import loader
from mlc_llm_b200.models import vision as V
from mlc_llm_b200.models.transformer import BatchInfo, DecoderModel

transformers = pytest.importorskip("transformers")


def _batch(plan):
    t = lambda k: torch.from_numpy(np.asarray(plan[k])).to(torch.int32)
    return BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                     page_indptr=t("page_indptr"), page_indices=t("page_indices"),
                     num_tokens=len(plan["positions"]))


def test_preprocessing_resizes_crops_and_normalises():
    from PIL import Image

    img = Image.new("RGB", (60, 40), (255, 0, 128))
    pixels, rows = V.preprocess_image(img, {"vision_config": {"image_size": 28, "patch_size": 14}})
    assert pixels.shape == (3, 28, 28) and rows == 4
    want = [(1.0 - V.CLIP_MEAN[0]) / V.CLIP_STD[0], (0.0 - V.CLIP_MEAN[1]) / V.CLIP_STD[1],
            (128 / 255 - V.CLIP_MEAN[2]) / V.CLIP_STD[2]]
    for c in range(3):
        assert torch.allclose(pixels[c], torch.full((28, 28), want[c]), atol=1e-5)
    # portrait input: the short edge becomes 28, the long edge is centre-cropped
    tall = torch.zeros(1, 3, 80, 40)
    tall[:, :, 26:54] = 255.0   # the band that survives the crop after scaling 40 -> 28
    out = V.preprocess_pixels(tall, 28)
    assert out.shape == (1, 3, 28, 28)
    assert out[0, 0, 10:18].mean() > out[0, 0, :2].mean()


def test_llava_matches_transformers(tmp_path):
    if not hasattr(transformers, "LlavaForConditionalGeneration"):
        pytest.skip("transformers has no LLaVA")
    torch.manual_seed(0)
    text = transformers.LlamaConfig(hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, vocab_size=160,
                                    max_position_embeddings=128)
    vis = transformers.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                                        num_attention_heads=4, image_size=28, patch_size=14,
                                        projection_dim=32)
    hf_cfg = transformers.LlavaConfig(vision_config=vis, text_config=text, image_token_index=159,
                                      vision_feature_layer=-2, vision_feature_select_strategy="default")
    hf = transformers.LlavaForConditionalGeneration(hf_cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)
    hf.save_pretrained(tmp_path, safe_serialization=True)
    raw = json.load(open(tmp_path / "config.json"))
    cfg = mc.from_dict(raw["model_type"], raw)
    assert cfg.extra["vision"]["image_size"] == 28 and cfg.hidden_size == 64

    # ---- image rows
    pixels = torch.randn(1, 3, 28, 28)
    tower = V.VisionTower(cfg.extra["vision"], V.load_hf_vision_params(str(tmp_path), cfg.extra["vision"], 64),
                          torch.device("cpu"), torch.float32)
    got_rows = tower.embed(pixels)
    with torch.no_grad():
        want_rows = hf.get_image_features(pixel_values=pixels, vision_feature_layer=-2,
                                          vision_feature_select_strategy="default")
    if hasattr(want_rows, "pooler_output"):   # newer transformers wrap the projected rows
        want_rows = want_rows.pooler_output
    want_rows = want_rows[0] if isinstance(want_rows, (list, tuple)) else want_rows
    want_rows = want_rows.reshape(-1, 64)
    assert got_rows.shape == (4, 64)
    assert (got_rows - want_rows).abs().max() < 1e-4, (got_rows - want_rows).abs().max()

    # ---- logits of a prompt with the image in the middle
    quant = Q.get("q0f32")
    store = loader.load_hf_params(str(tmp_path), cfg, quant, torch.device("cpu"))
    model = DecoderModel(cfg, quant, store, torch.device("cpu"))
    model.create_kv_cache(16, 16)
    kv = _core.KVManager(16, 16, 4)
    kv.add_sequence(0)
    before, after = torch.randint(0, 150, (5,)), torch.randint(0, 150, (6,))
    ids = torch.cat([before, torch.full((4,), 159), after])
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=pixels).logits[0].float()
    x = torch.cat([model.embed(before.to(torch.int32)), got_rows.to(model.dtype),
                   model.embed(after.to(torch.int32))])
    plan = kv.begin_forward([0], [15])
    h = model.forward(x, _batch(plan))
    got = model.logits(h, torch.arange(15, dtype=torch.int32)).float()
    assert (got - want).abs().max() < 2e-3, (got - want).abs().max()


def test_image_request_through_the_chat_api():
    from PIL import Image

    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.engine import MLCEngine

    img = Image.fromarray((np.random.default_rng(0).random((40, 60, 3)) * 255).astype(np.uint8))
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    eng = MLCEngine("random://tiny-llava?quant=q0f32&seed=2", "cpu", mode="server",
                    engine_config=EngineConfig(max_num_sequence=4, max_total_sequence_length=1024,
                                               prefill_chunk_size=64))
    try:
        text_only = eng.chat.completions.create(messages=[{"role": "user", "content": "what is this"}],
                                                max_tokens=4, temperature=0.0)
        with_image = eng.chat.completions.create(
            messages=[{"role": "user", "content": [{"type": "text", "text": "what is this"},
                                                    {"type": "image_url", "image_url": {"url": url}}]}],
            max_tokens=4, temperature=0.0)
        # four patch rows and the newline that follows an image
        assert with_image.usage.prompt_tokens == text_only.usage.prompt_tokens + 4 + 1
        assert with_image.usage.completion_tokens == 4
    finally:
        eng.terminate()
