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


def test_image_request_through_the_json_ffi_engine():
    """The native JSON front end takes image content parts: it pulls the bytes out of the data URL, the host
    embeds them, and the rows sit between the text pieces of the rendered prompt."""
    from PIL import Image

    from mlc_llm_b200 import _core
    from mlc_llm_b200.json_ffi.engine import JSONFFIEngine
    from mlc_llm_b200.serve.config import EngineConfig

    img = Image.fromarray((np.random.default_rng(0).random((40, 60, 3)) * 255).astype(np.uint8))
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    assert _core.JsonFFIEngine.decode_data_url(url) == buf.getvalue()
    with pytest.raises(Exception, match="data URL"):
        _core.JsonFFIEngine.decode_data_url("http://example.com/cat.png")
    eng = JSONFFIEngine("random://tiny-llava?quant=q0f32&seed=2", "cpu", mode="server",
                        engine_config=EngineConfig(max_num_sequence=4, max_total_sequence_length=1024,
                                                   prefill_chunk_size=64))
    try:
        def usage(messages):
            last = None
            for chunk in eng.chat.completions.create(messages=messages, max_tokens=4, temperature=0.0,
                                                     stream_options={"include_usage": True}):
                last = chunk
            return last.usage

        text_only = usage([{"role": "user", "content": "what is this"}])
        with_image = usage([{"role": "user", "content": [{"type": "text", "text": "what is this"},
                                                         {"type": "image_url", "image_url": {"url": url}}]}])
        assert with_image.prompt_tokens == text_only.prompt_tokens + 4 + 1
        assert with_image.completion_tokens == 4
    finally:
        eng.terminate()


# ---------------------------------------------------------------------------- Phi-3-vision
def test_phi3v_hd_geometry():
    """Tile grid and prompt-row count of the high-definition transform for the sizes the full model uses
    (336-pixel tiles of 24x24 patches, at most four tiles)."""
    from mlc_llm_b200.models import vision as V

    # 1000 x 600 (w x h): two tiles wide, 403 rows padded to two tiles high -> 2x2 tiles
    new_h, new_w, padded_h = V.hd_target_shape(600, 1000, 336, 4)
    assert (new_h, new_w, padded_h) == (403, 672, 672)
    assert V.hd_embed_size(2, 2, 24) == (2 * 2 + 1) * 144 + 1 + (2 + 1) * 12  # 757, the published count
    # a very wide image: four tiles in one row
    new_h, new_w, padded_h = V.hd_target_shape(100, 1200, 336, 4)
    assert (new_w // 336, padded_h // 336) == (4, 1)
    px = V.hd_preprocess_pixels(torch.rand(3, 600, 1000) * 255, 336, 4)
    assert tuple(px.shape) == (3, 672, 672)
    # portrait images are tiled the other way round
    px = V.hd_preprocess_pixels(torch.rand(3, 1200, 100) * 255, 336, 4)
    assert tuple(px.shape) == (3, 4 * 336, 336)
    # padding is white: the first row of a padded landscape image is the normalised value of 255
    px = V.hd_preprocess_pixels(torch.zeros(3, 100, 500), 336, 4)
    white = (1.0 - V.CLIP_MEAN[0]) / V.CLIP_STD[0]
    assert abs(float(px[0, 0, 0]) - white) < 1e-5


def test_phi3v_embedding_order_matches_a_per_entry_restatement():
    """Rows: tile-grid features (2x2 patch blocks on the channel axis, a separator after every feature
    row), the view separator, then the global view; checked entry by entry against plain loops over the
    tower's own CLIP features."""
    from mlc_llm_b200.models import config as C
    from mlc_llm_b200.models import presets
    from mlc_llm_b200.models import vision as V

    cfg = C.from_dict("phi3_v", presets.MODEL_PRESETS["tiny-phi3v"])
    vis = cfg.extra["vision"]
    assert vis["kind"] == "phi3v"
    params = V.Phi3VisionTower.random_params(vis, cfg.hidden_size, 5)
    g = torch.Generator().manual_seed(1)
    params[V.Phi3VisionTower.G + "sub_GN"] = torch.randn(1, 1, 1, 256, generator=g)
    params[V.Phi3VisionTower.G + "glb_GN"] = torch.randn(1, 1, 256, generator=g)
    tower = V.Phi3VisionTower(vis, params, torch.device("cpu"), torch.float32)
    s, side = 56, 4
    h_crop, w_crop = 1, 3
    pixels = torch.randn(3, h_crop * s, w_crop * s, generator=g)
    rows = tower.embed(pixels)
    assert rows.shape == (V.hd_embed_size(h_crop, w_crop, side), cfg.hidden_size)

    # restatement with loops
    glob = torch.nn.functional.interpolate(pixels.unsqueeze(0), size=(s, s), mode="bicubic", align_corners=False)
    views = [glob[0]] + [pixels[:, i * s:(i + 1) * s, j * s:(j + 1) * s] for i in range(h_crop) for j in range(w_crop)]
    feats = tower.features(torch.stack(views))[:, 1:]  # [1 + tiles, 16, 64]
    m = side // 2

    def block(view, r, c):  # the 2x2 patch block (r, c) of one view, row-major on the channel axis
        idx = [(2 * r + dr) * side + (2 * c + dc) for dr in range(2) for dc in range(2)]
        return torch.cat([feats[view, i] for i in idx])

    sub_gn = params[V.Phi3VisionTower.G + "sub_GN"].view(-1)
    glb_gn = params[V.Phi3VisionTower.G + "glb_GN"].view(-1)
    seq = []
    for gr in range(h_crop * m):
        for gc in range(w_crop * m):
            tile = (gr // m) * w_crop + (gc // m)
            seq.append(block(1 + tile, gr % m, gc % m))
        seq.append(sub_gn)
    seq.append(glb_gn)
    for r in range(m):
        for c in range(m):
            seq.append(block(0, r, c))
        seq.append(sub_gn)
    x = torch.stack(seq)
    P = V.Phi3VisionTower.P
    want = torch.nn.functional.gelu(x @ params[P + "0.weight"].t() + params[P + "0.bias"]) @ params[P + "2.weight"].t() \
        + params[P + "2.bias"]
    assert torch.allclose(rows, want, atol=1e-5, rtol=1e-4)


def test_phi3v_image_request_through_the_chat_api():
    from PIL import Image

    from mlc_llm_b200.models import vision as V
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.engine import MLCEngine

    img = Image.fromarray((np.random.default_rng(0).random((40, 100, 3)) * 255).astype(np.uint8))
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    eng = MLCEngine("random://tiny-phi3v?quant=q0f32&seed=2", "cpu", mode="server",
                    engine_config=EngineConfig(max_num_sequence=4, max_total_sequence_length=1024,
                                               prefill_chunk_size=64))
    try:
        text_only = eng.chat.completions.create(messages=[{"role": "user", "content": "what is this"}],
                                                max_tokens=4, temperature=0.0)
        with_image = eng.chat.completions.create(
            messages=[{"role": "user", "content": [{"type": "text", "text": "what is this"},
                                                    {"type": "image_url", "image_url": {"url": url}}]}],
            max_tokens=4, temperature=0.0)
        # 100 x 40: ratio 2.5 -> scale 2... the grid follows hd_target_shape; rows follow hd_embed_size
        new_h, new_w, padded_h = V.hd_target_shape(40, 100, 56, 4)
        rows = V.hd_embed_size(padded_h // 56, new_w // 56, 4)
        assert with_image.usage.prompt_tokens == text_only.usage.prompt_tokens + rows + 1
        assert with_image.usage.completion_tokens == 4
    finally:
        eng.terminate()
