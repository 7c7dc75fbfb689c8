"""Multimodal rotary positions: position triples for prompts with image / video grids and the sectioned
rotation, against HuggingFace's Qwen2.5-VL code where its conventions agree and against hand-written
expectations elsewhere; the Qwen2.5-VL language model on text against transformers."""
import json

import numpy as np
import pytest
import torch

from mlc_llm_b200.ops import mrope

transformers = pytest.importorskip("transformers")

META = mrope.VisionPositionMetadata(vision_start_token_id=90, image_token_id=91, video_token_id=92,
                                    spatial_merge_size=2, tokens_per_second=1.0)


def test_text_only_positions_count_up():
    pos, delta = mrope.sequence_position_ids([1, 2, 3, 4], META)
    assert pos.tolist() == [[0, 1, 2, 3]] * 3 and delta == 0


def test_image_block_positions_by_hand():
    # two text tokens, start marker, a 1x4x6 patch grid (2x3 after merging), two text tokens
    toks = [5, 6, 90] + [91] * 6 + [7, 8]
    pos, delta = mrope.sequence_position_ids(toks, META, image_grids=[(1, 4, 6)])
    assert pos[:, :3].tolist() == [[0, 1, 2]] * 3
    assert pos[0, 3:9].tolist() == [3] * 6                       # one frame
    assert pos[1, 3:9].tolist() == [3, 3, 3, 4, 4, 4]            # rows
    assert pos[2, 3:9].tolist() == [3, 4, 5, 3, 4, 5]            # columns
    assert pos[:, 9:].tolist() == [[6, 7]] * 3                   # text resumes after the largest index used
    assert delta == 8 - len(toks)


def test_video_block_time_axis_by_hand():
    meta = mrope.VisionPositionMetadata(90, 91, 92, spatial_merge_size=2, tokens_per_second=25.0)
    toks = [90] + [92] * 12 + [7]
    pos, _ = mrope.sequence_position_ids(toks, meta, video_grids=[(3, 4, 4)], second_per_grid=[2.0])
    # three frames of 2x2 merged patches, 50 positions apart in time
    assert pos[0, 1:13].tolist() == [1] * 4 + [51] * 4 + [101] * 4
    assert pos[1, 1:5].tolist() == [1, 1, 2, 2] and pos[2, 1:5].tolist() == [1, 2, 1, 2]
    assert pos[:, 13].tolist() == [102] * 3


def test_image_positions_match_transformers():
    from transformers.models.qwen2_5_vl import modeling_qwen2_5_vl as M

    cfg = transformers.Qwen2_5_VLConfig(
        text_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                         num_key_value_heads=2, vocab_size=100, rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3],
                                                                                  "rope_theta": 10000.0}),
        vision_config=dict(depth=1, hidden_size=16, intermediate_size=32, num_heads=2, out_hidden_size=32,
                           spatial_merge_size=2, tokens_per_second=1),
        vision_start_token_id=90, image_token_id=91, video_token_id=92)
    model = M.Qwen2_5_VLModel(cfg)
    rows = [[0, 0, 0, 5, 6, 90] + [91] * 6 + [7, 8, 90] + [91] * 4 + [9],
            [0, 0, 0, 0, 3, 90] + [91] * 8 + [4, 4, 4, 4, 4, 4]]
    grids = [(1, 4, 6), (1, 4, 4), (1, 8, 4)]
    ids = torch.tensor(rows)
    mask = torch.ones_like(ids)
    mask[1, :4] = 0
    mask[0, :3] = 0
    types = (ids == 91).int()
    want, want_delta = model.get_rope_index(ids, types, image_grid_thw=torch.tensor(grids), attention_mask=mask)
    got, got_delta = mrope.mrope_position_ids(ids.numpy(), META, attention_mask=mask.numpy(), image_grids=grids)
    keep = mask.bool().numpy()
    assert np.array_equal(got[:, keep], want.numpy()[:, keep])
    assert np.array_equal(got_delta, want_delta.numpy())


def test_sectioned_rotation_matches_transformers():
    from transformers.models.qwen2_5_vl import modeling_qwen2_5_vl as M

    torch.manual_seed(0)
    t, hq, hk, d = 7, 4, 2, 16
    section = [2, 3, 3]
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    pos = torch.randint(0, 50, (3, t))
    q, k = torch.randn(t, hq, d), torch.randn(t, hk, d)
    got_q, got_k = mrope.apply_mrope(q, k, pos, inv_freq, section)
    ang = pos[:, None, :, None].float() * inv_freq          # [3, 1, T, D/2]
    emb = torch.cat([ang, ang], dim=-1)
    want_q, want_k = M.apply_multimodal_rotary_pos_emb(q.transpose(0, 1)[None], k.transpose(0, 1)[None], emb.cos(),
                                                       emb.sin(), section)
    assert torch.allclose(got_q, want_q[0].transpose(0, 1), atol=1e-5)
    assert torch.allclose(got_k, want_k[0].transpose(0, 1), atol=1e-5)
    # equal positions on the three axes: plain rotary embedding
    same = pos[:1].expand(3, -1)
    a, _ = mrope.apply_mrope(q, k, same, inv_freq, section)
    angle = same[0].float()[:, None] * inv_freq
    cos, sin = torch.cat([angle.cos()] * 2, -1)[:, None], torch.cat([angle.sin()] * 2, -1)[:, None]
    plain = q * cos + torch.cat([-q[..., d // 2:], q[..., : d // 2]], -1) * sin
    assert torch.allclose(a, plain, atol=1e-5)


def test_qwen2_5_vl_text_logits_match_transformers(tmp_path):
    from mlc_llm_b200 import _core
    from mlc_llm_b200 import quantization as Q
    from mlc_llm_b200.models import config as mc
    from mlc_llm_b200.models import loader
    from mlc_llm_b200.models.transformer import BatchInfo, DecoderModel

    torch.manual_seed(0)
    cfg = transformers.Qwen2_5_VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=160, max_position_embeddings=128,
                         rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3], "rope_theta": 10000.0}),
        vision_config=dict(depth=1, hidden_size=16, intermediate_size=32, num_heads=2, out_hidden_size=64),
        vision_start_token_id=150, image_token_id=151, video_token_id=152)
    hf = transformers.Qwen2_5_VLForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.05)
    hf.save_pretrained(tmp_path, safe_serialization=True)
    raw = json.load(open(tmp_path / "config.json"))
    mcfg = mc.from_dict(raw["model_type"], raw)
    assert mcfg.extra["mrope_section"] == [2, 3, 3] and mcfg.attention_bias
    quant = Q.get("q0f32")
    store = loader.load_hf_params(str(tmp_path), mcfg, quant, torch.device("cpu"))
    model = DecoderModel(mcfg, quant, store, torch.device("cpu"))
    model.create_kv_cache(16, 16)
    kv = _core.KVManager(16, 16, 4)
    kv.add_sequence(0)
    toks = torch.randint(0, 140, (20,))
    with torch.no_grad():
        want = hf(input_ids=toks[None]).logits[0].float()
    plan = kv.begin_forward([0], [20])
    t = lambda key: torch.from_numpy(np.asarray(plan[key])).to(torch.int32)
    b = BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                  page_indptr=t("page_indptr"), page_indices=t("page_indices"), num_tokens=20)
    h = model.forward(model.embed(toks.to(torch.int32)), b)
    got = model.logits(h, torch.arange(20, dtype=torch.int32)).float()
    assert (got - want).abs().max() < 2e-3, (got - want).abs().max()
