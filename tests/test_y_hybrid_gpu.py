"""GPU runs of the recurrent-hybrid decoder and of the tiled image embedding against the same code on the
CPU in fp32 (the GEMMs, norms, rotary/append and attention go through this package's kernels on the GPU)."""
import numpy as np
import pytest
import torch

from mlc_llm_b200 import _core, quantization as Q
from mlc_llm_b200.models import config as mc, loader
from mlc_llm_b200.models.presets import MODEL_PRESETS
from mlc_llm_b200.models.transformer import BatchInfo

pytestmark = pytest.mark.gpu


def _batch(plan, device, seq_ids, starts):
    t = lambda k: torch.from_numpy(np.asarray(plan[k])).to(torch.int32).to(device)
    b = BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                  page_indptr=t("page_indptr"), page_indices=t("page_indices"), num_tokens=len(plan["positions"]))
    b.seq_ids, b.q_indptr, b.start_positions = np.asarray(seq_ids), np.asarray(plan["q_indptr"]), np.asarray(starts)
    return b


@pytest.mark.parametrize("quant", ["q0f16", "q4f16_1"])
def test_qwen35_forward_matches_cpu(quant):
    from mlc_llm_b200.models.qwen35 import Qwen35Model

    hf = dict(MODEL_PRESETS["tiny-qwen35"])
    cfg = mc.from_dict(hf["model_type"], hf)
    models = {}
    for dev in ("cuda", "cpu"):
        q = Q.get(quant)
        store = loader.random_params(cfg, q, 3, torch.device(dev), gen_device=torch.device("cpu"))
        models[dev] = Qwen35Model(cfg, q, store, torch.device(dev))
        models[dev].create_kv_cache(64, 16)
    kv = _core.KVManager(64, 16, 16)
    rng = np.random.default_rng(0)
    lens = [19, 5]
    for i in range(2):
        kv.add_sequence(i)
    steps = [(lens, [0, 0]), ([1, 1], lens), ([1, 1], [n + 1 for n in lens])]
    for qlens, starts in steps:
        plan = kv.begin_forward([0, 1], qlens)
        toks = rng.integers(0, 32000, sum(qlens)).astype(np.int32)
        rows = torch.from_numpy((np.cumsum(qlens) - 1).astype(np.int32))
        outs = []
        for dev, m in models.items():
            h = m.forward(m.embed(torch.from_numpy(toks).to(dev)), _batch(plan, dev, [0, 1], starts))
            outs.append(m.logits(h, rows.to(dev)).float().cpu())
        assert (outs[0] - outs[1]).abs().max() < 2e-2, (outs[0] - outs[1]).abs().max()


def test_phi3v_image_rows_match_cpu():
    from mlc_llm_b200.models import vision as V

    cfg = mc.from_dict("phi3_v", MODEL_PRESETS["tiny-phi3v"])
    vis = cfg.extra["vision"]
    params = V.Phi3VisionTower.random_params(vis, cfg.hidden_size, 5)
    pixels = torch.randn(3, 56, 168, generator=torch.Generator().manual_seed(1))
    cpu = V.Phi3VisionTower(vis, params, torch.device("cpu"), torch.float32).embed(pixels)
    gpu = V.Phi3VisionTower(vis, params, torch.device("cuda"), torch.float16).embed(pixels).float().cpu()
    assert gpu.shape == cpu.shape == (V.hd_embed_size(1, 3, 4), cfg.hidden_size)
    assert (gpu - cpu).abs().max() < 2e-2
