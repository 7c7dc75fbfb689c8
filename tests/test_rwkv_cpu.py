"""RWKV-5 recurrent model: the batched / chunked forward against a naive token-by-token restatement of the
reference math, and generation through the engine (chunked prefill, several sequences, greedy)."""
import json

import numpy as np
import torch
import torch.nn.functional as F

from mlc_llm_b200 import quantization as Q
from mlc_llm_b200.models import config as mc
from mlc_llm_b200.models import loader
from mlc_llm_b200.models.presets import MODEL_PRESETS
from mlc_llm_b200.models.rwkv import RwkvModel
from mlc_llm_b200.models.transformer import BatchInfo
from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.sync_engine import SyncMLCEngine


def _model(seed=3, preset="tiny-rwkv5"):
    hf = dict(MODEL_PRESETS[preset])
    cfg = mc.from_dict(hf["model_type"], hf)
    quant = Q.get("q0f32")
    m = RwkvModel(cfg, quant, loader.random_params(cfg, quant, seed, torch.device("cpu"), std=0.1),
                  torch.device("cpu"))
    m.create_kv_cache(4, 16)
    return m


def _batch(seq_ids, lens, starts):
    qi = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    z = torch.zeros(0, dtype=torch.int32)
    b = BatchInfo(positions=z, slots=z, q_seq=z, q_kvlen=z, page_indptr=z, page_indices=z, num_tokens=int(qi[-1]))
    b.seq_ids, b.q_indptr, b.start_positions = np.asarray(seq_ids), qi, np.asarray(starts)
    return b


def _naive_logits(m, tokens):
    """One sequence, one token at a time, written directly from the block equations."""
    c, p = m.cfg, m.p
    n, hs, hdim = c.hidden_size // c.head_dim, c.head_dim, c.hidden_size
    ln = lambda x, name: F.layer_norm(x, (hdim,), p.tensors[name + ".weight"], p.tensors[name + ".bias"], c.rms_norm_eps)
    att_x = [torch.zeros(hdim) for _ in range(c.num_hidden_layers)]
    ffn_x = [torch.zeros(hdim) for _ in range(c.num_hidden_layers)]
    S = [torch.zeros(n, hs, hs) for _ in range(c.num_hidden_layers)]
    outs = []
    for tok in tokens:
        x = p.tensors["model.embeddings.weight"][tok]
        for li in range(c.num_hidden_layers):
            pre = f"model.blocks.{li}."
            if li == 0:
                x = ln(x, pre + "pre_ln")
            h = ln(x, pre + "ln1")
            a = pre + "attention."
            v6 = c.extra["rwkv"] == 6
            if v6:
                t_ = p.tensors
                dx = att_x[li] - h
                low = torch.tanh((h + dx * t_[a + "time_maa_x"]) @ t_[a + "time_maa_w1"]).view(5, -1)
                corr = [low[j] @ t_[a + "time_maa_w2"][j] for j in range(5)]
                xw, xk_, xv_, xr_, xg_ = (h + dx * (t_[a + f"time_maa_{nm}"] + corr[j]) for j, nm in enumerate("wkvrg"))
                w = torch.exp(-torch.exp(t_[a + "time_decay"].view(n, hs) + (
                    torch.tanh(xw @ t_[a + "time_decay_w1"]) @ t_[a + "time_decay_w2"]).view(n, hs)))
            else:
                mix = lambda name: h * p.tensors[a + name] + att_x[li] * (1 - p.tensors[a + name])
                xr_, xk_, xv_, xg_ = mix("time_mix_receptance"), mix("time_mix_key"), mix("time_mix_value"), mix("time_mix_gate")
                w = p.tensors[a + "time_decay"]
            r = (p.linears[a + "receptance"].w @ xr_).view(n, hs)
            k = (p.linears[a + "key"].w @ xk_).view(n, hs)
            v = (p.linears[a + "value"].w @ xv_).view(n, hs)
            g = F.silu(p.linears[a + "gate"].w @ xg_)
            att_x[li] = h
            u = p.tensors[a + "time_faaaa"]
            out = torch.zeros(n, hs)
            for hd in range(n):
                for i in range(hs):
                    for kk in range(hs):
                        xkv = k[hd, kk] * v[hd, i]
                        out[hd, i] += r[hd, kk] * (u[hd, kk] * xkv + S[li][hd, i, kk])
                        S[li][hd, i, kk] = S[li][hd, i, kk] * w[hd, kk] + xkv
            out = F.group_norm(out.view(1, hdim), n, p.tensors[a + "ln_x.weight"], p.tensors[a + "ln_x.bias"], eps=1e-5)[0]
            x = x + p.linears[a + "output"].w @ (out * g)
            h = ln(x, pre + "ln2")
            f = pre + "feed_forward."
            if v6:
                xk = h + (ffn_x[li] - h) * p.tensors[f + "time_maa_k"]
                xr = h + (ffn_x[li] - h) * p.tensors[f + "time_maa_r"]
            else:
                xk = h * p.tensors[f + "time_mix_key"] + ffn_x[li] * (1 - p.tensors[f + "time_mix_key"])
                xr = h * p.tensors[f + "time_mix_receptance"] + ffn_x[li] * (1 - p.tensors[f + "time_mix_receptance"])
            ffn_x[li] = h
            rr = torch.sigmoid(p.linears[f + "receptance"].w @ xr)
            kk2 = torch.square(torch.relu(p.linears[f + "key"].w @ xk))
            x = x + rr * (p.linears[f + "value"].w @ kk2)
        outs.append(p.linears["head"].w @ ln(x, "model.ln_out"))
    return torch.stack(outs)


import pytest


@pytest.mark.parametrize("preset", ["tiny-rwkv5", "tiny-rwkv6"])
def test_batched_chunked_forward_equals_naive_recurrence(preset):
    m = _model(preset=preset)
    rng = np.random.default_rng(0)
    seq_a, seq_b = rng.integers(0, 32000, 7).tolist(), rng.integers(0, 32000, 5).tolist()
    want_a, want_b = _naive_logits(m, seq_a), _naive_logits(m, seq_b)
    # step 1: first 4 tokens of a together with all of b; step 2: the rest of a, one decode-sized chunk
    toks = torch.tensor(seq_a[:4] + seq_b, dtype=torch.int32)
    h = m.forward(m.embed(toks), _batch([11, 22], [4, 5], [0, 0]))
    got = m.logits(h, None)
    assert torch.allclose(got[:4], want_a[:4], atol=1e-4) and torch.allclose(got[4:], want_b, atol=1e-4)
    h = m.forward(m.embed(torch.tensor(seq_a[4:], dtype=torch.int32)), _batch([11], [3], [4]))
    assert torch.allclose(m.logits(h, None), want_a[4:], atol=1e-4)
    # a sequence restarted at position 0 gets a fresh state
    h = m.forward(m.embed(torch.tensor(seq_b, dtype=torch.int32)), _batch([11], [5], [0]))
    assert torch.allclose(m.logits(h, None), want_b, atol=1e-4)


@pytest.mark.parametrize("preset", ["tiny-rwkv5", "tiny-rwkv6"])
def test_engine_generates_with_recurrent_state(preset):
    eng = SyncMLCEngine(f"random://{preset}?quant=q0f32&seed=4", "cpu",
                        engine_config=EngineConfig(mode="server", max_num_sequence=4, prefill_chunk_size=16,
                                                   max_total_sequence_length=1024))
    assert json.loads(eng.runtime.complete_config_json)["prefix_cache_mode"] == "disable"
    rng = np.random.default_rng(1)
    prompts = [rng.integers(10, 31000, n).tolist() for n in (25, 9, 40)]
    cfg = {"max_tokens": 6, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    _, batched = eng.generate(prompts, cfg)
    single = [eng.generate([p], cfg)[1][0] for p in prompts]
    assert [b[0] for b in batched] == [s[0] for s in single]
    assert all(len(b[0]) == 6 for b in batched)
