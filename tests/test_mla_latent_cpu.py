"""Latent attention over the compressed cache (one [rotary key | latent] row per token for all heads) against the
expanded form (per-head keys and values cached): same tokens, a fraction of the cache."""
import numpy as np
import torch

from mlc_llm_b200 import ops
from mlc_llm_b200.ops import reference as ref
from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

from test_distributed_cpu import _run

MODEL = "random://tiny-deepseek-v2?quant=q0f32&seed=5"
GREEDY = {"temperature": 0.0, "debug_config": {"ignore_eos": True}, "max_tokens": 12}


def _engine(extra="", **kw):
    cfg = dict(mode="server", max_num_sequence=8, prefill_chunk_size=32, max_total_sequence_length=2048)
    cfg.update(kw)
    return SyncMLCEngine(MODEL + extra, "cpu", engine_config=EngineConfig(**cfg))


def test_latent_cache_gives_the_tokens_of_the_expanded_cache():
    rng = np.random.default_rng(0)
    prompts = [rng.integers(10, 31000, int(n)).tolist() for n in (37, 9, 70)]  # 70 > chunk: chunked prefill
    want_eng = _engine()
    got_eng = _engine("&mla_cache=latent")
    big, small = want_eng.runtime.models[0], got_eng.runtime.models[0]
    assert not big.mla_latent and small.mla_latent
    m = small.cfg.extra["mla"]
    assert small.kv_pages.shape[2:] == (1, 1, 16, m["qk_rope_head_dim"] + m["kv_lora_rank"])
    assert small.kv_bytes_per_token() * 8 == big.kv_bytes_per_token()  # 4 heads x (192 + 192) against 192
    _, want = want_eng.generate(prompts, GREEDY)
    _, got = got_eng.generate(prompts, GREEDY)
    assert [t[0] for t in got] == [t[0] for t in want]


def test_latent_cache_with_speculative_verification_and_prefix_reuse():
    """Tree verification (the tree-mask rule of the latent kernel's reference) and copy-on-write / token moves of
    the one-row cache: a small draft model proposes, output stays the plain greedy output; a second request
    sharing a prefix reuses pages."""
    rng = np.random.default_rng(1)
    shared = rng.integers(10, 31000, 48).tolist()
    prompts = [shared + rng.integers(10, 31000, 7).tolist(), shared + rng.integers(10, 31000, 11).tolist()]
    _, want = _engine().generate(prompts, GREEDY)
    eng = _engine("&mla_cache=latent", speculative_mode="small_draft", spec_draft_length=3,
                  additional_models=["random://tiny-llama?quant=q0f32&seed=2"], prefix_cache_mode="radix")
    _, got = eng.generate(prompts, GREEDY)
    assert [t[0] for t in got] == [t[0] for t in want]


def test_absorbed_scores_equal_expanded_scores():
    """The identity the latent path rests on, on random tensors: with k = [k_rope | W_uk latent] and
    v = W_uv latent per head, attention over (k, v) equals absorbed attention over rows [k_rope | latent]
    followed by W_uv."""
    torch.manual_seed(0)
    t, hq, rope, nope, rank, vd, page = 5, 3, 64, 32, 128, 48, 16
    n_ctx = 40
    latent = torch.randn(n_ctx, rank)
    k_rope = torch.randn(n_ctx, rope)
    w_uk = torch.randn(hq, nope, rank) * 0.1
    w_uv = torch.randn(hq, vd, rank) * 0.1
    q = torch.randn(t, hq, rope + nope)
    kvlen = torch.tensor([36, 37, 38, 39, 40], dtype=torch.int32)
    # expanded oracle
    k = torch.cat([k_rope[:, None, :].expand(n_ctx, hq, rope), torch.einsum("hnr,cr->chn", w_uk, latent)], -1)
    v = torch.einsum("hvr,cr->chv", w_uv, latent)
    want = torch.zeros(t, hq, vd)
    for i in range(t):
        n = int(kvlen[i])
        s = torch.einsum("hd,chd->hc", q[i], k[:n]) * 0.11
        want[i] = torch.einsum("hc,chv->hv", torch.softmax(s, -1), v[:n])
    # absorbed over a paged cache
    pages = 4
    cache = torch.zeros(pages, 1, 1, page, rope + rank)
    slots = torch.arange(n_ctx, dtype=torch.int32) + page  # pages 1..3
    ops.mla_append(torch.cat([k_rope, latent], -1), cache, slots, page)
    q_abs = torch.cat([q[..., :rope], torch.einsum("thn,hnr->thr", q[..., rope:], w_uk)], -1)
    ctx = ops.mla_attention(q_abs, cache, torch.zeros(t, dtype=torch.int32), kvlen,
                            torch.tensor([0, 3], dtype=torch.int32), torch.tensor([1, 2, 3], dtype=torch.int32),
                            rope, rank, page, 0.11)
    got = torch.einsum("thr,hvr->thv", ctx, w_uv)
    assert torch.allclose(got, want, atol=1e-4), float((got - want).abs().max())
    assert ref.mla_attention is not None


def test_tp2_latent_cache_matches_single_rank():
    """Heads split over two gloo ranks, the latent row replicated on both."""
    single = _run(1, MODEL, port=29561)
    tp2 = _run(2, MODEL + "&mla_cache=latent", port=29562)
    assert single == tp2
