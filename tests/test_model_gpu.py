"""Whole-model numerics on the GPU against the fp32 CPU execution of the same weights, and the
engine end to end on the GPU."""
import json

import numpy as np
import pytest
import torch

from mlc_llm_b200 import _core, quantization as Q
from mlc_llm_b200.models import config as mc, loader
from mlc_llm_b200.models.presets import MODEL_PRESETS
from mlc_llm_b200.models.transformer import BatchInfo, DecoderModel

pytestmark = pytest.mark.gpu


def _build(preset, quant_name, device):
    hf = dict(MODEL_PRESETS[preset])
    cfg = mc.from_dict(hf["model_type"], hf)
    quant = Q.get(quant_name)
    store = loader.random_params(cfg, quant, 3, torch.device(device), gen_device=torch.device("cpu"))
    m = DecoderModel(cfg, quant, store, torch.device(device))
    m.create_kv_cache(64, 16)
    return m


def _batch(plan, device):
    t = lambda k, dt=torch.int32: torch.from_numpy(np.asarray(plan[k])).to(dt).to(device)
    return BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                     page_indptr=t("page_indptr"), page_indices=t("page_indices"),
                     num_tokens=len(plan["positions"]))


@pytest.mark.parametrize("preset,quant", [("tiny-llama-gpu", "q0f16"), ("tiny-llama-gpu", "q4f16_1"),
                                          ("tiny-llama-gpu", "q0bf16"), ("tiny-mixtral-gpu", "q0f16"),
                                          ("tiny-mixtral-gpu", "q4f16_1"), ("tiny-deepseek-v2", "q0f16"),
                                          ("tiny-deepseek-v2-latent", "q0f16"), ("tiny-deepseek-v2-latent", "q0bf16"),
                                          ("tiny-gpt2-gpu", "q0f16"), ("tiny-neox-gpu", "q0f16"),
                                          ("tiny-starcoder2-gpu", "q0f16"), ("tiny-gemma2-gpu", "q0bf16")])
def test_forward_matches_cpu(preset, quant):
    gpu = _build(preset, quant, "cuda")
    cpu = _build(preset, quant, "cpu")
    kv = _core.KVManager(64, 16, 16)
    rng = np.random.default_rng(0)
    lens = [37, 5, 64]
    for i in range(3):
        kv.add_sequence(i)
    plan = kv.begin_forward([0, 1, 2], lens)
    toks = rng.integers(0, 32000, sum(lens)).astype(np.int32)
    rows = np.cumsum(lens) - 1
    outs = []
    for m, dev in ((gpu, "cuda"), (cpu, "cpu")):
        b = _batch(plan, dev)
        x = m.embed(torch.from_numpy(toks).to(dev))
        h = m.forward(x, b)
        outs.append(m.logits(h, torch.from_numpy(rows.astype(np.int32)).to(dev)).float().cpu())
    tol = 6e-2 if quant == "q0bf16" else 2e-2
    assert (outs[0] - outs[1]).abs().max() < tol, (outs[0] - outs[1]).abs().max()
    # one decode step on top of the cached prefix
    plan2 = kv.begin_forward([0, 1, 2], [1, 1, 1])
    toks2 = rng.integers(0, 32000, 3).astype(np.int32)
    outs = []
    for m, dev in ((gpu, "cuda"), (cpu, "cpu")):
        b = _batch(plan2, dev)
        x = m.embed(torch.from_numpy(toks2).to(dev))
        h = m.forward(x, b)
        outs.append(m.logits(h, None).float().cpu())
    assert (outs[0] - outs[1]).abs().max() < tol, (outs[0] - outs[1]).abs().max()


def test_engine_latent_cache_gpu():
    """The engine on the GPU with the compressed latent cache (decode steps replayed from CUDA graphs, chunked
    prefill, several sequences) against the same engine with expanded keys / values."""
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 32000, int(n)).tolist() for n in (90, 7, 33, 150)]
    cfg = {"max_tokens": 12, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    outs = []
    for extra in ("", "&mla_cache=latent"):
        eng = SyncMLCEngine("random://tiny-deepseek-v2?quant=q0f16&seed=0" + extra, "cuda",
                            engine_config=EngineConfig(mode="server", max_num_sequence=8, prefill_chunk_size=64,
                                                       max_total_sequence_length=4096))
        assert eng.runtime.models[0].mla_latent == bool(extra)
        _, toks = eng.generate(prompts, cfg)
        outs.append([t[0] for t in toks])
        del eng
    same = sum(int(a == b) for x, y in zip(*outs) for a, b in zip(x, y))
    assert [x[0] for x in outs[0]] == [y[0] for y in outs[1]] and same >= 0.7 * 48, outs


def test_engine_end_to_end_gpu():
    from mlc_llm_b200.ops import _lib
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

    eng = SyncMLCEngine("random://tiny-llama-gpu?quant=q4f16_1&seed=0", "cuda",
                        engine_config=EngineConfig(mode="server", max_num_sequence=16, prefill_chunk_size=256,
                                                   max_total_sequence_length=4096))
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 32000, int(n)).tolist() for n in rng.integers(5, 120, 12)]
    cfg = {"max_tokens": 16, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    _, toks = eng.generate(prompts, cfg)
    _lib.check_status(torch.device("cuda"))
    assert all(len(t[0]) == 16 for t in toks)
    # continuous batching must not change greedy results: rerun one by one
    for i in (0, 5):
        _, one = eng.generate([prompts[i]], cfg)
        agree = np.mean(np.asarray(one[0][0]) == np.asarray(toks[i][0]))
        assert agree >= 0.75, (i, one[0][0], toks[i][0])
    # sampling path
    _, toks2 = eng.generate(prompts[:4], {"max_tokens": 8, "temperature": 0.8, "top_p": 0.9, "seed": 7,
                                          "logprobs": True, "top_logprobs": 3,
                                          "debug_config": {"ignore_eos": True}})
    assert all(len(t[0]) == 8 for t in toks2)
    stats = json.loads(eng.debug_stats())
    assert stats["num_decode_steps"] > 0 and stats["num_prefill_steps"] > 0


def test_fused_forward_single_rank_with_graphs(monkeypatch):
    """The fused tensor-parallel forward run with one rank (peer tables point at local memory), eagerly
    and replayed from CUDA graphs: its call numbers come from device memory, so replays stay valid.
    Greedy tokens must agree with the plain forward of the same weights."""
    from mlc_llm_b200.ops import _lib
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

    model = "random://tiny-llama-gpu?quant=q4f16_1&seed=3"
    ecfg = dict(mode="server", max_num_sequence=8, prefill_chunk_size=256, max_total_sequence_length=4096)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, 32000, int(n)).tolist() for n in (33, 70, 12, 51)]
    cfg = {"max_tokens": 24, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    monkeypatch.setenv("MLCB_FUSED_TP", "0")
    plain = SyncMLCEngine(model, "cuda", engine_config=EngineConfig(**ecfg))
    _, want = plain.generate(prompts, cfg)
    monkeypatch.setenv("MLCB_FUSED_TP", "1")
    monkeypatch.setenv("MLCB_CUDA_GRAPH", "0")
    eager = SyncMLCEngine(model, "cuda", engine_config=EngineConfig(**ecfg))
    assert eager.runtime.fused_tp and not eager.runtime.executor.use_graphs
    _, got_eager = eager.generate(prompts, cfg)
    monkeypatch.setenv("MLCB_CUDA_GRAPH", "1")
    eng = SyncMLCEngine(model, "cuda", engine_config=EngineConfig(**ecfg))
    assert eng.runtime.fused_tp
    _, got = eng.generate(prompts, cfg)
    _, got2 = eng.generate(prompts, cfg)  # every shape is replayed from its graph this time
    _lib.check_status(torch.device("cuda"))
    assert eng.runtime.executor.graph_replays > 0
    fused = eng.runtime.models[0].fused
    assert int(fused.epoch_dev[0].item()) == fused.base  # host mirror and device word in step

    def agreement(a, b):
        return float(np.mean([np.mean(np.asarray(x[0]) == np.asarray(y[0])) for x, y in zip(a, b)]))

    assert agreement(got, got_eager) >= 0.95 and agreement(got2, got_eager) >= 0.95
    # against the unfused forward: different summation order, so only near agreement
    assert all(a[0][0] == b[0][0] for a, b in zip(got, want))
    assert agreement(got, want) >= 0.6


def test_varying_batch_replays_bucketed_graphs(monkeypatch):
    """A decode batch that loses a sequence every few steps: padded to bucket sizes, nearly every step of a
    second pass is a graph replay, and the tokens equal those of the run without graphs."""
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.executor import graph_bucket
    from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

    assert [graph_bucket(n) for n in (1, 2, 3, 5, 17, 32, 33, 48, 49, 250)] == [1, 2, 4, 8, 32, 32, 48, 48, 64, 256]
    model = "random://tiny-llama-gpu?quant=q4f16_1&seed=5"
    ecfg = dict(mode="server", max_num_sequence=48, prefill_chunk_size=512, max_total_sequence_length=8192)
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, 32000, int(rng.integers(5, 40))).tolist() for _ in range(40)]
    cfgs = [{"max_tokens": 6 + 2 * i, "temperature": 0.0, "debug_config": {"ignore_eos": True}} for i in range(40)]
    monkeypatch.setenv("MLCB_CUDA_GRAPH", "0")
    plain = SyncMLCEngine(model, "cuda", engine_config=EngineConfig(**ecfg))
    _, want = plain.generate(prompts, cfgs)
    monkeypatch.setenv("MLCB_CUDA_GRAPH", "1")
    eng = SyncMLCEngine(model, "cuda", engine_config=EngineConfig(**ecfg))
    _, first = eng.generate(prompts, cfgs)
    ex = eng.runtime.executor
    steps0, replays0 = ex.graph_eligible_steps, ex.graph_replays
    _, got = eng.generate(prompts, cfgs)
    steps, replays = ex.graph_eligible_steps - steps0, ex.graph_replays - replays0
    assert steps >= 60 and replays >= 0.95 * steps, (steps, replays)
    # padded batches take other kernel variants (tile widths, split-K) than exact ones: near agreement

    def agreement(x, y):
        return float(np.mean([np.mean(np.asarray(p[0]) == np.asarray(q[0])) for p, q in zip(x, y)]))

    assert agreement(first, want) >= 0.9 and agreement(got, want) >= 0.9
    assert all(a[0][0] == b[0][0] for a, b in zip(got, want))


def _tokens(model, device, prompts, cfg, **engine_kw):
    from mlc_llm_b200.serve.config import EngineConfig
    from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

    ecfg = dict(mode="server", max_num_sequence=8, prefill_chunk_size=128, max_total_sequence_length=4096,
                prefix_cache_mode="disable")
    ecfg.update(engine_kw)
    eng = SyncMLCEngine(model, device, engine_config=EngineConfig(**ecfg))
    _, toks = eng.generate(prompts, cfg)
    return [t[0] for t in toks], eng


def _agreement(a, b):
    return float(np.mean([np.mean(np.asarray(x) == np.asarray(y)) for x, y in zip(a, b)]))


@pytest.mark.parametrize("case", ["gemma2", "window_sink"])
def test_masked_attention_models_match_the_cpu_engine(case, monkeypatch):
    """Per-layer sliding windows with logit soft-capping (gemma2) and an engine-wide window with attention
    sinks run on the tensor-core attention kernel's masked variant; greedy tokens against the CPU engine
    holding the same weights. Prompts are longer than the window and cross prefill chunks."""
    from mlc_llm_b200.ops import _lib

    monkeypatch.setenv("MLCB_RANDOM_INIT_DEVICE", "cpu")
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, 32000, int(n)).tolist() for n in (150, 40, 97, 260)]
    cfg = {"max_tokens": 12, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    if case == "gemma2":
        model, kw = "random://tiny-gemma2-gpu?quant=q0f16&seed=4", {}
    else:
        model, kw = "random://tiny-llama-gpu?quant=q0f16&seed=4", dict(sliding_window_size=64, attention_sink_size=4)
    lib = _lib.lib()
    lib.mlcb_launch_count.restype = __import__("ctypes").c_longlong
    got, eng = _tokens(model, "cuda", prompts, cfg, **kw)
    _lib.check_status(torch.device("cuda"))
    assert eng.runtime.executor._tc_attention_ok(eng.runtime.models[0])  # not the CUDA-core fallback
    want, _ = _tokens(model, "cpu", prompts, cfg, **kw)
    assert all(a[0] == b[0] for a, b in zip(got, want))
    assert _agreement(got, want) >= 0.85, (got, want)


def test_speculative_decoding_on_the_gpu_keeps_greedy_outputs():
    """Draft-and-verify with a small draft model: the verify step's token trees go through the tensor-core
    attention kernel's tree mask; greedy outputs equal plain greedy decoding up to near-ties."""
    from mlc_llm_b200.ops import _lib

    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, 32000, int(n)).tolist() for n in (33, 70, 12, 129)]
    cfg = {"max_tokens": 24, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    model = "random://tiny-llama-gpu?quant=q0f16&seed=3"
    want, _ = _tokens(model, "cuda", prompts, cfg)
    for mode_kw in (dict(spec_draft_length=3), dict(spec_draft_length=4, spec_tree_width=2)):
        got, eng = _tokens(model, "cuda", prompts, cfg, speculative_mode="small_draft",
                           additional_models=["random://tiny-llama-gpu?quant=q0f16&seed=3"], **mode_kw)
        _lib.check_status(torch.device("cuda"))
        stats = json.loads(eng.debug_stats()) if hasattr(eng, "debug_stats") else {}
        assert all(len(t) == 24 for t in got)
        assert all(a[0] == b[0] for a, b in zip(got, want))
        # the draft is the target itself, so nearly every proposal is accepted and outputs agree
        assert _agreement(got, want) >= 0.9, (mode_kw, got, want, stats)


def test_smoke_entry():
    import __graft_entry__ as g

    g.smoke()


def test_bert_encoder_on_the_gpu_matches_the_cpu():
    """BERT on the GPU (encoder-attention, LayerNorm and GELU kernels, fp16) against the fp32 CPU model with the
    same weights, on a right-padded batch."""
    from mlc_llm_b200.models.bert import BertConfig, BertModel, hf_names

    torch.manual_seed(21)
    cfg = BertConfig(vocab_size=1000, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                     intermediate_size=512, max_position_embeddings=128)
    shapes = {"embed.word": (1000, 256), "embed.position": (128, 256), "embed.token_type": (2, 256)}
    tensors = {}
    for name, _ in hf_names(cfg):
        if name in shapes:
            tensors[name] = torch.randn(*shapes[name]) * 0.05
        elif name.endswith("ln.weight"):
            tensors[name] = torch.rand(256) + 0.5
        elif name.endswith("ln.bias"):
            tensors[name] = torch.randn(256) * 0.05
        elif name.endswith(".weight"):
            out_in = {"qkv": (768, 256), "attn_out": (256, 256), "up": (512, 256), "down": (256, 512)}
            tensors[name] = torch.randn(*out_in[name.split(".")[-2]]) * 0.05
        else:
            width = {"qkv": 768, "attn_out": 256, "up": 512, "down": 256}[name.split(".")[-2]]
            tensors[name] = torch.randn(width) * 0.02
    ids = torch.randint(0, 1000, (3, 70))
    mask = torch.ones(3, 70, dtype=torch.long)
    mask[1, 40:] = 0
    mask[2, 9:] = 0
    want = BertModel(cfg, tensors, torch.device("cpu")).forward(ids, mask)
    got = BertModel(cfg, tensors, torch.device("cuda")).forward(ids.cuda(), mask.cuda()).float().cpu()
    valid = mask.bool()
    assert (got[valid] - want[valid]).abs().max() < 3e-2, (got[valid] - want[valid]).abs().max()
