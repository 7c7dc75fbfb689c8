"""EAGLE and Medusa speculative modes on CPU: greedy output equals plain decoding, and the draft heads
are fed the target model's true features of the right positions."""
import numpy as np
import pytest
import torch

from mlc_llm_b200.serve.config import EngineConfig
from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

MODEL = "random://tiny-llama?quant=q0f32&seed=11"
HEADS = {"eagle": "random://tiny-eagle?quant=q0f32&seed=3", "medusa": "random://tiny-medusa?quant=q0f32&seed=4"}
GREEDY = {"temperature": 0.0, "debug_config": {"ignore_eos": True}, "max_tokens": 10}


def _engine(mode=None, chunk=32):
    kw = dict(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=chunk,
              prefix_cache_mode="disable")
    if mode:
        kw.update(speculative_mode=mode, spec_draft_length=3, additional_models=[HEADS[mode]])
    return SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(**kw))


def _prompts(n, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(10, 31000, int(rng.integers(20, 60))).tolist() for _ in range(n)]


def _reference_features(tokens):
    """Final-normed hidden states of every position of ``tokens``, from one plain prefill pass."""
    eng = _engine(chunk=256)
    model = eng.runtime.models[0]
    seen = []
    orig = model.logits

    def logits(hidden, rows):
        seen.append(model.final_features(hidden).detach().clone())
        return orig(hidden, rows)

    model.logits = logits
    eng.generate([tokens], dict(GREEDY, max_tokens=1))
    return seen[0]


@pytest.mark.parametrize("mode", ["eagle", "medusa"])
def test_greedy_output_equals_plain_decoding(mode):
    prompts = _prompts(4)
    _, want = _engine().generate(prompts, GREEDY)
    eng = _engine(mode)
    _, got = eng.generate(prompts, GREEDY)
    assert [t[0] for t in got] == [t[0] for t in want]
    import json

    stats = json.loads(eng.debug_stats())
    assert stats["num_verify_steps"] > 0 and stats["num_running"] == 0


def test_eagle_head_reads_true_features_of_the_previous_position():
    prompt = _prompts(1, seed=5)[0][:45] + _prompts(1, seed=6)[0][:5]   # > one prefill chunk of 32
    eng = _engine("eagle")
    ex = eng.runtime.executor
    head = eng.runtime.models[1]
    events = []
    orig_fuse, orig_head, orig_verify = head.fuse_embed_hidden, ex._forward_spec_head, ex.forward_verify

    def fuse(embed, feats):
        events[-1]["prev"] = feats.detach().clone()
        return orig_fuse(embed, feats)

    def spec_head(model_id, plan, dev, n_rows):
        events.append({"kind": "head", "pos": np.asarray(plan["positions"]).copy(), "sampling": n_rows > 0})
        return orig_head(model_id, plan, dev, n_rows)

    def verify(*a, **k):
        events.append({"kind": "verify"})
        return orig_verify(*a, **k)

    head.fuse_embed_hidden, ex._forward_spec_head, ex.forward_verify = fuse, spec_head, verify
    _, toks = eng.generate([prompt], GREEDY)
    full = prompt + toks[0][0]
    ref = _reference_features(full[:-1] + [1])[: len(full) - 1]
    checked_prefill = checked_round0 = 0
    prev_kind = "start"
    for ev in events:
        if ev["kind"] == "head":
            first_after_target_pass = prev_kind in ("start", "verify", "prefill")
            if not ev["sampling"] or first_after_target_pass:
                # prefill of the head, or the first draft round after a target pass: every row pairs its
                # token with the target's feature of the position before it (zeros before position 0)
                for row, p in enumerate(ev["pos"].tolist()):
                    want = ref[p - 1] if p > 0 else torch.zeros_like(ref[0])
                    assert torch.allclose(ev["prev"][row], want, atol=2e-4), (p, ev["sampling"])
                    if ev["sampling"]:
                        checked_round0 += 1
                    else:
                        checked_prefill += 1
            prev_kind = "head" if ev["sampling"] else "prefill"
        else:
            prev_kind = "verify"
    assert checked_prefill >= len(prompt) and checked_round0 >= 3


def test_medusa_round_r_uses_head_r_on_the_newest_true_feature():
    prompt = _prompts(1, seed=7)[0][:40]
    eng = _engine("medusa")
    ex = eng.runtime.executor
    head = eng.runtime.models[1]
    events = []
    orig_logits, orig_head, orig_verify = head.medusa_logits, ex._forward_spec_head, ex.forward_verify

    def medusa_logits(feats, which):
        events[-1].update(feats=feats.detach().clone(), head=which)
        return orig_logits(feats, which)

    def spec_head(model_id, plan, dev, n_rows):
        if n_rows:
            events.append({"kind": "head", "last_pos": int(np.asarray(plan["positions"])[-1])})
        return orig_head(model_id, plan, dev, n_rows)

    def verify(*a, **k):
        events.append({"kind": "verify"})
        return orig_verify(*a, **k)

    head.medusa_logits, ex._forward_spec_head, ex.forward_verify = medusa_logits, spec_head, verify
    _, toks = eng.generate([prompt], GREEDY)
    full = prompt + toks[0][0]
    ref = _reference_features(full[:-1] + [1])[: len(full) - 1]
    rnd, base, n = 0, None, 0
    for ev in events:
        if ev["kind"] == "verify":
            rnd = 0
            continue
        if rnd == 0:
            base = ev["last_pos"]  # position of the last committed token
        assert ev["head"] == rnd and ev["last_pos"] == base + rnd
        assert torch.allclose(ev["feats"][0], ref[base - 1], atol=2e-4)
        rnd += 1
        n += 1
    assert n >= 6


def test_eagle_and_medusa_checkpoints_load_from_huggingface_names(tmp_path):
    from safetensors.torch import save_file

    from mlc_llm_b200 import quantization as Q
    from mlc_llm_b200.models import config as mc
    from mlc_llm_b200.models import loader
    from mlc_llm_b200.models.presets import MODEL_PRESETS

    g = torch.Generator().manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, generator=g) * 0.05
    # ---- EAGLE: tensors without the "model." prefix, separate q / k / v and gate / up, fc with bias
    cfg = mc.from_dict("eagle", dict(MODEL_PRESETS["tiny-eagle"]))
    h, d, hq, hkv, inter = 256, 64, 4, 2, 688
    sd = {"embed_tokens.weight": rnd(32000, h), "fc.weight": rnd(h, 2 * h), "fc.bias": rnd(h),
          "layers.0.self_attn.q_proj.weight": rnd(hq * d, h), "layers.0.self_attn.k_proj.weight": rnd(hkv * d, h),
          "layers.0.self_attn.v_proj.weight": rnd(hkv * d, h), "layers.0.self_attn.o_proj.weight": rnd(h, hq * d),
          "layers.0.mlp.gate_proj.weight": rnd(inter, h), "layers.0.mlp.up_proj.weight": rnd(inter, h),
          "layers.0.mlp.down_proj.weight": rnd(h, inter), "layers.0.post_attention_layernorm.weight": rnd(h)}
    (tmp_path / "eagle").mkdir()
    save_file(sd, str(tmp_path / "eagle" / "model.safetensors"))
    store = loader.load_hf_params(str(tmp_path / "eagle"), cfg, Q.get("q0f32"), torch.device("cpu"))
    assert torch.equal(store.linears["model.fc"].w, sd["fc.weight"])
    assert torch.equal(store.linears["model.fc"].bias, sd["fc.bias"])
    qkv = torch.cat([sd[f"layers.0.self_attn.{n}_proj.weight"] for n in "qkv"])
    assert torch.equal(store.linears["model.layers.0.self_attn.qkv_proj"].w, qkv)
    assert "model.layers.0.input_layernorm.weight" not in store.tensors  # the first block has none
    # ---- Medusa: names are kept
    mcfg = mc.from_dict("medusa", dict(MODEL_PRESETS["tiny-medusa"]))
    msd = {}
    for i in range(3):
        msd[f"medusa_head.{i}.0.linear.weight"] = rnd(h, h)
        msd[f"medusa_head.{i}.0.linear.bias"] = rnd(h)
        msd[f"medusa_head.{i}.1.weight"] = rnd(32000, h)
    (tmp_path / "medusa").mkdir()
    save_file(msd, str(tmp_path / "medusa" / "model.safetensors"))
    mstore = loader.load_hf_params(str(tmp_path / "medusa"), mcfg, Q.get("q0f32"), torch.device("cpu"))
    assert torch.equal(mstore.linears["medusa_head.2.1"].w, msd["medusa_head.2.1.weight"])
    assert torch.equal(mstore.linears["medusa_head.1.0.linear"].bias, msd["medusa_head.1.0.linear.bias"])


def _tree_engine(mode, width):
    kw = dict(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=32,
              prefix_cache_mode="disable", speculative_mode=mode, spec_draft_length=3, spec_tree_width=width,
              additional_models=[HEADS[mode]])
    return SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(**kw))


@pytest.mark.parametrize("mode", ["eagle", "medusa"])
def test_draft_trees_keep_the_greedy_output(mode):
    """``spec_tree_width = 2``: every round gives each leaf two children (14 nodes after three rounds); the
    verified output is still the plain greedy output."""
    prompts = _prompts(3, seed=3)
    _, want = _engine().generate(prompts, GREEDY)
    eng = _tree_engine(mode, 2)
    _, got = eng.generate(prompts, GREEDY)
    assert [t[0] for t in got] == [t[0] for t in want]
    import json

    stats = json.loads(eng.debug_stats())
    assert stats["num_verify_steps"] > 0 and stats["num_running"] == 0


def test_medusa_tree_accepts_a_second_choice_that_a_chain_misses():
    """Heads whose best guess is always wrong and whose second guess is always right: a chain accepts nothing,
    a tree of width two accepts every level, so it needs far fewer verification steps. Both under greedy
    sampling (the draft's sampling distribution is one-hot there: children are ranked by the plain softmax) and
    at a low temperature."""
    import json

    prompt = _prompts(1, seed=5)[0]
    _, plain = _engine().generate([prompt], dict(GREEDY, max_tokens=16))
    full = prompt + plain[0][0]

    def rigged(eng):
        head, ex = eng.runtime.models[1], eng.runtime.executor
        orig = ex._forward_spec_head
        state = {}

        def spec_head(model_id, plan, dev, n_rows):
            # the newest committed token's position tells which tokens come next
            state["last"] = int(np.asarray(plan["positions"])[int(np.asarray(plan["q_indptr"])[1]) - 1])
            return orig(model_id, plan, dev, n_rows)

        def medusa_logits(feats, which):
            lg = torch.full((feats.shape[0], head.cfg.vocab_size), -10.0)
            # called for draft round `which`: the chunk's last token sits `which` levels below the newest
            # committed token, so the token this head should predict is at position last + 1
            nxt = state["last"] + 1
            right = full[nxt] if nxt < len(full) else 0
            lg[:, (right + 1) % head.cfg.vocab_size] = 5.0   # best guess: wrong
            lg[:, right] = 4.995                              # second guess: right (0.7 % at this temperature)
            return lg

        ex._forward_spec_head, head.medusa_logits = spec_head, medusa_logits

    for temperature in (0.0, 1e-3):
        steps = {}
        for width in (1, 2):
            eng = _tree_engine("medusa", width)
            rigged(eng)
            _, got = eng.generate([prompt], dict(GREEDY, max_tokens=16, temperature=temperature, seed=7))
            if temperature == 0.0:
                assert got[0][0] == plain[0][0]
            else:
                assert got[0][0][:4] == plain[0][0][:4]  # peaked distributions: sampling follows the arg-max
            steps[width] = json.loads(eng.debug_stats())["num_verify_steps"]
        assert steps[2] * 2 <= steps[1], (temperature, steps)


def test_eagle_tree_nodes_continue_from_their_parents_output():
    """In every tree round a node is fused with the head's output for its parent from the round before (children
    of the root: with the head's output at the last committed token)."""
    eng = _tree_engine("eagle", 2)
    head, ex = eng.runtime.models[1], eng.runtime.executor
    calls = []
    orig_fuse, orig_forward, orig_spec = head.fuse_embed_hidden, head.forward, ex._forward_spec_head

    def spec_head(model_id, plan, dev, n_rows):
        calls.append({"mask": [int(m) for m in np.asarray(plan["tree_mask"]).astype(np.uint64).tolist()],
                      "qi": np.asarray(plan["q_indptr"]).tolist()})
        return orig_spec(model_id, plan, dev, n_rows)

    def fuse(x, prev):
        calls[-1]["prev"] = prev.detach().clone()
        return orig_fuse(x, prev)

    def forward(x, b):
        h = orig_forward(x, b)
        calls[-1]["h"] = h.detach().clone()
        return h

    ex._forward_spec_head, head.fuse_embed_hidden, head.forward = spec_head, fuse, forward
    eng.generate(_prompts(1, seed=9), dict(GREEDY, max_tokens=6))
    checked = 0
    for at in range(1, len(calls)):
        before, cur = calls[at - 1], calls[at]
        if not cur["mask"]:
            continue
        n = len(cur["mask"])
        for j, m in enumerate(cur["mask"]):
            parent = (m & ((1 << j) - 1)).bit_length() - 1
            if parent < 0:
                # the newest chain call before this draft phase's tree rounds ended at the last committed token
                root = next(c for c in reversed(calls[:at]) if not c["mask"])
                assert torch.equal(cur["prev"][j], root["h"][-1])
            else:
                assert before["mask"] and parent < len(before["mask"])
                assert torch.equal(cur["prev"][j], before["h"][parent])
            checked += 1
        assert n in (2, 6)  # levels of two and of two + four nodes are fed
    assert checked >= 8


def test_parallel_samples_inherit_the_target_features():
    """``n = 2`` with an EAGLE head: a sample forks from the prompt's sequence, and the head's first call for it
    must see the target's true features of the prompt (carried over with the fork), not zeros."""
    eng = _engine("eagle")
    head, ex = eng.runtime.models[1], eng.runtime.executor
    seen = []
    orig_fuse, orig_spec = head.fuse_embed_hidden, ex._forward_spec_head

    def spec_head(model_id, plan, dev, n_rows):
        seen.append({"ids": [int(s) for s in np.asarray(plan["seq_ids"]).tolist()],
                     "qi": np.asarray(plan["q_indptr"]).tolist(), "pos": np.asarray(plan["positions"]).tolist()})
        return orig_spec(model_id, plan, dev, n_rows)

    def fuse(x, prev):
        seen[-1]["prev"] = prev.detach().clone()
        return orig_fuse(x, prev)

    ex._forward_spec_head, head.fuse_embed_hidden = spec_head, fuse
    prompt = _prompts(1, seed=12)[0]
    _, plain = _engine().generate([prompt], GREEDY)
    _, got = eng.generate([prompt], dict(GREEDY, n=2))
    assert got[0] == [plain[0][0], plain[0][0]]
    parent = seen[0]["ids"][0]
    first_child_call = next(c for c in seen if parent not in c["ids"])
    assert len(first_child_call["ids"]) == 2
    for i in range(2):
        a, b = first_child_call["qi"][i], first_child_call["qi"][i + 1]
        rows = first_child_call["prev"][a:b]
        assert b > a and bool((rows.abs().sum(dim=-1) > 0).all()), "a sample's first draft call saw zero features"


@pytest.mark.parametrize("spec", [dict(speculative_mode="small_draft", spec_draft_length=3,
                                       additional_models=["random://tiny-llama?quant=q0f32&seed=2"]),
                                  dict(speculative_mode="small_draft", spec_draft_length=2, spec_tree_width=2,
                                       additional_models=["random://tiny-llama?quant=q0f32&seed=2"]),
                                  dict(speculative_mode="eagle", spec_draft_length=2,
                                       additional_models=[HEADS["eagle"]])])
def test_json_mode_under_speculative_decoding_equals_plain_json_mode(spec):
    """A schema-constrained request verified over draft tokens: the row after a draft node must be masked with the
    grammar state after that node's path (and penalised with its tokens), not with the state of the last
    committed token; a draft token outside the grammar is never accepted. Output equals plain constrained
    decoding, for one sample and for two."""
    import json

    schema = json.dumps({"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}},
                         "required": ["name", "age"]})
    gen = {"temperature": 0.0, "max_tokens": 30, "repetition_penalty": 1.1,
           "response_format": {"type": "json_object", "schema": schema}}
    prompts = _prompts(3, seed=21)
    _, want = _engine().generate(prompts, gen)
    kw = dict(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=32,
              prefix_cache_mode="disable", **spec)
    eng = SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(**kw))
    _, got = eng.generate(prompts, gen)
    assert [g[0] for g in got] == [w[0] for w in want]
    assert json.loads(eng.debug_stats())["num_verify_steps"] > 0
    _, two = eng.generate(prompts[:1], dict(gen, n=2))
    assert two[0] == [want[0][0], want[0][0]]


def test_chosen_tree_children_keep_the_target_distribution():
    """Draft-tree children are the draft's best tokens, chosen rather than drawn, so they are verified against
    point-mass draft rows: accept with probability p(token), otherwise drop the token from p. Over many draws
    the token that ends up at the first position is distributed as the target's p (with the min(1, p / q) rule
    and q = p, the best token would be taken every time)."""
    from mlc_llm_b200 import ops

    torch.manual_seed(0)
    p = torch.tensor([0.05, 0.4, 0.25, 0.2, 0.1])
    n = 6000
    children = [1, 2]                                   # the two best tokens
    rows = 3 * n
    model = p.repeat(rows, 1).clone()
    draft_tok = torch.zeros(rows, dtype=torch.int32)
    first_child = torch.full((rows,), -1, dtype=torch.int32)
    next_sibling = torch.full((rows,), -1, dtype=torch.int32)
    roots = torch.arange(n, dtype=torch.int32) * 3
    first_child[roots.long()] = roots + 1
    next_sibling[(roots + 1).long()] = roots + 2
    draft_tok[(roots + 1).long()], draft_tok[(roots + 2).long()] = children[0], children[1]
    draft = torch.zeros(rows, 5)
    draft.scatter_(1, draft_tok.long().unsqueeze(1), 1.0)
    uniform = torch.rand(rows)
    parent = roots.clone()
    ops.verify_tree(draft, draft_tok, model, first_child, next_sibling, uniform, parent)
    final, _ = ops.sample(model, parent, torch.rand(n), torch.ones(n), None)
    out = torch.where(parent == roots, final.to(torch.int64), draft_tok[parent.long()].to(torch.int64))
    freq = torch.bincount(out, minlength=5).float() / n
    assert torch.allclose(freq, p, atol=0.025), freq


def test_tree_verification_in_the_engine_does_not_collapse_to_the_best_token():
    """A draft model with the target's weights and a tree of width two at temperature one: with point-mass draft
    rows a chosen child is accepted with the (small) probability the target gives it; with the drawn-candidate
    rule it would be accepted every time and sampling would turn into arg-max decoding."""
    prompt = _prompts(1, seed=31)[0]
    kw = dict(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=64,
              prefix_cache_mode="disable", speculative_mode="small_draft", spec_draft_length=2, spec_tree_width=2,
              additional_models=[MODEL])
    eng = SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(**kw))
    plain = _engine()
    same = 0
    for seed in range(24):
        # the first token is drawn after the prefill; the second comes out of a verification of the tree under it
        _, toks = eng.generate([prompt], {"temperature": 1.0, "seed": seed, "max_tokens": 2,
                                          "debug_config": {"ignore_eos": True}})
        first, second = toks[0][0]
        _, best = plain.generate([prompt + [first]], dict(GREEDY, max_tokens=1))
        same += int(second == best[0][0][0])
    assert same <= 8, same


@pytest.mark.parametrize("spec", [dict(spec_draft_length=3), dict(spec_draft_length=2, spec_tree_width=2)])
def test_top_k_applies_to_the_verified_distribution(spec):
    """``top_k = 1`` at temperature one leaves a single token per position, so sampling is arg-max decoding; the
    verification of draft tokens must see that truncated distribution too."""
    prompts = _prompts(3, seed=41)
    _, want = _engine().generate(prompts, dict(GREEDY, max_tokens=10))
    kw = dict(mode="server", max_num_sequence=8, max_total_sequence_length=2048, prefill_chunk_size=32,
              prefix_cache_mode="disable", speculative_mode="small_draft",
              additional_models=["random://tiny-llama?quant=q0f32&seed=2"], **spec)
    eng = SyncMLCEngine(MODEL, "cpu", engine_config=EngineConfig(**kw))
    _, got = eng.generate(prompts, {"temperature": 1.0, "top_k": 1, "seed": 9, "max_tokens": 10,
                                    "debug_config": {"ignore_eos": True}})
    assert [t[0] for t in got] == [t[0] for t in want]


@pytest.mark.parametrize("spec", [dict(speculative_mode="small_draft", spec_draft_length=3,
                                       additional_models=[MODEL]),                    # everything accepted
                                  dict(speculative_mode="small_draft", spec_draft_length=3,
                                       additional_models=["random://tiny-llama?quant=q0f32&seed=2"]),
                                  dict(speculative_mode="small_draft", spec_draft_length=2, spec_tree_width=2,
                                       additional_models=[MODEL])])
def test_logprobs_under_speculative_decoding_are_the_targets(spec):
    """The probability and the best alternatives reported for a committed token are the target model's, whether
    the token was proposed by a draft and accepted, or sampled after the accepted path: equal to plain decoding."""
    from mlc_llm_b200.serve.engine import MLCEngine

    prompt = _prompts(1, seed=51)[0]
    kw = dict(mode="server", max_num_sequence=4, max_total_sequence_length=1024, prefill_chunk_size=64,
              prefix_cache_mode="disable")
    req = dict(prompt=prompt, max_tokens=9, temperature=0.0, logprobs=True, top_logprobs=3,
               debug_config={"ignore_eos": True})
    plain = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**kw))
    eng = MLCEngine(MODEL, "cpu", engine_config=EngineConfig(**kw, **spec))
    try:
        want = plain.completions.create(**req).choices[0].logprobs.content
        got = eng.completions.create(**req).choices[0].logprobs.content
    finally:
        plain.terminate()
        eng.terminate()
    assert [c.token for c in got] == [c.token for c in want]
    for g, w in zip(got, want):
        assert abs(g.logprob - w.logprob) < 1e-3
        assert [t.token for t in g.top_logprobs] == [t.token for t in w.top_logprobs]
        assert all(abs(a.logprob - b.logprob) < 1e-3 for a, b in zip(g.top_logprobs, w.top_logprobs))
