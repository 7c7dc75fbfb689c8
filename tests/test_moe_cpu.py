"""MoE block on CPU against a direct per-token evaluation."""
import torch

from mlc_llm_b200 import ops
from mlc_llm_b200.ops import reference as ref


def test_permute_combine_match_direct():
    torch.manual_seed(0)
    t, e, k, h, inter = 23, 4, 2, 32, 48
    x = torch.randn(t, h)
    gate = torch.randn(t, e)
    w13 = torch.randn(e, 2 * inter, h) * 0.1
    w2 = torch.randn(e, h, inter) * 0.1
    wts, idx = ops.moe_router(gate, k, True)
    off, spos, src = ops.moe_permute(idx, e)
    xp = ops.row_gather(x, src)
    l13 = ops.LinearWeight("dense", w13, None, None, None, 2 * inter, h)
    l2 = ops.LinearWeight("dense", w2, None, None, None, h, inter)
    y = ops.grouped_linear(ops.act_mul(ops.grouped_linear(xp, l13, off)), l2, off)
    out = ops.moe_combine(y, wts, spos, None)
    direct = ref.moe_ffn(x, w13, w2, wts, idx)
    assert torch.allclose(out, direct, atol=1e-4)
    # routing equals "top-k of the logits then softmax over the k"
    w2_, i2_ = ref.moe_topk_softmax(gate, k)
    assert torch.equal(i2_, idx) and torch.allclose(w2_, wts, atol=1e-6)


def test_group_limited_router_keeps_experts_of_the_best_groups():
    """DeepSeek-V2 routing: only experts inside the ``topk_group`` best groups (by their best single
    softmax score) can be chosen; weights are the unnormalised softmax scores."""
    import torch

    from mlc_llm_b200.models.moe import _group_limited_router

    torch.manual_seed(0)
    t, e, groups, keep, k = 9, 16, 4, 2, 3
    logits = torch.randn(t, e)
    w, idx = _group_limited_router(logits, k, groups, keep, renorm=False)
    probs = torch.softmax(logits, -1)
    for r in range(t):
        best = probs[r].view(groups, -1).max(-1).values
        allowed_groups = set(torch.topk(best, keep).indices.tolist())
        allowed = [j for j in range(e) if j // (e // groups) in allowed_groups]
        want = sorted(allowed, key=lambda j: -float(probs[r, j]))[:k]
        assert sorted(idx[r].tolist()) == sorted(want)
        for slot in range(k):
            assert abs(float(w[r, slot]) - float(probs[r, int(idx[r, slot])])) < 1e-6
    w2, _ = _group_limited_router(logits, k, groups, keep, renorm=True)
    assert torch.allclose(w2.sum(-1), torch.ones(t), atol=1e-6)
