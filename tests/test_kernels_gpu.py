"""CUDA kernels against the fp32 PyTorch oracle (``ops.reference``)."""
import math

import numpy as np

import pytest
import torch

from mlc_llm_b200 import ops, quantization as Q
from mlc_llm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, rtol, atol):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g}, worst tol {tol.min().item():.4g}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (16, 256, 256), (100, 384, 512), (256, 512, 4096),
                                   (300, 1376, 256), (1000, 640, 704), (513, 128, 128)])
def test_gemm_dense(dtype, m, n, k):
    torch.manual_seed(0)
    x = (torch.randn(m, k) * 0.5).to(dtype).to(DEV)
    w = (torch.randn(n, k) * 0.05).to(dtype).to(DEV)
    y = ops.linear(x, ops.dense_weight(w))
    ops.check_status(x.device)
    yr = ref.linear_dense(x.cpu(), w.cpu())
    _close(y, yr, 2e-2, 2e-2)


def test_gemm_dense_bias_fp32_out():
    torch.manual_seed(1)
    x = (torch.randn(40, 256) * 0.5).half().to(DEV)
    w = (torch.randn(384, 256) * 0.05).half().to(DEV)
    b = torch.randn(384).half().to(DEV)
    y = ops.linear(x, ops.dense_weight(w, b), out_dtype=torch.float32)
    ops.check_status(x.device)
    assert y.dtype == torch.float32
    _close(y, ref.linear_dense(x.cpu(), w.cpu(), b.cpu(), torch.float32), 1e-2, 1e-2)


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (7, 256, 128), (64, 512, 4096), (256, 384, 1024),
                                   (600, 1376, 256), (24, 256, 688)])  # 688: groups padded, dequantised cold path
def test_gemm_q4f16(m, n, k):
    torch.manual_seed(2)
    quant = Q.get("q4f16_1")
    w = (torch.randn(n, k) * 0.02).half()
    qw, qs = Q.group_quantize(w, quant)
    lw = ops.LinearWeight("q4", qw, qs, None, quant, n, k).to(DEV)
    x = (torch.randn(m, k) * 0.5).half().to(DEV)
    y = ops.linear(x, lw)
    ops.check_status(x.device)
    wd = Q.group_dequantize(qw, qs, quant, k=k)
    yr = ref.linear_dense(x.cpu(), wd)
    _close(y, yr, 2e-2, 2e-2)


@pytest.mark.parametrize("m,n,k", [(7, 256, 128), (64, 512, 4096), (600, 1376, 256)])
def test_gemm_q4bf16(m, n, k):
    """bf16 models with int4 group weights (q4bf16_1): bf16 scales in the tile records, bf16 activations."""
    torch.manual_seed(2)
    quant = Q.get("q4bf16_1")
    w = (torch.randn(n, k) * 0.02).bfloat16()
    qw, qs = Q.group_quantize(w, quant)
    assert qs.dtype == torch.bfloat16
    lw = ops.LinearWeight("q4", qw, qs, None, quant, n, k).to(DEV)
    assert lw.q4_tileable(k)
    x = (torch.randn(m, k) * 0.5).bfloat16().to(DEV)
    y = ops.linear(x, lw)
    ops.check_status(x.device)
    assert y.dtype == torch.bfloat16
    wd = Q.group_dequantize(qw, qs, quant, k=k)
    yr = ref.linear_dense(x.cpu(), wd)
    _close(y, yr, 3e-2, 3e-2)


def test_q4_device_layout_roundtrip():
    qw = torch.randint(-2**31, 2**31 - 1, (64, 32), dtype=torch.int64).to(torch.int32)
    assert torch.equal(Q.from_device_layout_q4(Q.to_device_layout_q4(qw)), qw)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hidden", [256, 4096, 8192])
def test_rmsnorm_and_add(dtype, hidden):
    torch.manual_seed(3)
    x = torch.randn(37, hidden).to(dtype).to(DEV)
    r = torch.randn(37, hidden).to(dtype).to(DEV)
    w = (1 + 0.1 * torch.randn(hidden)).to(dtype).to(DEV)
    _close(ops.rmsnorm(x, w, 1e-5), ref.rmsnorm(x.cpu(), w.cpu(), 1e-5), 1e-2, 1e-2)
    r_ref = r.cpu().clone()
    out_ref = ref.add_rmsnorm(x.cpu(), r_ref, w.cpu(), 1e-5)
    out = ops.add_rmsnorm(x, r, w, 1e-5)
    _close(out, out_ref, 1e-2, 1e-2)
    assert torch.equal(r.cpu(), r_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_act_mul(dtype):
    x = torch.randn(33, 2 * 1376).to(dtype).to(DEV)
    _close(ops.act_mul(x), ref.act_mul(x.cpu()), 1e-2, 1e-2)
    _close(ops.act_mul(x, "gelu"), ref.act_mul(x.cpu(), "gelu"), 1e-2, 1e-2)


def _mk_paged(nseq, lens, hkv, d, page, dtype):
    npages = sum((l + page - 1) // page for l in lens) + 3
    perm = torch.randperm(npages)
    indptr, indices, c = [0], [], 0
    for l in lens:
        n = (l + page - 1) // page
        indices += perm[c:c + n].tolist()
        c += n
        indptr.append(len(indices))
    kv = (torch.randn(npages, 2, hkv, page, d) * 0.5).to(dtype)
    return kv, torch.tensor(indptr, dtype=torch.int32), torch.tensor(indices, dtype=torch.int32)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rope_append(dtype):
    torch.manual_seed(4)
    hq, hkv, d, page = 8, 2, 128, 16
    t = 19
    qkv = torch.randn(t, (hq + 2 * hkv) * d).to(dtype)
    kv = torch.zeros(6, 2, hkv, page, d, dtype=dtype)
    pos = torch.randint(0, 5000, (t,), dtype=torch.int32)
    slot = torch.randperm(6 * page)[:t].to(torch.int32)
    slot[3] = -1
    inv = ref.rope_inv_freq(d, 500000.0)
    q_ref, kv_ref = qkv.clone(), kv.clone()
    ref.rope_append(q_ref, kv_ref, pos, slot, inv, hq, hkv, d, d, page)
    qg, kvg = qkv.to(DEV), kv.to(DEV)
    ops.rope_append(qg, kvg, pos.to(DEV), slot.to(DEV), inv.to(DEV), hq, hkv, d, d, page)
    _close(qg[:, : (hq + hkv) * d], q_ref[:, : (hq + hkv) * d], 2e-2, 2e-2)
    _close(kvg, kv_ref, 2e-2, 2e-2)


@pytest.mark.parametrize("d", [64, 128])
def test_attention_simt(d):
    torch.manual_seed(5)
    hq, hkv, page = 8, 2, 16
    lens = [5, 33, 16, 70]
    kv, indptr, indices = _mk_paged(len(lens), lens, hkv, d, page, torch.float16)
    q_seq, q_kvlen = [], []
    for b, l in enumerate(lens):
        nq = min(l, 3)
        for i in range(nq):
            q_seq.append(b)
            q_kvlen.append(l - nq + i + 1)
    t = len(q_seq)
    q = (torch.randn(t, hq * d) * 0.5).half()
    q_seq = torch.tensor(q_seq, dtype=torch.int32)
    q_kvlen = torch.tensor(q_kvlen, dtype=torch.int32)
    o_ref = ops.paged_attention(q, kv, q_seq, q_kvlen, indptr, indices, hq, hkv, d, page, d ** -0.5)
    o = ops.paged_attention(q.to(DEV), kv.to(DEV), q_seq.to(DEV), q_kvlen.to(DEV), indptr.to(DEV),
                            indices.to(DEV), hq, hkv, d, page, d ** -0.5)
    _close(o, o_ref, 2e-2, 2e-2)


def test_attention_simt_tree_and_window():
    torch.manual_seed(6)
    hq, hkv, d, page = 4, 2, 64, 16
    lens = [40]
    kv, indptr, indices = _mk_paged(1, lens, hkv, d, page, torch.float16)
    # 4 tree tokens appended at positions 36..39; prefix 36; masks: chain 0-1, 0-2, 2-3
    q_seq = torch.zeros(4, dtype=torch.int32)
    q_kvlen = torch.full((4,), 36, dtype=torch.int32)
    masks = torch.tensor([0b0001, 0b0011, 0b0101, 0b1101], dtype=torch.int64)
    start = torch.full((4,), 20, dtype=torch.int32)
    q = (torch.randn(4, hq * d) * 0.5).half()
    o_ref = ops.paged_attention(q, kv, q_seq, q_kvlen, indptr, indices, hq, hkv, d, page, 0.125,
                                q_kvstart=start, sink=4, tree_mask=masks)
    o = ops.paged_attention(q.to(DEV), kv.to(DEV), q_seq.to(DEV), q_kvlen.to(DEV), indptr.to(DEV),
                            indices.to(DEV), hq, hkv, d, page, 0.125, q_kvstart=start.to(DEV), sink=4,
                            tree_mask=masks.to(DEV))
    _close(o, o_ref, 2e-2, 2e-2)


def test_softmax_argmax_sample():
    torch.manual_seed(7)
    n, v = 6, 32000
    logits = torch.randn(n, v) * 3
    temp = torch.tensor([1.0, 0.7, 0.0, 1.3, 0.0, 1.0])
    p_ref = ref.softmax_temperature(logits, temp)
    p = ops.softmax_temperature(logits.to(DEV), temp.to(DEV))
    _close(p, p_ref, 1e-3, 1e-7)
    assert torch.equal(ops.argmax(logits.to(DEV)).cpu().long(), logits.argmax(-1))
    u = torch.tensor([0.1, 0.5, 0.9, 0.3, 0.7, 0.999])
    for top_p in (1.0, 0.9, 0.3):
        tp = torch.full((n,), top_p)
        tok_ref, pr_ref = ref.sample(p_ref, None, u, tp)
        tok, pr = ops.sample(p, None, u.to(DEV), tp.to(DEV))
        # kept sets agree up to fp summation order; tokens must agree except at CDF boundaries
        agree = (tok.cpu() == tok_ref).float().mean().item()
        assert agree >= 0.8, (top_p, tok.cpu(), tok_ref)
        for r in range(n):
            if tok.cpu()[r] == tok_ref[r]:
                assert abs(pr.cpu()[r] - pr_ref[r]) < 1e-3 * max(1.0, pr_ref[r])


def test_sample_distribution_top_p():
    torch.manual_seed(8)
    v = 1000
    probs = torch.softmax(torch.randn(1, v) * 2, -1)
    n = 4000
    u = torch.rand(n)
    rows = torch.zeros(n, dtype=torch.int32)
    tp = torch.full((n,), 0.8)
    tok, _ = ops.sample(probs.to(DEV), rows.to(DEV), u.to(DEV), tp.to(DEV))
    cutoff, mass = ref.top_p_cutoff(probs[0], 0.8)
    kept = probs[0] >= cutoff
    assert bool(kept[tok.cpu().long()].all())
    emp = torch.bincount(tok.cpu().long(), minlength=v).float() / n
    expect = torch.where(kept, probs[0] / mass, torch.zeros(v))
    assert (emp - expect).abs().max() < 0.03


def test_logit_edits_and_take_probs_and_verify():
    torch.manual_seed(9)
    n, v = 3, 515
    logits = torch.randn(n, v)
    lg = logits.to(DEV)
    pos2seq = torch.tensor([0, 0, 2], dtype=torch.int32)
    token = torch.tensor([5, 9, 100], dtype=torch.int32)
    bias = torch.tensor([1.5, -2.0, 3.0])
    cnt = torch.tensor([2, 1, 4], dtype=torch.int32)
    pen = torch.tensor([[0.5, 0.2, 1.2], [0, 0, 1], [0.1, 0.3, 0.8]])
    lr = logits.clone()
    ref.apply_logit_bias(lr, pos2seq, token, bias)
    ref.apply_penalty(lr, pos2seq, token, cnt, pen)
    ops.apply_logit_bias(lg, pos2seq.to(DEV), token.to(DEV), bias.to(DEV))
    ops.apply_penalty(lg, pos2seq.to(DEV), token.to(DEV), cnt.to(DEV), pen.to(DEV))
    rows = torch.tensor([1], dtype=torch.int32)
    bm = torch.randint(-2**31, 2**31 - 1, (1, (v + 31) // 32), dtype=torch.int64).to(torch.int32)
    ref.apply_bitmask(lr, rows, bm)
    ops.apply_bitmask(lg, rows.to(DEV), bm.to(DEV))
    _close(lg, lr, 1e-5, 1e-5)
    probs = torch.softmax(torch.randn(n, v), -1)
    tok = torch.tensor([3, 4, 5], dtype=torch.int32)
    o, tp, ti = ops.take_probs(probs.to(DEV), None, tok.to(DEV), 5)
    orf, tpr, tir = ref.take_probs(probs, None, tok, 5)
    _close(o, orf, 1e-6, 1e-8)
    _close(tp, tpr, 1e-6, 1e-8)
    assert torch.equal(ti.cpu(), tir)
    # verify: 2 sequences, chain of 2 drafts each. nodes: 0,1 roots; 2,3 children of 0; 4 child of 1
    nodes = 6
    dp = torch.softmax(torch.randn(nodes, v), -1)
    mp = torch.softmax(torch.randn(nodes, v), -1)
    dt = torch.randint(0, v, (nodes,), dtype=torch.int32)
    fc = torch.tensor([2, 4, -1, -1, 5, -1], dtype=torch.int32)
    ns = torch.tensor([-1, -1, 3, -1, -1, -1], dtype=torch.int32)
    u = torch.rand(nodes)
    pp = torch.tensor([0, 1], dtype=torch.int32)
    mp_ref, pp_ref = mp.clone(), pp.clone()
    ref.verify_tree(dp, dt, mp_ref, fc, ns, u, pp_ref)
    mpg, ppg = mp.to(DEV), pp.to(DEV)
    ops.verify_tree(dp.to(DEV), dt.to(DEV), mpg, fc.to(DEV), ns.to(DEV), u.to(DEV), ppg)
    assert torch.equal(ppg.cpu(), pp_ref)
    _close(mpg, mp_ref, 1e-4, 1e-7)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (8, 1), (4, 4), (32, 8)])
@pytest.mark.parametrize("mode,splits", [("prefill", 1), ("decode", 1), ("mixed", 1), ("decode", 3),
                                         ("verify", 1), ("verify", 2), ("decode_many", 1), ("decode_many", 2)])
def test_attention_tcgen05(dtype, hq, hkv, mode, splits):
    from mlc_llm_b200.ops.attention import AttentionPlan, build_tiles

    torch.manual_seed(11)
    d, page = 128, 16
    if mode == "prefill":
        lens, appended = [70, 200, 33, 129], [70, 200, 33, 129]
    elif mode == "decode":
        lens, appended = [1, 17, 64, 65, 300, 128], [1, 1, 1, 1, 1, 1]
    elif mode == "decode_many":
        # more (sequence, kv head) units than the persistent decode kernel has CTAs: every CTA walks
        # several units of different lengths, so its page ring carries on across unit boundaries
        rng = np.random.default_rng(4)
        lens = [int(x) for x in rng.integers(1, 420, 330)]
        appended = [1] * len(lens)
    elif mode == "verify":
        lens, appended = [33, 500, 7, 260], [3, 4, 2, 4]
    else:
        lens, appended = [300, 40, 90], [44, 1, 90]
    kv, indptr, indices = _mk_paged(len(lens), lens, hkv, d, page, dtype)
    q_seq, q_kvlen, q_indptr = [], [], [0]
    for b, (l, a) in enumerate(zip(lens, appended)):
        for i in range(a):
            q_seq.append(b)
            q_kvlen.append(l - a + i + 1)
        q_indptr.append(len(q_seq))
    t = len(q_seq)
    qkv = (torch.randn(t, (hq + 2 * hkv) * d) * 0.7).to(dtype)
    q_seq = torch.tensor(q_seq, dtype=torch.int32)
    q_kvlen = torch.tensor(q_kvlen, dtype=torch.int32)
    scale = d ** -0.5
    o_ref, lse_ref = ops.paged_attention(qkv[:, : hq * d], kv, q_seq, q_kvlen, indptr, indices, hq, hkv, d,
                                         page, scale, return_lse=True)
    tiles = build_tiles(np.asarray(q_indptr), hq // hkv)
    dev = lambda a: torch.as_tensor(a).to(DEV)
    plan = AttentionPlan(dev(tiles["tile_seq"]), dev(tiles["tile_qstart"]), dev(tiles["tile_ntok"]),
                         q_kvlen.to(DEV), indptr.to(DEV), indices.to(DEV), len(tiles["tile_seq"]),
                         dec_seq=dev(tiles["dec_seq"]), dec_qstart=dev(tiles["dec_qstart"]),
                         dec_ntok=dev(tiles["dec_ntok"]), num_dec=len(tiles["dec_seq"]), dec_splits=splits)
    qg = qkv.to(DEV)
    o, lse = ops.paged_attention(qg[:, : hq * d], kv.to(DEV), q_seq.to(DEV), q_kvlen.to(DEV), indptr.to(DEV),
                                 indices.to(DEV), hq, hkv, d, page, scale, return_lse=True, plan=plan)
    ops.check_status(qg.device)
    _close(o, o_ref, 2e-2, 2e-2)
    _close(lse, lse_ref, 1e-2, 1e-2)


@pytest.mark.parametrize("quant_name", ["q0f16", "q4f16_1"])
@pytest.mark.parametrize("tokens", [1, 4, 37, 700])
def test_moe_block_kernels(quant_name, tokens):
    torch.manual_seed(21)
    e, k, hidden, inter = 8, 2, 256, 512
    quant = Q.get(quant_name)
    x = (torch.randn(tokens, hidden) * 0.5).half()
    gate = (torch.randn(tokens, e)).half()
    w13 = (torch.randn(e, 2 * inter, hidden) * 0.05).half()
    w2 = (torch.randn(e, hidden, inter) * 0.05).half()

    def mk(w):
        if quant.kind == "no-quant":
            return ops.LinearWeight("dense", w, None, None, None, w.shape[1], w.shape[2])
        qw, qs = Q.group_quantize(w, quant)
        return ops.LinearWeight("q4", qw, qs, None, quant, w.shape[1], w.shape[2])

    l13, l2 = mk(w13), mk(w2)

    def run(dev):
        xx, gg = x.to(dev), gate.to(dev)
        a13, a2 = l13.to(dev), l2.to(dev)
        wts, idx = ops.moe_router(gg, k, True)
        off, spos, src = ops.moe_permute(idx, e)
        xp = ops.row_gather(xx, src)
        h1 = ops.grouped_linear(xp, a13, off)
        y = ops.grouped_linear(ops.act_mul(h1), a2, off)
        return ops.moe_combine(y, wts, spos, None), wts, idx, off

    o_cpu, w_cpu, i_cpu, off_cpu = run("cpu")
    o_gpu, w_gpu, i_gpu, off_gpu = run(DEV)
    ops.check_status(torch.device(DEV))
    assert torch.equal(i_cpu.cpu(), i_gpu.cpu())
    assert torch.equal(off_cpu.cpu(), off_gpu.cpu())
    _close(w_gpu, w_cpu, 1e-3, 1e-5)
    _close(o_gpu, o_cpu, 3e-2, 3e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,rope,rank", [(4, 64, 128), (16, 64, 512), (5, 64, 192), (8, 128, 256)])
@pytest.mark.parametrize("masked", [False, True])
def test_latent_attention_kernel(dtype, hq, rope, rank, masked):
    """Absorbed latent attention over the compressed cache against the fp32 reference on the same 16-bit values:
    a prefill chunk on top of a cached prefix, decode tokens of other lengths (among them one row and a
    non-multiple of the four rows the kernel keeps in flight), scattered pages; with ``masked`` also window
    starts with sink rows and tree masks."""
    torch.manual_seed(hq + rank)
    page, d = 16, rope + rank
    kv_lens = [75, 1, 34, 130]
    q_lens = [11, 1, 1, 3]
    n_pages = 40
    perm = torch.randperm(n_pages - 1)[: sum((n + page - 1) // page for n in kv_lens)] + 1
    indptr, indices, at = [0], [], 0
    for n in kv_lens:
        k = (n + page - 1) // page
        indices += perm[at: at + k].tolist()
        at += k
        indptr.append(len(indices))
    cache = torch.zeros(n_pages, 1, 1, page, d, dtype=dtype)
    rows, slots, q_seq, q_kvlen = [], [], [], []
    for b, n in enumerate(kv_lens):
        r = (torch.randn(n, d) * 0.5).to(dtype)
        rows.append(r)
        pg = torch.tensor(indices[indptr[b]: indptr[b + 1]])
        slots.append(pg[torch.arange(n) // page] * page + torch.arange(n) % page)
        for j in range(q_lens[b]):
            q_seq.append(b)
            q_kvlen.append(n - q_lens[b] + j + 1)
    rows, slots = torch.cat(rows), torch.cat(slots).to(torch.int32)
    t = len(q_seq)
    q = (torch.randn(t, hq, d) * 0.5).to(dtype)
    q_seq, q_kvlen = torch.tensor(q_seq, dtype=torch.int32), torch.tensor(q_kvlen, dtype=torch.int32)
    kvstart = tree = None
    sink = 0
    if masked:
        sink = 2
        kvstart = torch.clamp(q_kvlen - 20, min=0).to(torch.int32)
        # the three tokens of the last sequence form a small tree behind the committed rows: a root and two
        # children that see the root and themselves
        q_kvlen[-3:] = kv_lens[-1] - 3
        kvstart[-3:] = 0
        tree = torch.zeros(t, dtype=torch.int64)
        tree[-3], tree[-2], tree[-1] = 0b001, 0b011, 0b101
    ipt, idx = torch.tensor(indptr, dtype=torch.int32), torch.tensor(indices, dtype=torch.int32)
    # the slot of a stand-in row is negative: it must be skipped
    rows_in = torch.cat([rows, torch.full((1, d), 7.0, dtype=dtype)])
    slots_in = torch.cat([slots, torch.tensor([-1], dtype=torch.int32)])
    ops.mla_append(rows_in.float(), cache_f := cache.float(), slots_in, page)
    want = ref.mla_attention(q.float(), cache_f, q_seq, q_kvlen, ipt, idx, rope, rank, page, 0.09, kvstart, sink, tree)
    cache_g = cache.to(DEV)
    ops.mla_append(rows_in.to(DEV), cache_g, slots_in.to(DEV), page)
    torch.cuda.synchronize()
    assert torch.equal(cache_g.cpu().float(), cache_f)
    mv = lambda x: None if x is None else x.to(DEV)
    got = ops.mla_attention(q.to(DEV), cache_g, mv(q_seq), mv(q_kvlen), mv(ipt), mv(idx), rope, rank, page, 0.09,
                            mv(kvstart), sink, mv(tree))
    ops.check_status(torch.device(DEV))
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    _close(got.float().cpu(), want, tol, tol)


@pytest.mark.parametrize("tokens,k,e", [(1, 2, 8), (7, 2, 8), (256, 2, 8), (300, 8, 128), (8192, 2, 8), (1000, 6, 256),
                                        (50, 4, 384)])
def test_moe_permute_is_the_stable_expert_major_order(tokens, k, e):
    """Offsets, row of every pair and source token of every row equal a stable sort by expert, for few and
    many experts (both kernels) and for pair counts below and above one pass of the CTA."""
    g = torch.Generator().manual_seed(tokens + e)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(tokens)]).to(torch.int32)
    if tokens > 8:  # a skewed case: most pairs on one expert
        idx[: tokens // 2, 0] = 1
    off_c, pos_c, src_c = ops.moe_permute(idx, e)
    off_g, pos_g, src_g = ops.moe_permute(idx.to(DEV), e)
    torch.cuda.synchronize()
    assert torch.equal(off_c, off_g.cpu())
    assert torch.equal(pos_c, pos_g.cpu())
    assert torch.equal(src_c, src_g.cpu())


@pytest.mark.parametrize("quant_name", ["q0f16", "q4f16_1", "q0bf16"])
@pytest.mark.parametrize("tokens,k", [(256, 2048), (37, 512), (1000, 1024), (70, 128)])
def test_fused_collective_gemm_single_rank(quant_name, tokens, k):
    """World size 1 runs the fused reduce-scatter / all-gather kernels in their degenerate form: the
    pushes go to this GPU's own buffers, so one GPU checks the epilogue addressing, the flags, the
    tail (residual add + RMSNorm) and the gather wait against the unfused ops."""
    from mlc_llm_b200.parallel.fused import FusedCollectives

    torch.manual_seed(5)
    hidden, inter = 512, 1536
    quant = Q.get(quant_name)
    dt = quant.torch_dtype
    x = (torch.randn(tokens, k) * 0.5).to(dt).to(DEV)
    res0 = (torch.randn(tokens, hidden) * 0.5).to(dt).to(DEV)
    nw = (1 + 0.1 * torch.randn(hidden)).to(dt).to(DEV)
    w_o = (torch.randn(hidden, k) * 0.05).to(dt)
    w_up = (torch.randn(inter, hidden) * 0.05).to(dt)

    def mk(w):
        if quant.kind == "no-quant":
            return ops.LinearWeight("dense", w, None, None, None, w.shape[0], w.shape[1]).to(DEV)
        qw, qs = Q.group_quantize(w, quant)
        return ops.LinearWeight("q4", qw, qs, None, quant, w.shape[0], w.shape[1]).to(DEV)

    l_o, l_up = mk(w_o), mk(w_up)
    fc = FusedCollectives(hidden, dt, 1024, torch.device(DEV), mode="rs")
    for rep in range(3):  # several epochs over the same buffers
        fc.begin(tokens)
        fc.scatter_residual(res0)
        fc.gemm_rs_norm(x, l_o, nw, 1e-5)
        y = fc.gemm_ag(l_up)
        xn = fc.wait_gather().clone()
        ops.check_status(torch.device(DEV))
        # unfused oracle with the same kernels
        res = res0.clone()
        o = ops.linear(x, l_o)
        want_xn = ops.add_rmsnorm(o, res, nw, 1e-5)
        want_y = ops.linear(want_xn, l_up)
        tol = 3e-2 if dt == torch.bfloat16 else 4e-3
        _close(fc.residual[:tokens], res, tol, tol)
        _close(xn, want_xn, tol, tol)
        _close(y, want_y, 10 * tol, 10 * tol)


@pytest.mark.parametrize("quant_name", ["q0f16", "q4f16_1", "q0bf16"])
@pytest.mark.parametrize("tokens,k", [(256, 2048), (37, 512), (1000, 1024), (5, 64)])
def test_fused_all_reduce_gemm_single_rank(quant_name, tokens, k):
    """World size 1 runs the GEMM + all-reduce + residual + RMSNorm kernel in its degenerate form: the
    grid-wide barrier, the call numbers over several launches and the tail's arithmetic against the
    unfused ops (the sum over ranks has a single term)."""
    from mlc_llm_b200.parallel.fused import FusedCollectives

    torch.manual_seed(6)
    hidden = 512
    quant = Q.get(quant_name)
    dt = quant.torch_dtype
    x = (torch.randn(tokens, k) * 0.5).to(dt).to(DEV)
    res0 = (torch.randn(tokens, hidden) * 0.5).to(dt).to(DEV)
    nw = (1 + 0.1 * torch.randn(hidden)).to(dt).to(DEV)
    w_o = (torch.randn(hidden, k) * 0.05).to(dt)
    if quant.kind == "no-quant":
        l_o = ops.LinearWeight("dense", w_o, None, None, None, hidden, k).to(DEV)
    else:
        qw, qs = Q.group_quantize(w_o, quant)
        l_o = ops.LinearWeight("q4", qw, qs, None, quant, hidden, k).to(DEV)
    fc = FusedCollectives(hidden, dt, 1024, torch.device(DEV), mode="ar")
    res = res0.clone()
    fc.begin(tokens)
    fc.scatter_residual(res0)
    for rep in range(4):  # the residual carries over from call to call, as it does from layer to layer
        xn = fc.gemm_ar_norm(x, l_o, nw, 1e-5).clone()
        ops.check_status(torch.device(DEV))
        o = ops.linear(x, l_o)
        want_xn = ops.add_rmsnorm(o, res, nw, 1e-5)
        tol = 3e-2 if dt == torch.bfloat16 else 4e-3
        _close(fc.residual[:tokens], res, tol * (rep + 1), tol * (rep + 1))
        _close(xn, want_xn, tol * (rep + 1), tol * (rep + 1))
    fc.end()


@pytest.mark.parametrize("quant_name", ["q0f16", "q4f16_1", "q0bf16", "fp8_e4m3fn_bf16_block_scale"])
@pytest.mark.parametrize("tokens", [1, 37, 300])
def test_expert_parallel_exchange_single_rank(quant_name, tokens):
    """World size 1 runs dispatch -> group table -> grouped GEMMs -> combine through this GPU's own
    exchange buffers; the result must equal the local (permute + grouped GEMM) MoE path."""
    from mlc_llm_b200.parallel.expert import ExpertParallel

    torch.manual_seed(9)
    e, k, hidden, inter = 8, 2, 256, 512
    quant = Q.get(quant_name)
    dt = quant.torch_dtype
    x = (torch.randn(tokens, hidden) * 0.5).to(dt).to(DEV)
    gate = torch.randn(tokens, e).to(dt).to(DEV)
    w13 = (torch.randn(e, 2 * inter, hidden) * 0.05).to(dt)
    w2 = (torch.randn(e, hidden, inter) * 0.05).to(dt)

    def mk(w):
        if quant.kind == "no-quant":
            return ops.LinearWeight("dense", w, None, None, None, w.shape[1], w.shape[2]).to(DEV)
        if quant.kind == "fp8-block-scale":
            fw, fs = Q.fp8_block_quantize(w.float(), (128, 128), "float8_e4m3fn")
            return ops.LinearWeight("fp8_block", fw.to(DEV), fs.float().to(DEV), None, quant, w.shape[1], w.shape[2])
        qw, qs = Q.group_quantize(w, quant)
        return ops.LinearWeight("q4", qw, qs, None, quant, w.shape[1], w.shape[2]).to(DEV)

    l13, l2 = mk(w13), mk(w2)
    wts, idx = ops.moe_router(gate, k, True)
    off, spos, src = ops.moe_permute(idx, e)
    h1 = ops.grouped_linear(ops.row_gather(x, src), l13, off)
    want = ops.moe_combine(ops.grouped_linear(ops.act_mul(h1), l2, off), wts, spos, None)
    ep = ExpertParallel(e, k, hidden, dt, 512, torch.device(DEV))
    for _ in range(3):
        got = ep.ffn(x, wts, idx, l13, l2)
        ops.check_status(torch.device(DEV))
        tol = 3e-2 if dt == torch.bfloat16 else 4e-3
        _close(got, want, tol, tol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (33, 384, 512), (256, 1024, 4096), (700, 512, 1024)])
def test_fp8_block_scale_linear(dtype, m, n, k, monkeypatch):
    """fp8 weights, 16-bit activations (the weights are expanded inside the 16-bit GEMM)."""
    from mlc_llm_b200.ops import fp8 as fp8_ops

    monkeypatch.setattr(fp8_ops, "_FP8_ACT", False)
    torch.manual_seed(3)
    w = torch.randn(n, k) * 0.05
    qw, sc = Q.fp8_block_quantize(w, (128, 128), "float8_e4m3fn")
    quant = Q.get("fp8_e4m3fn_bf16_block_scale")
    x = (torch.randn(m, k) * 0.5).to(dtype)
    lw = ops.LinearWeight("fp8_block", qw.to(DEV), sc.float().to(DEV), None, quant, n, k)
    y = ops.linear(x.to(DEV), lw)
    ops.check_status(torch.device(DEV))
    want = x.float() @ Q.fp8_block_dequantize(qw, sc, (128, 128)).float().t()
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    _close(y, want, tol, tol * want.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k", [(1, 128), (37, 512), (300, 4096)])
def test_fp8_activation_quantisation_matches_the_reference_formula(dtype, m, k):
    from mlc_llm_b200.ops.fp8 import act_quant_fp8

    torch.manual_seed(4)
    x = (torch.randn(m, k) * torch.rand(m, 1) * 3).to(dtype)
    x[0, :5] = 0
    xq, st = act_quant_fp8(x.to(DEV))
    q_ref, s_ref = Q.fp8_rowwise_group_quantize(x.float(), 128, "float8_e4m3fn")
    assert torch.equal(st[:, :m].t().cpu(), s_ref)
    assert torch.equal(xq.cpu().view(torch.uint8), q_ref.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(17, 256, 256), (33, 384, 512), (256, 1024, 4096), (700, 512, 1024),
                                   (2048, 640, 1280)])
def test_fp8_w8a8_linear(dtype, m, n, k):
    """fp8 weights and fp8 activations on the fp8 tensor-core path. The oracle is the fp32 product of the two
    dequantised operands (activations quantised per row and 128-element group by the reference formula), so
    the tolerance only has to cover fp32 summation order and the rounding of the output."""
    torch.manual_seed(5)
    w = torch.randn(n, k) * 0.05
    qw, sc = Q.fp8_block_quantize(w, (128, 128), "float8_e4m3fn")
    quant = Q.get("fp8_e4m3fn_bf16_block_scale")
    x = (torch.randn(m, k) * 0.5).to(dtype)
    bias = (torch.randn(n) * 0.1).to(dtype)
    lw = ops.LinearWeight("fp8_block", qw.to(DEV), sc.float().to(DEV), bias.to(DEV), quant, n, k)
    y = ops.linear(x.to(DEV), lw)
    ops.check_status(torch.device(DEV))
    xq, xs = Q.fp8_rowwise_group_quantize(x.float(), 128, "float8_e4m3fn")
    x_deq = xq.float() * xs.repeat_interleave(128, dim=1)[:, :k]
    want = x_deq @ Q.fp8_block_dequantize(qw, sc, (128, 128)).float().t() + bias.float()
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-3
    _close(y, want, tol, tol * want.abs().max().item())
    # and the end-to-end error against unquantised activations stays at the few-percent level of e4m3
    full = x.float() @ Q.fp8_block_dequantize(qw, sc, (128, 128)).float().t() + bias.float()
    rel = (y.float().cpu() - full).norm() / full.norm()
    assert rel < 0.05, rel


@pytest.fixture
def pair_mode():
    """CTA-pair (cta_group::2) form of the GEMM kernel for the duration of a test."""
    from mlc_llm_b200.ops._lib import lib
    lib().mlcb_gemm_set_pair_mode(1)
    yield
    lib().mlcb_gemm_set_pair_mode(2)


@pytest.mark.parametrize("quant_name", ["q0f16", "q0bf16", "q4f16_1"])
@pytest.mark.parametrize("m,n,k", [(64, 256, 512), (256, 512, 4096), (256, 384, 1024), (300, 1152, 2048),
                                   (2048, 1024, 1024), (1000, 640, 512)])
def test_gemm_cta_pair_mode(pair_mode, quant_name, m, n, k):
    torch.manual_seed(11)
    quant = Q.get(quant_name)
    dt = quant.torch_dtype
    w = (torch.randn(n, k) * 0.05).to(dt)
    x = (torch.randn(m, k) * 0.5).to(dt)
    if quant.kind == "no-quant":
        lw = ops.LinearWeight("dense", w, None, None, None, n, k).to(DEV)
        wref = w.float()
    else:
        qw, qs = Q.group_quantize(w, quant)
        lw = ops.LinearWeight("q4", qw, qs, None, quant, n, k).to(DEV)
        wref = Q.group_dequantize(qw, qs, quant, k=k).float()
    for _ in range(2):
        y = ops.linear(x.to(DEV), lw)
        ops.check_status(torch.device(DEV))
        want = x.float() @ wref.t()
        tol = 2e-2 if dt == torch.bfloat16 else 3e-3
        _close(y, want, tol, tol * want.abs().max().item())


@pytest.mark.parametrize("per_token_decay", [False, True])
@pytest.mark.parametrize("head_size", [64, 32])
def test_wkv5_recurrence_kernel(head_size, per_token_decay):
    """RWKV-5 / RWKV-6 recurrence: one launch over three sequences of different lengths (one of them
    continuing from a non-zero state) against the per-token fp32 loop; RWKV-6 has one decay per token."""
    from mlc_llm_b200.models.rwkv import wkv5, wkv5_batch

    torch.manual_seed(0)
    n, layers, pos = 3, 2, 1
    lens = [5, 1, 17]
    qi = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    t_all = int(qi[-1])
    r, k, v = (torch.randn(t_all, n, head_size) * 0.5 for _ in range(3))
    w = torch.rand(*((t_all,) if per_token_decay else ()), n, head_size) * 0.7 + 0.25
    u = torch.randn(n, head_size) * 0.3
    states = [torch.randn(layers, n, head_size, head_size) * (0.2 if i == 2 else 0.0) for i in range(3)]
    want_states = [s.clone() for s in states]
    want = torch.cat([wkv5(r[qi[i]:qi[i + 1]], k[qi[i]:qi[i + 1]], v[qi[i]:qi[i + 1]],
                           w[qi[i]:qi[i + 1]] if per_token_decay else w, u, want_states[i][pos])
                      for i in range(3)])
    dev_states = [s.cuda() for s in states]
    got = wkv5_batch(r.cuda(), k.cuda(), v.cuda(), w.cuda(), u.cuda(), dev_states, pos, qi)
    torch.cuda.synchronize()
    assert torch.allclose(got.cpu(), want, atol=1e-4, rtol=1e-4), (got.cpu() - want).abs().max()
    for a, b in zip(dev_states, want_states):
        assert torch.allclose(a.cpu(), b, atol=1e-4, rtol=1e-4)
        assert torch.equal(a[0].cpu(), b[0])  # the other layer's rows are untouched


@pytest.mark.parametrize("form", [1, 2])
@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1000, 14336), (77, 128), (28672, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_gemv_q4_matches_dequantised_matmul(m, n, k, out_dtype, form, monkeypatch):
    """One to four tokens against q4f16_1 weights take the CUDA-core GEMV; rows that are not a multiple
    of the 32 rows of a CTA, a K that leaves lanes idle, bias, fp32 output."""
    torch.manual_seed(m * 1000 + n + k)
    quant = Q.get("q4f16_1")
    w = torch.randn(n, k) * 0.05
    qw, qs = Q.group_quantize(w.half(), quant)
    wd = Q.group_dequantize(qw, qs, quant, k=k, out_dtype=torch.float32)
    bias = (torch.randn(n) * 0.1).half()
    lw = ops.LinearWeight("q4", qw, qs, bias, quant, n, k, False).to("cuda")
    x = (torch.randn(m, k) * 0.5).half()
    want = x.float() @ wd.t() + bias.float()
    monkeypatch.setattr(ops, "_GEMV_Q4", True)
    ops.lib().mlcb_gemv_set_form(form)   # 1: one warp per four rows; 2: K split across warps + prefetch
    try:
        got = ops.linear(x.cuda(), lw, out_dtype=out_dtype)
    finally:
        ops.lib().mlcb_gemv_set_form(2)
    ops.check_status(torch.device("cuda"))
    assert got.dtype == out_dtype and got.shape == (m, n)
    err = (got.float().cpu() - want).abs().max()
    assert err < 2e-2 * max(1.0, float(want.abs().max())), err


@pytest.mark.parametrize("m", [5, 8, 9, 13, 16])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1000, 14336), (77, 128), (28672, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_gemm_q4_low_token_counts_matches_dequantised_matmul(m, n, k, out_dtype, monkeypatch):
    """Five to sixteen tokens against q4f16_1 weights: nibbles expanded in registers into mma.sync fragments."""
    torch.manual_seed(m * 1000 + n + k)
    quant = Q.get("q4f16_1")
    w = torch.randn(n, k) * 0.05
    qw, qs = Q.group_quantize(w.half(), quant)
    wd = Q.group_dequantize(qw, qs, quant, k=k, out_dtype=torch.float32)
    bias = (torch.randn(n) * 0.1).half()
    lw = ops.LinearWeight("q4", qw, qs, bias, quant, n, k, False).to("cuda")
    x = (torch.randn(m, k) * 0.5).half()
    want = x.float() @ wd.t() + bias.float()
    monkeypatch.setattr(ops, "_LOWM_Q4", True)
    got = ops.linear(x.cuda(), lw, out_dtype=out_dtype)
    ops.check_status(torch.device("cuda"))
    assert got.dtype == out_dtype and got.shape == (m, n)
    err = (got.float().cpu() - want).abs().max()
    assert err < 2e-2 * max(1.0, float(want.abs().max())), err


def test_bounded_device_wait_reports_through_the_status_word():
    """A cross-GPU flag that nobody raises: the waiting kernel gives up after its time limit (about two
    seconds), records the reason in the device status word and returns; the context stays usable."""
    import ctypes
    import time

    from mlc_llm_b200.ops import _lib

    dev = torch.device("cuda")
    _lib.check_status(dev)                      # start from a clean word
    flags = torch.zeros(64, dtype=torch.int32, device=dev)   # call number 0 everywhere
    base = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.time()
    rc = _lib.lib().mlcb_flag_wait(_lib.ptr(flags), ctypes.c_int(16), ctypes.c_int(1), _lib.ptr(base),
                                   _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.0 < waited < 10.0, waited          # it did wait, and it did stop
    with pytest.raises(_lib.KernelError, match="peer GPU"):
        _lib.check_status(dev)
    _lib.check_status(dev)                      # reading the status cleared it
    x = torch.randn(8, 64, device=dev, dtype=torch.float16)
    y = ops.rmsnorm(x, torch.ones(64, device=dev, dtype=torch.float16), 1e-5, 0.0)
    assert torch.isfinite(y).all()


@pytest.mark.gpu
def test_page_copy_all_layers_one_launch():
    """Copy-on-write page copies: (src, dst) pairs applied to every layer by one kernel, against indexing."""
    import ctypes

    from mlc_llm_b200.ops._lib import check, lib, ptr, stream_ptr

    torch.manual_seed(0)
    kv = torch.randn(3, 20, 2, 4, 16, 128, device="cuda", dtype=torch.float16)
    pairs = torch.tensor([1, 7, 3, 9, 1, 12], dtype=torch.int32, device="cuda")
    want = kv.clone()
    want[:, pairs[1::2].long()] = want[:, pairs[0::2].long()]
    es = kv.element_size()
    check(lib().mlcb_page_copy(ptr(kv), ptr(pairs), ctypes.c_int(3), ctypes.c_int(kv.shape[0]),
                               ctypes.c_longlong(kv.stride(1) * es), ctypes.c_longlong(kv.stride(0) * es),
                               stream_ptr()), "mlcb_page_copy")
    torch.cuda.synchronize()
    assert torch.equal(kv, want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (16, 2), (4, 4)])
@pytest.mark.parametrize("case", ["window", "window_sink", "softcap", "tree", "tree_window_softcap", "decode_window"])
@pytest.mark.parametrize("decode_items,splits", [(False, 1), (True, 1), (True, 3)])
def test_attention_tcgen05_masked(dtype, hq, hkv, case, decode_items, splits):
    """Windows (with and without sinks, whole blocks skipped), logit soft-capping and token-tree masks on the
    tensor-core kernel, against the fp32 reference of the same visibility rule."""
    from mlc_llm_b200.ops.attention import AttentionPlan, build_tiles

    torch.manual_seed(12)
    d, page = 128, 16
    window = sink = 0
    softcap = 0.0
    tree = None
    if case in ("window", "window_sink"):
        lens, appended = [700, 90, 300, 1500], [130, 90, 5, 1]
        window, sink = 256, (0 if case == "window" else 70)
    elif case == "decode_window":
        lens, appended = [900, 40, 257, 513, 2000], [1, 1, 1, 1, 1]
        window, sink = 256, 4
    elif case == "softcap":
        lens, appended = [200, 77, 300], [200, 3, 1]
        softcap = 30.0
    else:
        # token trees of 5, 7 and 3 nodes behind prefixes of 300, 61 and 0 tokens
        parents = [[-1, 0, 0, 1, 3], [-1, -1, 0, 1, 1, 4, 2], [-1, 0, 1]]
        prefix = [300, 61, 0]
        appended = [len(p) for p in parents]
        lens = [a + b for a, b in zip(prefix, appended)]
        tree = parents
        if case == "tree_window_softcap":
            window, sink, softcap = 128, 16, 20.0
    kv, indptr, indices = _mk_paged(len(lens), lens, hkv, d, page, dtype)
    q_seq, q_kvlen, q_indptr, masks = [], [], [0], []
    for b, (l, a) in enumerate(zip(lens, appended)):
        node_masks = []
        for i in range(a):
            q_seq.append(b)
            if tree is None:
                q_kvlen.append(l - a + i + 1)
            else:
                q_kvlen.append(l - a)
                par = tree[b][i]
                node_masks.append((node_masks[par] if par >= 0 else 0) | (1 << i))
        masks.extend(node_masks)
        q_indptr.append(len(q_seq))
    t = len(q_seq)
    qkv = (torch.randn(t, (hq + 2 * hkv) * d) * (3.0 if softcap else 0.7)).to(dtype)
    q_seq = torch.tensor(q_seq, dtype=torch.int32)
    q_kvlen = torch.tensor(q_kvlen, dtype=torch.int32)
    kvstart = torch.clamp(q_kvlen - window, min=0).to(torch.int32) if window else None
    tmask = torch.tensor(masks, dtype=torch.int64) if tree is not None else None
    scale = d ** -0.5
    o_ref, lse_ref = ops.paged_attention(qkv[:, : hq * d], kv, q_seq, q_kvlen, indptr, indices, hq, hkv, d,
                                         page, scale, q_kvstart=kvstart, sink=sink, tree_mask=tmask,
                                         softcap=softcap, return_lse=True)
    # decode-sized items go to the decode kernel's masked variant, the rest to the tcgen05 kernel's;
    # `splits` also cuts the decode items' (window-compacted) page ranges
    tiles = build_tiles(np.asarray(q_indptr), hq // hkv, decode_items=decode_items)
    dev = lambda a: torch.as_tensor(a).to(DEV)
    plan = AttentionPlan(dev(tiles["tile_seq"]), dev(tiles["tile_qstart"]), dev(tiles["tile_ntok"]),
                         q_kvlen.to(DEV), indptr.to(DEV), indices.to(DEV), len(tiles["tile_seq"]),
                         dec_seq=dev(tiles["dec_seq"]), dec_qstart=dev(tiles["dec_qstart"]),
                         dec_ntok=dev(tiles["dec_ntok"]), num_dec=len(tiles["dec_seq"]), dec_splits=splits)
    if decode_items and (case == "decode_window" or (case == "tree" and hq // hkv <= 4)):
        assert plan.num_dec > 0
    qg = qkv.to(DEV)
    from mlc_llm_b200.ops._lib import lib

    lib().mlcb_launch_count.restype = __import__("ctypes").c_longlong
    o, lse = ops.paged_attention(qg[:, : hq * d], kv.to(DEV), q_seq.to(DEV), q_kvlen.to(DEV), indptr.to(DEV),
                                 indices.to(DEV), hq, hkv, d, page, scale,
                                 q_kvstart=None if kvstart is None else kvstart.to(DEV), sink=sink,
                                 tree_mask=None if tmask is None else tmask.to(DEV), softcap=softcap,
                                 return_lse=True, plan=plan)
    ops.check_status(qg.device)
    _close(o, o_ref, 2e-2, 2e-2)
    _close(lse, lse_ref, 1e-2, 1e-2)


@pytest.mark.parametrize("m", [3, 40, 300])
def test_fp8_per_tensor_linear_runs_on_the_block_scale_kernels(m):
    """A per-tensor fp8 weight is a block-scaled one whose blocks share one scale: no dense copy is made."""
    torch.manual_seed(8)
    n, k = 384, 512
    w = torch.randn(n, k) * 0.05
    qw, sc = Q.fp8_per_tensor_quantize(w, "float8_e4m3fn")
    x = (torch.randn(m, k) * 0.5).to(torch.bfloat16)
    lw = ops.LinearWeight("fp8_tensor", qw.to(DEV), sc.float().to(DEV), None, None, n, k)
    y = ops.linear(x.to(DEV), lw)
    ops.check_status(torch.device(DEV))
    assert lw._dense is None and lw.block_scale().shape == (3, 4)
    want = x.float() @ (qw.float() * sc.float()).t()
    rel = (y.float().cpu() - want).norm() / want.norm()
    assert rel < 0.05, rel


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hidden", [768, 4096, 5120])
def test_layernorm_and_plain_activations(dtype, hidden):
    torch.manual_seed(9)
    t = 37
    x = (torch.randn(t, hidden) * 2 + 0.3).to(dtype)
    res = torch.randn(t, hidden).to(dtype)
    w = (torch.rand(hidden) + 0.5).to(dtype)
    b = (torch.randn(hidden) * 0.1).to(dtype)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    for bias in (b, None):
        want = ref.layernorm(x, w, bias, 1e-5)
        got = ops.layernorm(x.to(DEV), w.to(DEV), None if bias is None else bias.to(DEV), 1e-5)
        _close(got, want, tol, tol)
    # fused residual add: the sum is written back and normalised
    r_dev = res.to(DEV).clone()
    got = ops.layernorm(x.to(DEV), w.to(DEV), b.to(DEV), 1e-5, residual=r_dev)
    summed = (x.float() + res.float()).to(dtype)
    _close(r_dev, summed, tol, tol)
    _close(got, ref.layernorm(summed, w, b, 1e-5), tol, tol)
    for act in ("silu", "gelu", "gelu_tanh", "relu2", "quick_gelu"):
        _close(ops.activation(x.to(DEV), act), ops.activation(x, act), tol, tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("e,n_group,topk_group,k,renorm", [(160, 8, 3, 6, False), (64, 8, 4, 6, True), (16, 4, 2, 2, True)])
def test_group_limited_router_kernel(dtype, e, n_group, topk_group, k, renorm):
    """DeepSeek-V2 routing on the GPU against the tensor-operation form on the CPU (same selection, same weights)."""
    from mlc_llm_b200.models.moe import _group_limited_router

    torch.manual_seed(13)
    logits = (torch.randn(301, e) * 2).to(dtype)
    w_ref, i_ref = _group_limited_router(logits.float(), k, n_group, topk_group, renorm)
    w, i = _group_limited_router(logits.to(DEV), k, n_group, topk_group, renorm)
    # fp16 logits tie often and the two sides break ties differently: compare what is tie-proof, the sorted
    # weights, and check that every chosen expert carries the weight it was given
    # (with fp16 logits even whole groups tie at the cut, so there only the self-consistency checks apply)
    if dtype == torch.float32:
        _close(w.cpu().sort(dim=1).values, w_ref.sort(dim=1).values, 1e-4, 1e-6)
        assert torch.equal(i.cpu().sort(dim=1).values, i_ref.sort(dim=1).values)
    groups_used = (i.cpu() // (e // n_group))
    assert all(len(set(row)) <= topk_group for row in groups_used.tolist())
    probs = torch.softmax(logits.float(), dim=-1)
    own = probs.gather(1, i.cpu().long())
    if renorm:
        own = own / own.sum(dim=1, keepdim=True)
    _close(w.cpu(), own, 1e-4, 1e-6)
    assert all(len(set(row)) == k for row in i.cpu().tolist())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("d", [32, 64, 96, 128])
@pytest.mark.parametrize("case", ["plain", "padded", "causal", "packed_qkv"])
def test_encoder_attention(dtype, d, case):
    """Whole-sequence attention (vision towers, BERT) against fp32 tensor operations: sequence lengths off the
    64-row tile size, per-batch key lengths, causal masking, and q / k / v as strided views of one projection."""
    torch.manual_seed(14)
    b, s, h = 3, 197, 4
    if case == "packed_qkv":
        qkv = (torch.randn(b, s, 3, h, d) * 0.8).to(dtype)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        qkv_d = qkv.to(DEV)
        qd, kd, vd = qkv_d[:, :, 0], qkv_d[:, :, 1], qkv_d[:, :, 2]
    else:
        q, k, v = ((torch.randn(b, s, h, d) * 0.8).to(dtype) for _ in range(3))
        qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    lens = torch.tensor([197, 64, 5], dtype=torch.int32) if case == "padded" else None
    want = ops.encoder_attention(q.float(), k.float(), v.float(), key_lens=lens, causal=case == "causal")
    got = ops.encoder_attention(qd, kd, vd, key_lens=None if lens is None else lens.to(DEV), causal=case == "causal")
    assert got.shape == (b, s, h, d) and got.is_contiguous()
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    _close(got, want, tol, tol)


@pytest.mark.parametrize("dk,dv", [(128, 128), (64, 128), (64, 256)])
def test_gated_delta_step_kernel(dk, dv):
    """One decode token of the gated delta rule, in place on a slot-indexed state pool, against the tensor form."""
    from mlc_llm_b200.models.qwen35 import _gdn_step_kernel, gated_delta_step

    torch.manual_seed(15)
    slots_cap, b, h = 9, 5, 4
    pool = torch.randn(slots_cap, h, dk, dv) * 0.3
    slots = [7, 0, 3, 8, 2]
    q = torch.nn.functional.normalize(torch.randn(b, h, dk), dim=-1) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(b, h, dk), dim=-1)
    v = torch.randn(b, h, dv)
    g = -torch.rand(b, h)
    beta = torch.rand(b, h)
    state = pool[slots].clone()
    want = gated_delta_step(state, q, k, v, g, beta)
    want_pool = pool.clone()
    want_pool[slots] = state
    pool_d = pool.to(DEV)
    out = torch.zeros(b, h, dv, device=DEV)
    rows = torch.arange(b, device=DEV)
    assert _gdn_step_kernel(pool_d, slots, q.to(DEV), k.to(DEV), v.to(DEV), g.to(DEV), beta.to(DEV), out, rows)
    _close(out, want, 1e-4, 1e-5)
    _close(pool_d, want_pool, 1e-4, 1e-5)


def test_sampling_cutoffs_top_k_and_top_p():
    """The multi-way cutoff search: top-k alone, top-p alone and both, on peaked and on flat rows; the sampled token
    always lies in the set the CPU reference keeps, and its reported probability is the renormalised one."""
    torch.manual_seed(16)
    n, v = 12, 128256
    logits = torch.randn(n, v) * torch.tensor([0.5, 1, 2, 3, 4, 6] * 2).view(n, 1)
    temp = torch.ones(n)
    p = ops.softmax_temperature(logits.to(DEV), temp.to(DEV))
    p_cpu = p.cpu()
    sorted_p, order = p_cpu.sort(dim=1, descending=True)
    for top_p, top_k in ((1.0, 5), (1.0, 1), (0.9, 0), (0.5, 40), (0.999, 3), (0.2, 1000)):
        for u0 in (0.0, 0.37, 0.93, 0.9999):
            u = torch.full((n,), u0)
            tp = torch.full((n,), top_p)
            tk = torch.full((n,), top_k, dtype=torch.int32) if top_k else None
            tok, pr = ops.sample(p, None, u.to(DEV), tp.to(DEV), None if tk is None else tk.to(DEV))
            tok, pr = tok.cpu().long(), pr.cpu()
            for r in range(n):
                # the kept set: smallest prefix of the sorted row reaching top_p, capped at top_k
                csum = sorted_p[r].cumsum(0)
                need = top_p * csum[-1]
                m = v if top_p >= 1.0 else int((csum < need - 1e-6).sum().item()) + 1
                if top_k:
                    m = min(m, top_k)
                floor = sorted_p[r][m - 1].item()
                assert p_cpu[r, tok[r]].item() >= floor * (1 - 1e-5), (top_p, top_k, u0, r)
                kept = sorted_p[r][:m].sum().item()
                assert abs(pr[r].item() - p_cpu[r, tok[r]].item() / kept) < 2e-3 * max(1.0, pr[r].item())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens", [1, 37, 700])
def test_grouped_gemm_fp8_block_scale_experts(dtype, tokens):
    """Stacked e4m3 expert weights with 128 x 128 block scales through the grouped GEMM (no dense copy): against
    the fp32 product with the dequantised weights."""
    torch.manual_seed(17)
    e, n, k = 4, 256, 384
    w = torch.randn(e, n, k) * 0.05
    qw, sc = Q.fp8_block_quantize(w, (128, 128), "float8_e4m3fn")
    quant = Q.get("fp8_e4m3fn_bf16_block_scale")
    lw = ops.LinearWeight("fp8_block", qw.to(DEV), sc.float().to(DEV), None, quant, n, k)
    counts = torch.tensor([tokens // 2, 0, tokens - tokens // 2 - tokens // 5, tokens // 5])
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(torch.int32)
    x = (torch.randn(tokens, k) * 0.5).to(dtype)
    y = ops.grouped_linear(x.to(DEV), lw, offsets.to(DEV))
    ops.check_status(torch.device(DEV))
    assert lw._dense is None
    wd = Q.fp8_block_dequantize(qw, sc, (128, 128)).float()
    want = torch.zeros(tokens, n)
    off = offsets.tolist()
    for i in range(e):
        want[off[i]:off[i + 1]] = x[off[i]:off[i + 1]].float() @ wd[i].t()
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    _close(y, want, tol, tol * max(1e-3, want.abs().max().item()))
