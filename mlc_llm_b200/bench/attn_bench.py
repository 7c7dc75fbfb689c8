"""Device-timed paged-attention benchmarks (decode and prefill) against the measured HBM / tensor
peaks.  KV caches are sized above L2 so every launch streams from HBM."""

from __future__ import annotations

import json

import numpy as np
import torch

from .. import ops
from ..ops.attention import AttentionPlan, build_tiles, choose_splits
from .kernel_bench import _peaks, _time, _time_graph


def _plan(batch: int, ctx: int, append: int, hq: int, hkv: int, dev) -> AttentionPlan:
    pages_per = (ctx + 15) // 16
    q_indptr = np.arange(batch + 1, dtype=np.int64) * append
    tiles = build_tiles(q_indptr, hq // hkv)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    q_kvlen = np.concatenate([np.arange(ctx - append + 1, ctx + 1, dtype=np.int32) for _ in range(batch)])
    page_indptr = (np.arange(batch + 1) * pages_per).astype(np.int32)
    rng = np.random.default_rng(0)
    page_indices = rng.permutation(batch * pages_per).astype(np.int32)
    n_dec = len(tiles["dec_seq"])
    return AttentionPlan(t(tiles["tile_seq"]), t(tiles["tile_qstart"]), t(tiles["tile_ntok"]), t(q_kvlen),
                         t(page_indptr), t(page_indices), len(tiles["tile_seq"]), dec_seq=t(tiles["dec_seq"]),
                         dec_qstart=t(tiles["dec_qstart"]), dec_ntok=t(tiles["dec_ntok"]), num_dec=n_dec,
                         dec_splits=choose_splits(n_dec, hkv, pages_per, dev) if n_dec else 1,
                         max_pages=pages_per)


def bench_attention(which: str, small: bool):
    dev = torch.device("cuda")
    hbm, tf, how = _peaks()
    hq, hkv, d = 32, 8, 128
    out = []
    cases = []
    if which in ("attn_decode", "all"):
        cases += [("attn_decode", b, c, 1) for b, c in ([(64, 1024)] if small else [(256, 640), (256, 2048), (8, 16384)])]
    if which in ("attn_prefill", "all"):
        cases += [("attn_prefill", b, c, c) for b, c in ([(4, 1024)] if small else [(16, 512), (4, 4096), (1, 16384)])]
    for kind, batch, ctx, append in cases:
        pages = batch * ((ctx + 15) // 16)
        kv = (torch.randn(pages, 2, hkv, 16, d, device=dev) * 0.5).half()
        plan = _plan(batch, ctx, append, hq, hkv, dev)
        t = batch * append
        q = (torch.randn(t, (hq + 2 * hkv) * d, device=dev) * 0.5).half()
        q_seq = torch.arange(batch, device=dev, dtype=torch.int32).repeat_interleave(append)
        fn = lambda: ops.paged_attention(q[:, : hq * d], kv, q_seq, plan.q_kvlen, plan.page_indptr,
                                         plan.page_indices, hq, hkv, d, 16, d ** -0.5, plan=plan)
        med, best = _time(fn)
        in_graph = _time_graph(fn)   # the kernel alone: the eager figure carries the host's launch time
        ops.check_status(dev)
        kv_bytes = pages * 2 * hkv * 16 * d * 2
        if kind == "attn_decode":
            flops = 4.0 * batch * hq * ctx * d
        else:
            flops = 4.0 * batch * hq * d * (ctx * (ctx + 1) / 2)
        byt = kv_bytes + 2 * t * hq * d * 2
        roof_ms = max(flops / (tf * 1e12), byt / (hbm * 1e9)) * 1e3
        rec = {"kernel": kind, "batch": batch, "ctx": ctx, "hq": hq, "hkv": hkv, "ms_median": round(med, 4),
               "ms_best": round(best, 4), "tflops": round(flops / med / 1e9, 1),
               "gbs": round(byt / med / 1e6, 1), "frac_of_roofline": round(roof_ms / med, 3), "ms_in_graph": round(in_graph, 4),
               "frac_of_roofline_in_graph": round(roof_ms / in_graph, 3), "peaks": how}
        print(json.dumps(rec), flush=True)
        out.append(rec)
        del kv, q
    return out
