"""Device-timed micro-benchmarks of the hot kernels, reported against measured peaks.

``python -m mlc_llm_b200.bench.kernel_bench [gemm|gemm_q4|gemm_fp8|gemv_q4|lowm_q4|attn_decode|attn_prefill|rope|norm|sampling|moe|all] [--small]``

Timing follows the usual hygiene: warm-up, CUDA events on the launching stream, and a buffer larger
than L2 written between timed launches so every launch starts cold.  ``--small`` shrinks the
problem (a few hundred MB) so the same command can be run under a profiler.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from .. import ops, quantization as Q


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path, encoding="utf-8") as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0]


def _time_graph(fn, reps: int = 5, replays: int = 3) -> float:
    """Milliseconds per call with the host out of the picture: ``reps`` calls captured in one CUDA graph,
    replayed ``replays`` times between two events.  For kernels of a few tens of microseconds the eager
    figure of :func:`_time` includes the time the host needs to issue the launch."""
    fn()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(reps):
                fn()
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / (reps * replays)


def bench_gemm(small: bool, q4: bool):
    dev = torch.device("cuda")
    hbm, tf, how = _peaks()
    flush = torch.zeros(160 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)
    shapes = [(256, 6144, 4096), (256, 28672, 4096), (256, 4096, 14336), (8192, 6144, 4096),
              (8192, 28672, 4096), (8192, 4096, 14336), (16, 28672, 4096), (1, 28672, 4096)]
    if small:
        shapes = [(256, 28672, 4096), (2048, 6144, 4096)]
    out = []
    quant = Q.get("q4f16_1")
    for m, n, k in shapes:
        x = (torch.randn(m, k, device=dev) * 0.5).half()
        if q4:
            qw = torch.randint(-2**31, 2**31 - 1, (n, k // 8), dtype=torch.int64, device=dev).to(torch.int32)
            qs = (torch.rand(n, k // 32, device=dev) * 0.01).half()
            lw = ops.LinearWeight("q4", qw, qs, None, quant, n, k, device_layout=True)
            wbytes = n * k // 2 + n * (k // 32) * 2
        else:
            lw = ops.dense_weight((torch.randn(n, k, device=dev) * 0.02).half())
            wbytes = n * k * 2
        med, best = _time(lambda: ops.linear(x, lw), flush=flush)
        ops.check_status(dev)
        flops = 2.0 * m * n * k
        byt = wbytes + m * k * 2 + m * n * 2
        roof_ms = max(flops / (tf * 1e12), byt / (hbm * 1e9)) * 1e3
        out.append({"kernel": "gemm_q4" if q4 else "gemm_f16", "M": m, "N": n, "K": k,
                    "ms_median": round(med, 4), "ms_best": round(best, 4),
                    "tflops": round(flops / med / 1e9, 1), "gbs": round(byt / med / 1e6, 1),
                    "frac_of_roofline": round(roof_ms / med, 3), "peaks": how})
        print(json.dumps(out[-1]), flush=True)
        if not q4:
            w = lw.w
            med_t, _ = _time(lambda: torch.matmul(x, w.t()), flush=flush)
            print(json.dumps({"kernel": "cublas_f16", "M": m, "N": n, "K": k, "ms_median": round(med_t, 4),
                              "tflops": round(flops / med_t / 1e9, 1)}), flush=True)
    return out


def bench_gemv_q4(small: bool):
    """One to four tokens against int4-group weights: the CUDA-core GEMV (``mlcb_gemv_q4``) and, for the
    same shapes, the tensor-core kernel it replaces (MLCB_GEMV_Q4=0 path), both against the HBM roofline."""
    dev = torch.device("cuda")
    hbm, _tf, how = _peaks()
    flush = torch.zeros(160 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)
    shapes = [(1, 6144, 4096), (1, 28672, 4096), (1, 4096, 14336), (1, 128256, 4096), (2, 28672, 4096),
              (4, 28672, 4096)]
    if small:
        shapes = [(1, 128256, 4096)]
    quant = Q.get("q4f16_1")
    out = []
    for m, n, k in shapes:
        x = (torch.randn(m, k, device=dev) * 0.5).half()
        qw = torch.randint(-2**31, 2**31 - 1, (n, k // 8), dtype=torch.int64, device=dev).to(torch.int32)
        qs = (torch.rand(n, k // 32, device=dev) * 0.01).half()
        lw = ops.LinearWeight("q4", qw, qs, None, quant, n, k, device_layout=True)
        byt = n * k // 2 + n * (k // 32) * 2 + m * k * 2 + m * n * 2
        try:
            set_form = ops.lib().mlcb_gemv_set_form
            variants = (("gemv_q4_split_k", True, 2), ("gemv_q4_row_per_warp", True, 1),
                        ("gemm_q4_tensor_core", False, 0))
        except AttributeError:  # library built before the second form existed
            set_form = None
            variants = (("gemv_q4", True, 0), ("gemm_q4_tensor_core", False, 0))
        for name, flag, form in variants:
            ops._GEMV_Q4 = flag  # pylint: disable=protected-access
            if set_form is not None and form:
                set_form(form)
            med, best = _time(lambda: ops.linear(x, lw), flush=flush)
            ops.check_status(dev)
            rec = {"kernel": name, "M": m, "N": n, "K": k, "ms_median": round(med, 4), "ms_best": round(best, 4),
                   "gbs": round(byt / med / 1e6, 1), "frac_of_roofline": round(byt / (hbm * 1e9) * 1e3 / med, 3),
                   "peaks": how}
            print(json.dumps(rec), flush=True)
            out.append(rec)
        ops._GEMV_Q4 = True  # pylint: disable=protected-access
        if set_form is not None:
            set_form(2)
    return out


def bench_lowm_q4(small: bool):
    """Five to sixteen tokens against int4-group weights: the warp-level MMA form (``mlcb_gemm_q4_lowm``) and the
    tcgen05 kernel on the same shapes."""
    dev = torch.device("cuda")
    hbm, _tf, how = _peaks()
    flush = torch.zeros(160 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)
    shapes = [(8, 6144, 4096), (8, 28672, 4096), (8, 4096, 14336), (16, 28672, 4096), (16, 4096, 14336)]
    if small:
        shapes = [(8, 28672, 4096)]
    quant = Q.get("q4f16_1")
    out = []
    for m, n, k in shapes:
        x = (torch.randn(m, k, device=dev) * 0.5).half()
        qw = torch.randint(-2**31, 2**31 - 1, (n, k // 8), dtype=torch.int64, device=dev).to(torch.int32)
        qs = (torch.rand(n, k // 32, device=dev) * 0.01).half()
        lw = ops.LinearWeight("q4", qw, qs, None, quant, n, k, device_layout=True)
        byt = n * k // 2 + n * (k // 32) * 2 + m * k * 2 + m * n * 2
        saved = ops._LOWM_Q4  # pylint: disable=protected-access
        for name, flag in (("gemm_q4_lowm_mma", True), ("gemm_q4_tensor_core", False)):
            ops._LOWM_Q4 = flag  # pylint: disable=protected-access
            med, best = _time(lambda: ops.linear(x, lw), flush=flush)
            ops.check_status(dev)
            rec = {"kernel": name, "M": m, "N": n, "K": k, "ms_median": round(med, 4), "ms_best": round(best, 4),
                   "gbs": round(byt / med / 1e6, 1), "frac_of_roofline": round(byt / (hbm * 1e9) * 1e3 / med, 3),
                   "peaks": how}
            print(json.dumps(rec), flush=True)
            out.append(rec)
        ops._LOWM_Q4 = saved  # pylint: disable=protected-access
    return out


def bench_misc(which: str, small: bool):
    """Memory-bound helpers: RoPE + KV append, add+RMSNorm, sampling; and the MoE grouped GEMM."""
    dev = torch.device("cuda")
    hbm, tf, how = _peaks()
    out = []

    def rec(name, med, byt, flops=0.0, **extra):
        roof = max(byt / (hbm * 1e9), flops / (tf * 1e12)) * 1e3
        r = {"kernel": name, "ms_median": round(med, 4), "gbs": round(byt / med / 1e6, 1),
             "tflops": round(flops / med / 1e9, 1), "frac_of_roofline": round(roof / med, 3), "peaks": how}
        r.update(extra)
        print(json.dumps(r), flush=True)
        out.append(r)

    flush = torch.zeros(160 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)
    if which in ("rope", "all"):
        t, hq, hkv, d = (8192 if small else 65536), 32, 8, 128
        qkv = (torch.randn(t, (hq + 2 * hkv) * d, device=dev) * 0.5).half()
        pages = t // 16 + 1
        kv = torch.zeros(pages, 2, hkv, 16, d, dtype=torch.float16, device=dev)
        pos = torch.arange(t, dtype=torch.int32, device=dev) % 4096
        slot = torch.arange(t, dtype=torch.int32, device=dev)
        inv = ops.reference.rope_inv_freq(d, 5e5).to(dev)
        med, _ = _time(lambda: ops.rope_append(qkv, kv, pos, slot, inv, hq, hkv, d, d, 16), flush=flush)
        # q and k are read and rewritten, v is read, k and v are written to their pages
        byt = t * d * 2 * (2 * (hq + hkv) + hkv + 2 * hkv)
        rec("rope_append", med, byt, tokens=t)
    if which in ("norm", "all"):
        t, h = (8192 if small else 65536), 4096
        x = torch.randn(t, h, device=dev).half()
        res = torch.randn(t, h, device=dev).half()
        w = torch.ones(h, device=dev).half()
        med, _ = _time(lambda: ops.add_rmsnorm(x, res, w, 1e-5), flush=flush)
        rec("add_rmsnorm", med, t * h * 2 * 4, tokens=t)
    if which in ("sampling", "all"):
        n, v = (64 if small else 256), 128256
        logits = torch.randn(n, v, device=dev)
        temp = torch.full((n,), 0.8, device=dev)
        u = torch.rand(n, device=dev)
        top_p = torch.full((n,), 0.9, device=dev)
        top_k = torch.full((n,), 50, dtype=torch.int32, device=dev)
        med, _ = _time(lambda: ops.softmax_temperature(logits, temp), flush=flush)
        rec("softmax_temperature", med, n * v * 4 * 2, rows=n)
        probs = ops.softmax_temperature(logits, temp)
        med, _ = _time(lambda: ops.sample(probs, None, u, top_p, top_k), flush=flush)
        rec("sample_top_p_top_k", med, n * v * 4, rows=n)
    if which in ("moe", "all"):
        e, k, h, inter = 8, 2, 4096, 14336
        t = 1024 if small else 8192
        x = (torch.randn(t, h, device=dev) * 0.5).half()
        gate = torch.randn(t, e, device=dev).half()
        w13 = ops.LinearWeight("dense", (torch.randn(e, 2 * inter, h, device=dev) * 0.02).half(), None, None,
                               None, 2 * inter, h)
        wts, idx = ops.moe_router(gate, k, True)
        off, spos, src = ops.moe_permute(idx, e)
        xp = ops.row_gather(x, src)
        med, _ = _time(lambda: ops.grouped_linear(xp, w13, off), flush=flush)
        rec("moe_grouped_gemm", med, e * 2 * inter * h * 2 + t * k * (h + 2 * inter) * 2,
            2.0 * t * k * 2 * inter * h, tokens=t, experts=e, top_k=k)
    return out


def bench_gemm_fp8(small: bool):
    """Block-scaled e4m3 weights: fp8 x fp8 tensor-core product with on-the-fly activation quantisation
    (W8A8), the same weights expanded inside the 16-bit GEMM (W8A16), this package's bf16 GEMM and cuBLAS
    bf16 on the same shape. Graph-timed (host out of the picture); operands exceed L2 on the large shapes."""
    from ..ops import fp8 as f8  # pylint: disable=import-outside-toplevel

    dev = torch.device("cuda")
    _, tf, how = _peaks()
    quant = Q.get("fp8_e4m3fn_bf16_block_scale")
    shapes = [(8192, 10240, 8192), (8192, 8192, 3584), (2048, 8192, 8192), (512, 8192, 8192), (256, 8192, 8192)]
    if small:
        shapes = [(2048, 8192, 8192)]
    out = []
    for m, n, k in shapes:
        x = (torch.randn(m, k, device=dev) * 0.5).bfloat16()
        w = torch.randn(n, k, device=dev) * 0.05
        qw, sc = Q.fp8_block_quantize(w, (128, 128), "float8_e4m3fn")
        lw = ops.LinearWeight("fp8_block", qw, sc.float(), None, quant, n, k)
        ld = ops.dense_weight(w.bfloat16())
        del w
        t_a8 = _time_graph(lambda: ops.linear(x, lw)) * 1e3
        t_q = _time_graph(lambda: f8.act_quant_fp8(x)) * 1e3
        keep = f8._FP8_ACT  # pylint: disable=protected-access
        f8._FP8_ACT = False  # pylint: disable=protected-access
        t_a16 = _time_graph(lambda: ops.linear(x, lw)) * 1e3
        f8._FP8_ACT = keep  # pylint: disable=protected-access
        t_bf = _time_graph(lambda: ops.linear(x, ld)) * 1e3
        t_cb = _time_graph(lambda: torch.matmul(x, ld.w.t())) * 1e3
        ops.check_status(dev)
        flops = 2.0 * m * n * k
        out.append({"kernel": "gemm_fp8_w8a8", "M": m, "N": n, "K": k, "us": round(t_a8, 1),
                    "of_which_act_quant_us": round(t_q, 1), "w8a16_us": round(t_a16, 1), "own_bf16_us": round(t_bf, 1),
                    "cublas_bf16_us": round(t_cb, 1), "tflops": round(flops / t_a8 / 1e6, 1),
                    "frac_of_bf16_peak": round(flops / t_a8 / 1e6 / tf, 3), "vs_own_bf16": round(t_bf / t_a8, 2),
                    "vs_w8a16": round(t_a16 / t_a8, 2), "peaks": how})
        print(json.dumps(out[-1]), flush=True)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="?", default="all")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    res = []
    if args.which in ("gemm", "all"):
        res += bench_gemm(args.small, q4=False)
    if args.which in ("gemm_fp8", "all"):
        res += bench_gemm_fp8(args.small)
    if args.which in ("gemv_q4", "all"):
        bench_gemv_q4(args.small)
    if args.which in ("lowm_q4", "all"):
        bench_lowm_q4(args.small)
    if args.which in ("gemm_q4", "all"):
        res += bench_gemm(args.small, q4=True)
    if args.which in ("attn_decode", "attn_prefill", "all"):
        try:
            from .attn_bench import bench_attention  # pylint: disable=import-outside-toplevel

            res += bench_attention(args.which, args.small)
        except ImportError:
            pass
    if args.which in ("rope", "norm", "sampling", "moe", "all"):
        res += bench_misc(args.which, args.small)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as f:
            json.dump(res, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
