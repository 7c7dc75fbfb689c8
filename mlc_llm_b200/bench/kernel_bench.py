"""Device-timed micro-benchmarks of the hot kernels, reported against measured peaks.

``python -m mlc_llm_b200.bench.kernel_bench [gemm|gemm_q4|attn_decode|attn_prefill|all] [--small]``

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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="?", default="all")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    res = []
    if args.which in ("gemm", "all"):
        res += bench_gemm(args.small, q4=False)
    if args.which in ("gemm_q4", "all"):
        res += bench_gemm(args.small, q4=True)
    if args.which in ("attn_decode", "attn_prefill", "all"):
        try:
            from .attn_bench import bench_attention  # pylint: disable=import-outside-toplevel

            res += bench_attention(args.which, args.small)
        except ImportError:
            pass
    if args.out:
        with open(args.out, "w", encoding="utf-8") as f:
            json.dump(res, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
