"""Fused tensor-parallel kernels against the NCCL baseline, device-timed, max over ranks.

``torchrun --nproc-per-node N -m mlc_llm_b200.bench.fused_bench [--hidden 4096 --inter 14336]``

Per token count it times one transformer-block worth of tensor-parallel linears:
  baseline:  o_proj GEMM, NCCL all-reduce, add+RMSNorm, gate_up GEMM
  fused:     o_proj GEMM with reduce-scatter epilogue + residual + RMSNorm + all-gather tail,
             gate_up GEMM with all-gather prologue
and reports the fused path's fraction of its roofline: the slower of the GEMM FLOPs at the measured
tensor peak and the bytes that must cross NVLink at the measured per-direction link bandwidth.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import ops, quantization as Q
from ..parallel.fused import FusedCollectives
from .kernel_bench import _peaks

NVLINK_GBS = 770.0  # measured peer copy bandwidth per direction per GPU


def _timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    times = []
    for _ in range(iters):
        flush.add_(1)
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    t = torch.tensor([sorted(times)[len(times) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--heads-dim", type=int, default=4096, help="attention context width (hq * d)")
    ap.add_argument("--quant", default="q0f16")
    ap.add_argument("--tokens", type=int, nargs="*", default=[256, 2048, 8192])
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    quant = Q.get(args.quant)
    dt = quant.torch_dtype
    hbm, tf, how = _peaks()
    torch.manual_seed(1)
    k_o = args.heads_dim // world
    n_up = 2 * args.inter // world

    def mk(n, k):
        w = (torch.randn(n, k, device=dev) * 0.02).to(dt)
        if quant.kind == "no-quant":
            return ops.dense_weight(w)
        qw, qs = Q.group_quantize(w.cpu(), quant)
        return ops.LinearWeight("q4", qw, qs, None, quant, n, k).to(dev)

    l_o, l_up = mk(args.hidden, k_o), mk(n_up, args.hidden)
    nw = torch.ones(args.hidden, dtype=dt, device=dev)
    flush = torch.zeros(160 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)
    fc = FusedCollectives(args.hidden, dt, max(args.tokens), dev, group=dist.group.WORLD, world_size=world)
    results = []
    for t in args.tokens:
        x = (torch.randn(t, k_o, device=dev) * 0.5).to(dt)
        res = (torch.randn(t, args.hidden, device=dev) * 0.5).to(dt)

        def baseline():
            o = ops.linear(x, l_o)
            dist.all_reduce(o)
            h = ops.add_rmsnorm(o, res, nw, 1e-5)
            return ops.linear(h, l_up)

        def fused():
            fc.gemm_rs_norm(x, l_o, nw, 1e-5)
            return fc.gemm_ag(l_up)

        def rs_only():
            fc.gemm_rs_norm(x, l_o, nw, 1e-5)
            fc.wait_gather()

        def gemms_only():
            o = ops.linear(x, l_o)
            return ops.linear(o, l_up)

        fc.begin(t)
        fc.scatter_residual(res)
        ms_base = _timed(baseline, 10, 3, flush)
        ms_fused = _timed(fused, 10, 3, flush)
        ms_rs = _timed(rs_only, 10, 3, flush)
        ms_gemm = _timed(gemms_only, 10, 3, flush)
        ops.check_status(dev)
        flops = 2.0 * t * (args.hidden * k_o + n_up * args.hidden)
        # every rank sends (world-1)/world of its partial sums and of its normalised rows
        nvl_bytes = 2.0 * t * args.hidden * 2 * (world - 1) / world
        roof_ms = max(flops / (tf * 1e12), nvl_bytes / (NVLINK_GBS * 1e9)) * 1e3
        rec = {"tokens": t, "world": world, "quant": args.quant, "ms_nccl_path": round(ms_base, 4),
               "ms_fused_path": round(ms_fused, 4), "ms_rs_kernel_plus_wait": round(ms_rs, 4),
               "ms_two_gemms_no_comm": round(ms_gemm, 4), "speedup_vs_nccl": round(ms_base / ms_fused, 3),
               "roofline_ms": round(roof_ms, 4), "frac_of_roofline": round(roof_ms / ms_fused, 3), "peaks": how}
        results.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w", encoding="utf-8") as f:
            json.dump(results, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
