"""Row-parallel GEMM with the all-reduce + residual + RMSNorm tail (``FusedCollectives.gemm_ar_norm``)
against the plain GEMM of the same shape, device-timed, max over ranks.

``torchrun --nproc-per-node N -m mlc_llm_b200.bench.fused_ar_bench [--hidden 4096 --mode ar]``

Per shape it reports the fused kernel's time, the plain local GEMM's time (what is left when the
collective, the residual add and the norm are taken out) and the fraction of the fused path's roofline:
the slower of the GEMM FLOPs at the measured tensor peak and the bytes a rank must receive over NVLink
((N - 1) / N of the partial sums) at the measured per-direction link bandwidth.  ``MLCB_MULTIMEM=0``
switches the tail from ``multimem.ld_reduce`` to plain peer loads; ``--mode rs`` times the
reduce-scatter / all-gather pair of kernels instead.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from .. import ops, parallel, quantization as Q
from ..ops import _lib
from ..parallel.fused import FusedCollectives
from .kernel_bench import _peaks

NVLINK_GBS = 770.0  # measured peer copy bandwidth per direction per GPU


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--mode", default="ar", choices=["ar", "rs"])
    ap.add_argument("--quant", default="q4f16_1", choices=["q4f16_1", "q0f16", "q0bf16"])
    args = ap.parse_args(argv)
    rank, world, local = parallel.env_world()
    comm = parallel.Communicator(tp_size=world, pp_size=1)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    quant = Q.get(args.quant)
    dt = quant.torch_dtype
    _, tflops, how = _peaks()
    fc = FusedCollectives(args.hidden, dt, 8192, dev, group=comm.tp_group if world > 1 else None, world_size=world,
                          mode=args.mode)
    torch.manual_seed(0)
    shapes = [(256, args.hidden // world), (256, args.inter // world), (2048, args.inter // world),
              (8192, args.inter // world)]
    for m, k in shapes:
        x = (torch.randn(m, k, device=dev) * 0.5).to(dt)
        w = (torch.randn(args.hidden, k, device=dev) * 0.02).to(dt)
        if quant.kind == "group-quant":
            qw, qs = Q.group_quantize(w.cpu(), quant)
            lw = ops.LinearWeight("q4", qw, qs, None, quant, args.hidden, k).to(dev)
        else:
            lw = ops.dense_weight(w)
        nw = torch.ones(args.hidden, device=dev, dtype=dt)
        r0 = torch.zeros(m, args.hidden, device=dev, dtype=dt)

        def forward(n):
            fc.begin(m)
            fc.scatter_residual(r0)
            for _ in range(n):
                if args.mode == "ar":
                    fc.gemm_ar_norm(x, lw, nw, 1e-5)
                else:
                    fc.gemm_rs_norm(x, lw, nw, 1e-5)
            if args.mode != "ar":
                fc.wait_gather()
            fc.end()

        forward(4)
        ops.linear(x, lw)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        reps = 20
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        forward(reps)
        e.record()
        torch.cuda.synchronize()
        fused_us = comm.max_over_ranks(s.elapsed_time(e) / reps * 1e3)
        s.record()
        for _ in range(reps):
            ops.linear(x, lw)
        e.record()
        torch.cuda.synchronize()
        plain_us = comm.max_over_ranks(s.elapsed_time(e) / reps * 1e3)
        flops = 2.0 * m * args.hidden * k
        link_bytes = (world - 1) / world * m * args.hidden * 2
        roof_us = max(flops / (tflops * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e6
        if rank == 0:
            print(json.dumps({"tokens": m, "N": args.hidden, "K_per_rank": k, "world": world, "mode": args.mode,
                              "multimem": bool(getattr(fc, "multimem", False)), "fused_us": round(fused_us, 1),
                              "plain_gemm_us": round(plain_us, 1), "roofline_us": round(roof_us, 1),
                              "frac_of_roofline": round(roof_us / fused_us, 3), "peaks": how}), flush=True)
    _lib.check_status(dev)
    comm.barrier()
    comm.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
