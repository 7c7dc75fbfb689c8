"""``mlc_llm_b200 router`` (reference: ``python/mlc_llm/cli/router.py``)."""
import argparse

from ..interface.router import serve


def main(argv=None):
    p = argparse.ArgumentParser("mlc_llm_b200 router")
    p.add_argument("model", type=str)
    p.add_argument("--model-lib", type=str, default=None)
    p.add_argument("--router-mode", type=str, choices=["disagg", "round-robin"], default="disagg")
    p.add_argument("--router-host", type=str, default="127.0.0.1")
    p.add_argument("--router-port", type=int, default=8000)
    p.add_argument("--endpoint-hosts", type=str, nargs="+", required=True)
    p.add_argument("--endpoint-ports", type=int, nargs="+", required=True)
    p.add_argument("--endpoint-num-gpus", type=int, nargs="+", required=True)
    p.add_argument("--enable-prefix-cache", action="store_true")
    p.add_argument("--pd-balance-factor", type=float, default=0.0)
    p.add_argument("--device", type=str, default="cuda")
    a = p.parse_args(argv)
    serve(a.model, a.model_lib, a.router_host, a.router_port, a.endpoint_hosts, a.endpoint_ports,
          a.endpoint_num_gpus, a.enable_prefix_cache, a.router_mode, a.pd_balance_factor, device=a.device)


if __name__ == "__main__":
    main()
