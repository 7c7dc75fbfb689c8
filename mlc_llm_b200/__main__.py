"""``python -m mlc_llm_b200 <subcommand>`` (reference: ``python/mlc_llm/__main__.py``)."""

import importlib
import sys

SUBCOMMANDS = {
    "compile": "compile", "convert_weight": "convert_weight", "gen_config": "gen_config", "chat": "chat",
    "serve": "serve", "package": "package", "calibrate": "calibrate", "router": "router", "bench": None,
    "worker": "worker", "check_device": "check_device", "model_metadata": "model_metadata",
    "delivery": "delivery",
}


def main() -> None:
    if len(sys.argv) < 2 or sys.argv[1] in ("-h", "--help") or sys.argv[1] not in SUBCOMMANDS:
        print("usage: python -m mlc_llm_b200 {" + ",".join(SUBCOMMANDS) + "} ...", file=sys.stderr)
        sys.exit(0 if len(sys.argv) > 1 and sys.argv[1] in ("-h", "--help") else 2)
    sub = sys.argv[1]
    if sub == "bench":
        from .bench.__main__ import main as bench_main  # pylint: disable=import-outside-toplevel

        bench_main(sys.argv[2:])
        return
    importlib.import_module(f".cli.{SUBCOMMANDS[sub]}", __package__).main(sys.argv[2:])


if __name__ == "__main__":
    main()
