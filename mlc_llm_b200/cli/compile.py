"""``mlc_llm_b200 compile`` (reference: ``python/mlc_llm/cli/compile.py``)."""
import argparse

from ..interface.compile import compile_model
from ..models.config import SUPPORTED_MODEL_TYPES
from ..quantization import QUANTIZATION


def _overrides(text: str):
    out = {}
    for item in filter(None, (x.strip() for x in text.split(";"))):
        k, v = item.split("=", 1)
        out[k.strip()] = int(v)
    return out


def main(argv=None):
    p = argparse.ArgumentParser("mlc_llm_b200 compile")
    p.add_argument("model", type=str)
    p.add_argument("--quantization", type=str, default=None, choices=sorted(QUANTIZATION))
    p.add_argument("--model-type", type=str, default="auto", choices=["auto"] + SUPPORTED_MODEL_TYPES)
    p.add_argument("--device", type=str, default="cuda")
    p.add_argument("--host", type=str, default="auto")
    p.add_argument("--opt", type=str, default="O2")
    p.add_argument("--system-lib-prefix", type=str, default="auto")
    p.add_argument("--output", "-o", type=str, required=True)
    p.add_argument("--overrides", type=_overrides, default={})
    p.add_argument("--debug-dump", type=str, default=None)
    a = p.parse_args(argv)
    quant = a.quantization
    if quant is None:
        import json
        import os

        path = a.model if a.model.endswith(".json") else os.path.join(a.model, "mlc-chat-config.json")
        with open(path, encoding="utf-8") as f:
            quant = json.load(f)["quantization"]
    out = compile_model(a.model, quant, a.model_type, a.device, a.opt, a.overrides, a.output)
    print(f"[compile] wrote {out}")


if __name__ == "__main__":
    main()
