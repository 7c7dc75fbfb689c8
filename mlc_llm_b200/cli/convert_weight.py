"""``mlc_llm_b200 convert_weight`` (reference: ``python/mlc_llm/cli/convert_weight.py``)."""
import argparse

from ..interface.convert_weight import convert_weight
from ..models.config import SUPPORTED_MODEL_TYPES
from ..quantization import QUANTIZATION


def main(argv=None):
    p = argparse.ArgumentParser("mlc_llm_b200 convert_weight")
    p.add_argument("config", type=str, help="model directory or config.json")
    p.add_argument("--quantization", type=str, required=True, choices=sorted(QUANTIZATION))
    p.add_argument("--model-type", type=str, default="auto", choices=["auto"] + SUPPORTED_MODEL_TYPES)
    p.add_argument("--device", type=str, default="auto")
    p.add_argument("--source", type=str, default="auto")
    p.add_argument("--source-format", type=str, default="auto",
                   choices=["auto", "huggingface-torch", "huggingface-safetensor", "awq"])
    p.add_argument("--output", "-o", type=str, required=True)
    p.add_argument("--lora-adapter", type=str, default=None)
    p.add_argument("--preshard", type=int, default=0,
                   help="write tensor-parallel parameters once per rank for this many ranks")
    a = p.parse_args(argv)
    convert_weight(a.config, a.quantization, a.model_type, a.device, a.source, a.source_format, a.output,
                   a.lora_adapter, preshard=a.preshard)


if __name__ == "__main__":
    main()
