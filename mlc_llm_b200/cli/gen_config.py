"""``mlc_llm_b200 gen_config`` (reference: ``python/mlc_llm/cli/gen_config.py``)."""
import argparse

from ..interface.gen_config import CONV_TEMPLATES, gen_config
from ..models.config import SUPPORTED_MODEL_TYPES
from ..quantization import QUANTIZATION


def main(argv=None):
    p = argparse.ArgumentParser("mlc_llm_b200 gen_config")
    p.add_argument("config", type=str, help="preset name, model directory or config.json")
    p.add_argument("--quantization", type=str, required=True, choices=sorted(QUANTIZATION))
    p.add_argument("--model-type", type=str, default="auto", choices=["auto"] + SUPPORTED_MODEL_TYPES)
    p.add_argument("--conv-template", type=str, required=True, choices=sorted(CONV_TEMPLATES))
    p.add_argument("--context-window-size", type=int, default=None)
    p.add_argument("--sliding-window-size", type=int, default=None)
    p.add_argument("--prefill-chunk-size", type=int, default=None)
    p.add_argument("--attention-sink-size", type=int, default=None)
    p.add_argument("--tensor-parallel-shards", type=int, default=None)
    p.add_argument("--pipeline-parallel-stages", type=int, default=None)
    p.add_argument("--disaggregation", action="store_true", default=None)
    p.add_argument("--max-batch-size", type=int, default=128)
    p.add_argument("--output", "-o", type=str, required=True)
    a = p.parse_args(argv)
    path = gen_config(a.config, a.model_type, a.quantization, a.conv_template, a.context_window_size,
                      a.sliding_window_size, a.prefill_chunk_size, a.attention_sink_size,
                      a.tensor_parallel_shards, a.pipeline_parallel_stages, a.disaggregation, a.max_batch_size,
                      a.output)
    print(f"[gen_config] wrote {path}")


if __name__ == "__main__":
    main()
