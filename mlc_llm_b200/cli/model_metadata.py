"""``mlc_llm_b200 model_metadata <model-lib.json | model dir>``: show the metadata ``compile`` records
(parameters, memory estimate, KV layout) (reference: ``python/mlc_llm/cli/model_metadata.py``)."""
import argparse
import json
import os

from .. import quantization as Q
from ..interface.compile import model_metadata
from ..models import config as model_config


def _load(path: str) -> dict:
    if os.path.isdir(path):
        with open(os.path.join(path, "mlc-chat-config.json"), encoding="utf-8") as f:
            chat = json.load(f)
        cfg = model_config.from_dict(chat["model_type"], chat["model_config"])
        return model_metadata(cfg, Q.get(chat["quantization"]))
    with open(path, encoding="utf-8") as f:
        return json.load(f)


def main(argv=None):
    p = argparse.ArgumentParser("mlc_llm_b200 model_metadata")
    p.add_argument("model_lib", type=str)
    p.add_argument("--mlc-chat-config", type=str, default=None)
    p.add_argument("--print-memory-usage-in-mb", action="store_true")
    p.add_argument("--print-kv-cache-metadata", action="store_true")
    a = p.parse_args(argv)
    meta = _load(a.model_lib)
    if a.print_memory_usage_in_mb:
        print(f"params: {meta['memory_usage']['params_bytes'] / 2**20:.2f} MB")
    elif a.print_kv_cache_metadata:
        print(json.dumps(meta["kv_cache"], indent=2))
    else:
        brief = dict(meta)
        brief["params"] = f"<{len(meta['params'])} tensors>"
        print(json.dumps(brief, indent=2))


if __name__ == "__main__":
    main()
