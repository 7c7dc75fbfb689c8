"""``mlc_llm_b200 chat`` (reference: ``python/mlc_llm/cli/chat.py``)."""
import argparse

from ..interface.chat import ChatCompletionOverride, chat


def main(argv=None):
    p = argparse.ArgumentParser("mlc_llm_b200 chat")
    p.add_argument("model", type=str)
    p.add_argument("--device", type=str, default="auto")
    p.add_argument("--model-lib", type=str, default=None)
    p.add_argument("--overrides", type=ChatCompletionOverride.from_str, default=None)
    a = p.parse_args(argv)
    chat(a.model, a.device, a.model_lib, a.overrides)


if __name__ == "__main__":
    main()
