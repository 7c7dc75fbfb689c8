"""``Tokenizer`` under the module path the reference uses (``python/mlc_llm/tokenizers/tokenizers.py``)."""

from . import Tokenizer

__all__ = ["Tokenizer"]
