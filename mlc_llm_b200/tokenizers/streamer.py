"""``TextStreamer`` and ``StopStrHandler`` under the module path the reference uses
(``python/mlc_llm/tokenizers/streamer.py``)."""

from . import StopStrHandler, TextStreamer

__all__ = ["TextStreamer", "StopStrHandler"]
