"""Paged radix tree over token sequences (the native class behind the prefix cache), under the module
path the reference uses (``python/mlc_llm/serve/radix_tree.py``: ``match``, ``add``, ``remove``,
``extend``, ``rollback``, ``fork``, ``get``, ``get_length``, ``free_capacity``)."""

from .._core import PagedRadixTree

__all__ = ["PagedRadixTree"]
