"""Interception of the operator layer (``mlc_llm_b200.ops``) for debugging tools.

Every model forward goes through the functions of ``ops`` looked up at call time, so replacing the
module attributes taps every kernel launch of a step (the reference instruments the VM's call
instruction instead: ``python/mlc_llm/testing/debug_chat.py:61-145``)."""

from __future__ import annotations

import contextlib
from typing import Callable, Iterable, Optional

from .. import ops

DEFAULT_OPS = ("linear", "grouped_linear", "rmsnorm", "add_rmsnorm", "act_mul", "embed", "rope_append",
               "paged_attention", "argmax", "row_gather", "softmax_temperature", "moe_router", "moe_permute",
               "moe_combine")


@contextlib.contextmanager
def tap_ops(before: Optional[Callable] = None, after: Optional[Callable] = None,
            names: Iterable[str] = DEFAULT_OPS):
    """Within the block, call ``before(name, args, kwargs)`` ahead of, and ``after(name, args, kwargs,
    result, token)`` behind every listed operator; ``token`` is whatever ``before`` returned."""
    saved = {}
    for name in names:
        fn = getattr(ops, name, None)
        if fn is None:
            continue
        saved[name] = fn

        def wrapped(*args, _fn=fn, _name=name, **kwargs):
            token = before(_name, args, kwargs) if before is not None else None
            out = _fn(*args, **kwargs)
            if after is not None:
                after(_name, args, kwargs, out, token)
            return out

        setattr(ops, name, wrapped)
    try:
        yield
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)
