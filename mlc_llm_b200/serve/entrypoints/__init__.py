"""FastAPI routers of the REST server."""
from . import debug_entrypoints, metrics_entrypoints, microserving_entrypoints, openai_entrypoints

__all__ = ["debug_entrypoints", "metrics_entrypoints", "microserving_entrypoints", "openai_entrypoints"]
