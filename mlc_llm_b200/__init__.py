"""B200-native LLM serving framework with the API surface and artifact formats of MLC LLM."""

__version__ = "0.1.0"

from . import build as _build

_build.build_core()  # no-op when the in-tree extension is current


def __getattr__(name):
    # heavy submodules are imported on first use
    if name in ("MLCEngine", "AsyncMLCEngine"):
        from .serve import engine as _engine

        return getattr(_engine, name)
    if name in ("EngineConfig",):
        from .serve.config import EngineConfig

        return EngineConfig
    raise AttributeError(name)
