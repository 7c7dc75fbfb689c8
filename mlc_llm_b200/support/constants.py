"""Environment-driven constants (reference: ``python/mlc_llm/support/constants.py:80-88``)."""
import os
from pathlib import Path


def _bool_env(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v.lower() in ("1", "true", "yes", "on")


def _home() -> Path:
    explicit = os.environ.get("MLC_LLM_HOME")
    if explicit:
        p = Path(explicit)
    else:
        p = Path(os.environ.get("XDG_CACHE_HOME", Path.home() / ".cache")) / "mlc_llm"
    return p


def _policy() -> str:
    v = os.environ.get("MLC_DOWNLOAD_CACHE_POLICY", "ON")
    if v not in ("ON", "OFF", "REDO", "READONLY"):
        raise ValueError(f"MLC_DOWNLOAD_CACHE_POLICY={v!r}; expected ON, OFF, REDO or READONLY")
    return v


MLC_LLM_HOME = _home()
MLC_TEMP_DIR = os.environ.get("MLC_TEMP_DIR")
MLC_MULTI_ARCH = os.environ.get("MLC_MULTI_ARCH")
MLC_JIT_POLICY = os.environ.get("MLC_JIT_POLICY", "ON")
MLC_DOWNLOAD_CACHE_POLICY = _policy()
MLC_LLM_READONLY_WEIGHT_CACHE = os.environ.get("MLC_LLM_READONLY_WEIGHT_CACHE")
MLC_DEBUG = _bool_env("MLC_DEBUG")
