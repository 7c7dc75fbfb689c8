"""JSON-in / JSON-out engine (native ``JsonFFIEngine``)."""
from .engine import JSONFFIEngine

__all__ = ["JSONFFIEngine"]
