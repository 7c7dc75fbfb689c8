"""Request routing over several server processes."""
from .router import Router

__all__ = ["Router"]
