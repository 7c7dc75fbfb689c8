"""HTTP server plumbing: the per-process registry of engines and a subprocess launcher."""
from .popen_server import PopenServer
from .server_context import ServerContext

__all__ = ["PopenServer", "ServerContext"]
