"""Descriptor of a KV hand-off between a prefill engine and a decode engine (disaggregated serving).

The decode engine's ``prep_recv`` step answers with *where* a prefill engine may write KV rows: which
pool (an in-process registry key, or the raw 64 bytes of a CUDA IPC memory handle plus an offset) and
which token slots.  That answer travels through the router and comes back to the prefill engine inside
an HTTP request, so the prefill engine has to treat it as untrusted input:

* the format is a fixed JSON schema of numbers and short strings; nothing in it is ever unpickled or
  called;
* the payload carries an HMAC-SHA256 over its canonical form, keyed with a secret that only the
  engines of one deployment share (``MLCB_KV_HANDOFF_SECRET``, or a per-user key file created with
  mode 0600 on first use).  A payload that was not produced by a ``prep_recv`` step of such an engine,
  or that was altered on the way, is rejected before any device memory is mapped;
* slots are checked on the host against the pool's real extent (see ``ModelExecutor.send_kv``).

Reference counterpart: the structured ``kv_append_metadata`` of
``cpp/serve/engine_actions/disagg_prepare_recv.cc`` / ``disagg_remote_send.cc``.
"""

from __future__ import annotations

import base64
import hashlib
import hmac
import json
import os
import secrets
from pathlib import Path
from typing import Any, Dict, List, Optional

SCHEMA_VERSION = 2
_ALLOWED_DTYPES = ("torch.float16", "torch.bfloat16", "torch.float32", "torch.float8_e4m3fn")
_MAX_SLOTS = 1 << 22
_secret_cache: Optional[bytes] = None


class HandoffError(RuntimeError):
    """The hand-off descriptor is malformed, forged, or does not fit the pools."""


def _key_file() -> Path:
    base = os.environ.get("XDG_CACHE_HOME") or os.path.join(os.path.expanduser("~"), ".cache")
    return Path(base) / "mlc_llm_b200" / "kv_handoff.key"


def handoff_secret() -> bytes:
    """Secret shared by the engines that may hand KV rows to each other."""
    global _secret_cache  # pylint: disable=global-statement
    env = os.environ.get("MLCB_KV_HANDOFF_SECRET")
    if env:
        return env.encode("utf-8")
    if _secret_cache is not None:
        return _secret_cache
    path = _key_file()
    try:
        data = path.read_bytes()
        if len(data) >= 32:
            _secret_cache = data
            return data
    except OSError:
        pass
    path.parent.mkdir(parents=True, exist_ok=True)
    fresh = secrets.token_bytes(32)
    try:
        fd = os.open(str(path), os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o600)
        with os.fdopen(fd, "wb") as f:
            f.write(fresh)
        _secret_cache = fresh
    except FileExistsError:  # another engine of this user won the race: use its key
        _secret_cache = path.read_bytes()
    return _secret_cache


def _canonical(obj: Dict[str, Any]) -> bytes:
    return json.dumps(obj, sort_keys=True, separators=(",", ":")).encode("utf-8")


def _mac(body: Dict[str, Any]) -> str:
    return hmac.new(handoff_secret(), _canonical(body), hashlib.sha256).hexdigest()


def pool_descriptor(key: str, shape: List[int], dtype: str, device: int, handle: bytes = b"",
                    offset: int = 0) -> Dict[str, Any]:
    return {"v": SCHEMA_VERSION, "key": key, "pid": os.getpid(), "device": int(device),
            "shape": [int(x) for x in shape], "dtype": dtype,
            "handle": base64.b64encode(handle).decode("ascii"), "offset": int(offset)}


def encode_payload(pool: Dict[str, Any], slots: List[int], begin: int, end: int) -> str:
    """Signed answer of a ``prep_recv`` step (base64 of JSON)."""
    body = {"pool": pool, "slots": [int(s) for s in slots], "begin": int(begin), "end": int(end)}
    return base64.b64encode(_canonical(dict(body, mac=_mac(body)))).decode("ascii")


def _is_int(x: Any) -> bool:
    return isinstance(x, int) and not isinstance(x, bool)


def decode_payload(metadata: str) -> Dict[str, Any]:
    """Verify and parse what :func:`encode_payload` produced. Raises :class:`HandoffError` on anything
    else; never executes or deserialises objects from the input."""
    if not isinstance(metadata, str) or len(metadata) > 64 * 1024 * 1024:
        raise HandoffError("hand-off metadata must be a base64 string")
    try:
        obj = json.loads(base64.b64decode(metadata, validate=True))
    except Exception as err:  # pylint: disable=broad-except
        raise HandoffError("hand-off metadata is not base64 JSON") from err
    if not isinstance(obj, dict) or set(obj) != {"pool", "slots", "begin", "end", "mac"}:
        raise HandoffError("hand-off metadata has unexpected fields")
    mac = obj.pop("mac")
    if not isinstance(mac, str) or not hmac.compare_digest(mac, _mac(obj)):
        raise HandoffError("hand-off metadata was not issued by an engine of this deployment")
    pool, slots = obj["pool"], obj["slots"]
    if not isinstance(pool, dict) or set(pool) != {"v", "key", "pid", "device", "shape", "dtype", "handle", "offset"}:
        raise HandoffError("pool descriptor has unexpected fields")
    if pool["v"] != SCHEMA_VERSION:
        raise HandoffError(f"pool descriptor version {pool['v']!r} is not supported")
    if not isinstance(pool["key"], str) or len(pool["key"]) > 64 or not pool["key"].isalnum():
        raise HandoffError("pool key is malformed")
    if not all(_is_int(pool[k]) for k in ("pid", "device", "offset")) or pool["offset"] < 0:
        raise HandoffError("pool descriptor numbers are malformed")
    shape = pool["shape"]
    if not isinstance(shape, list) or len(shape) != 6 or not all(_is_int(x) and 0 < x < (1 << 31) for x in shape):
        raise HandoffError("pool shape is malformed")
    if pool["dtype"] not in _ALLOWED_DTYPES:
        raise HandoffError("pool dtype is not a KV dtype")
    try:
        handle = base64.b64decode(pool["handle"], validate=True) if isinstance(pool["handle"], str) else None
    except Exception as err:  # pylint: disable=broad-except
        raise HandoffError("pool handle is not base64") from err
    if handle is None or len(handle) not in (0, 64):
        raise HandoffError("pool handle must be empty or 64 bytes")
    pool = dict(pool, handle=handle)
    if not isinstance(slots, list) or len(slots) > _MAX_SLOTS or not all(_is_int(s) for s in slots):
        raise HandoffError("slot list is malformed")
    if not _is_int(obj["begin"]) or not _is_int(obj["end"]):
        raise HandoffError("window bounds are malformed")
    return {"pool": pool, "slots": slots, "begin": obj["begin"], "end": obj["end"]}


def check_slots(slots, num_pages: int, page: int, what: str) -> None:
    """Host-side range check of token slots against a pool of ``num_pages`` pages."""
    import numpy as np  # pylint: disable=import-outside-toplevel

    arr = np.asarray(slots, dtype=np.int64)
    if arr.size and (int(arr.min()) < 0 or int(arr.max()) >= num_pages * page):
        raise HandoffError(f"{what} slot outside [0, {num_pages * page})")
