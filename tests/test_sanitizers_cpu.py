"""The native serving runtime under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer.

``csrc/selftest/runtime_selftest.cc`` drives the paged KV manager, the radix tree, the prefix cache and a full
engine (deterministic in-process model, four client threads adding and aborting requests against the two
background loops of the threaded engine) and checks every finished request's tokens; the sanitizers turn any
out-of-bounds access, use after free, leak, undefined operation or data race on the way into a failure."""
import os
import subprocess

import pytest

from mlc_llm_b200 import build


@pytest.mark.parametrize("sanitizer", ["address", "thread"])
def test_runtime_selftest_is_clean(sanitizer):
    try:
        exe = build.build_selftest(sanitizer)
    except FileNotFoundError as err:
        pytest.skip(str(err))
    env = dict(os.environ)
    env.pop("LD_PRELOAD", None)
    env["ASAN_OPTIONS"] = "detect_leaks=1:abort_on_error=0"
    env["UBSAN_OPTIONS"] = "print_stacktrace=1:halt_on_error=1"
    env["TSAN_OPTIONS"] = "halt_on_error=1"
    for seed in ("1", "7"):
        out = subprocess.run([str(exe), seed], capture_output=True, text=True, timeout=600, env=env)
        assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-6000:])
        assert "selftest ok" in out.stdout
        assert "Sanitizer" not in out.stderr, out.stderr[-6000:]
