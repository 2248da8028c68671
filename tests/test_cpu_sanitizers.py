"""The host runtime under ThreadSanitizer and AddressSanitizer: a stand-alone driver of the scheduler, its handler threads,
run-ahead, replica add / remove and an injected task failure, all against the fake executor (no GPU)."""
import subprocess

import pytest

from crossbow_b200.ops import build


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_runtime_selftest_is_clean(sanitizer):
    try:
        exe = build.build_rt_selftest(sanitizer)
    except RuntimeError as e:                                   # a toolchain without that sanitizer's run-time library
        pytest.skip(f"cannot build with -fsanitize={sanitizer}: {str(e)[-200:]}")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "SELFTEST_OK" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])
    assert "Sanitizer" not in r.stderr, r.stderr[-3000:]
