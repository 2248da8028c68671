"""The host runtime under ThreadSanitizer and AddressSanitizer: a stand-alone driver of the scheduler, its handler threads,
run-ahead, replica add / remove and an injected task failure, all against the fake executor (no GPU); and the JPEG decoder
fed truncated and corrupted files from several threads."""
import subprocess

import pytest

from crossbow_b200.ops import build


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_runtime_selftest_is_clean(sanitizer, tmp_path):
    args = []
    try:                                                        # two small JPEG files for the decoder scenario
        import io
        import numpy as np
        from PIL import Image
        g = np.random.default_rng(0)
        img = (np.kron(g.random((6, 8, 3)), np.ones((8, 8, 1))) * 255).astype(np.uint8)
        for name, kw in (("seq.jpg", {}), ("prog.jpg", {"progressive": True})):
            Image.fromarray(img).save(tmp_path / name, format="JPEG", quality=85, **kw)
            args.append(str(tmp_path / name))
    except ImportError:
        pass
    try:
        exe = build.build_rt_selftest(sanitizer)
    except RuntimeError as e:                                   # a toolchain without that sanitizer's run-time library
        pytest.skip(f"cannot build with -fsanitize={sanitizer}: {str(e)[-200:]}")
    r = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "SELFTEST_OK" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])
    assert "Sanitizer" not in r.stderr, r.stderr[-3000:]
