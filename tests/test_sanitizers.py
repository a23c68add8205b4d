"""The native runtime's concurrency stress program under ThreadSanitizer and AddressSanitizer
(host only; the reference has no sanitizer runs, its safety comes from Rust ownership --
here the C++ runtime is checked dynamically instead)."""
import shutil
import subprocess

import pytest

from monarch_b200 import _build


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_runtime_stress_is_clean(sanitizer):
    if shutil.which(_build.CXX) is None:
        pytest.skip("no C++ compiler")
    try:
        exe = _build.build_runtime_stress(sanitizer)
    except Exception as e:  # noqa: BLE001 - e.g. the sanitizer runtime is not installed
        pytest.skip(f"cannot build with -fsanitize={sanitizer}: {e}")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-500:], r.stderr[-4000:])
    assert "runtime_stress: all ok" in r.stdout
    assert "Sanitizer" not in r.stderr, r.stderr[-4000:]
