"""The CPU tier under ThreadSanitizer and AddressSanitizer/UBSan: a stand-alone program (no Python in the
process) drives the thread pool, the SIMD kernels and the task pipeline, including a two-node ring over loopback."""
import shutil
import socket
import subprocess

import pytest


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("sanitizer,marker", [("thread", "WARNING: ThreadSanitizer"), ("address", "ERROR: AddressSanitizer")])
def test_cpu_tier_selftest_is_clean(sanitizer, marker, tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("no compiler")
    from stellatrain_b200 import _build

    try:
        exe = _build.build_selftest(sanitizer, out_dir=tmp_path)
    except RuntimeError as e:
        if "sanitize" in str(e) and ("cannot find" in str(e) or "unrecognized" in str(e)):
            pytest.skip("sanitizer runtime not installed")
        raise
    for _ in range(3 if sanitizer == "thread" else 1):      # races depend on the schedule: several runs
        out = subprocess.run([str(exe), str(_free_port())], capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-4000:]
        assert "selftest ok" in out.stdout
        assert marker not in out.stderr, out.stderr[-4000:]
        assert "runtime error:" not in out.stderr, out.stderr[-4000:]      # UBSan
