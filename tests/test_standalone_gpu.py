"""The torch-free attention check binary (CPU fp32 reference inside the program) builds and passes on the GPU."""

import subprocess

import pytest

pytestmark = pytest.mark.gpu


def test_standalone_attention_check_passes():
    from astrai_b200.ops.build import build_standalone

    exe = build_standalone()
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert "all checks passed" in proc.stdout and "FAIL" not in proc.stdout
