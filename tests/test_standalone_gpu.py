"""The torch-free check binaries (CPU fp32 references inside the programs) build and pass on the GPU."""

import subprocess

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which", ["attn_check", "quant_paged_check"])
def test_standalone_check_passes(which):
    from astrai_b200.ops.build import build_standalone

    exe = build_standalone(which)
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert "all checks passed" in proc.stdout and "FAIL" not in proc.stdout
