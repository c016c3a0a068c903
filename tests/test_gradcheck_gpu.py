"""Runs the reference's own finite-difference test (tests/gradcheck.c, unmodified,
with its unmodified host modules) linked against this library's kernels.  The
binary is built by oracle/Makefile where the reference sources are mounted."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run(exe):
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (needs the reference sources at build time)")
    return subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)


def test_reference_gradcheck_passes_with_our_kernels():
    res = _run(ROOT / "oracle" / "_ref" / "gradcheck_b200")
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "ALL GRADIENTS OK" in res.stdout
    assert res.stdout.count("[PASS]") == 15


def test_c_host_modules_of_fused_entry_points():
    """csrc/host/b200_fused_modules.c (Module vtable + public optimizer/EMA API of the reference)
    against the reference's own host modules and central differences; see tests/host/."""
    res = _run(ROOT / "oracle" / "_ref" / "fused_modules_check")
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "0 failure(s)" in res.stdout
    assert res.stdout.count("PASS") == 25 and "FAIL" not in res.stdout
