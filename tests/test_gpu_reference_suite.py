"""The reference's OWN test scripts, unmodified, running on this library.

The reference's bridge loads whatever library the NWC_DLL variable names (reference: nwc/nwc_torch.py:14-22), so its
package and tests - staged by __graft_entry__.build() into the git-ignored baseline/_ref/ - exercise this library's ten
reference entry points exactly as the reference's users would: encoder through host pointers, table builder, dequant,
gather, token matvec, the native fp8 matvec, error codes.  Skipped where the staging folder is absent."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SUITE = os.path.join(ROOT, "baseline", "_ref")
LIB = os.path.join(ROOT, "nwc_b200", "lib", "nwc_ops.so")


def run_script(name, extra_env=None, timeout=900):
    script = os.path.join(SUITE, "tests", name)
    if not os.path.exists(script): pytest.skip("the reference's test scripts are not staged (baseline/_ref is made by build() where the reference is mounted)")
    env = dict(os.environ, NWC_DLL=LIB, **(extra_env or {}))
    return subprocess.run([sys.executable, script], env=env, capture_output=True, text=True, timeout=timeout, cwd=SUITE)


def test_reference_fp8_suite_passes_on_this_library():
    out = run_script("test_fp8.py")
    assert out.returncode == 0 and out.stdout.strip().endswith("OK"), out.stdout[-3000:] + out.stderr[-2000:]
    assert out.stdout.count("FAIL") == 0 and "NaN rejected: ok" in out.stdout


def test_reference_format_suite_passes_on_this_library():
    """The reference's pure-Python decoder applied to what this library's encoder wrote (bf16, all three layouts, the
    reference's shapes with planted escapes)."""
    out = run_script("test_format_cpu.py")
    assert out.returncode == 0 and out.stdout.strip().endswith("OK"), out.stdout[-3000:] + out.stderr[-2000:]
    assert out.stdout.count("bit-exact") == 18 and "MISMATCH" not in out.stdout


def test_reference_checkpoint_suite_passes_on_this_library():
    try:
        import accelerate  # noqa: F401
    except ImportError:
        pytest.skip("the reference's load_pretrained needs the accelerate package, which this image does not have")
    out = run_script("test_checkpoint.py")
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
