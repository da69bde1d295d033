"""The kernels' index arithmetic under the bounds-checked debug build: the loss, domain and trainer GPU tests are run once
more in a child process that loads ``_C_bounds`` (same sources, ``-DSC_BOUNDS=1``: every computed global index is compared
with its limit, a miss is recorded and the access skipped, nothing traps). The child's session fails if a miss was
recorded (tests/conftest.py). No bad input is fed to a kernel here; the launchers' refusals are tested on the CPU."""
import glob
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_gpu_suite_under_the_bounds_checked_build():
    if not glob.glob(os.path.join(ROOT, "scalingcontrasts_b200", "_C_bounds*.so")):
        pytest.skip("the bounds-checked build is not present (built with SC_BUILD_BOUNDS=0)")
    environment = dict(os.environ, PYTHONPATH=ROOT, SC_NATIVE_VARIANT="bounds")
    result = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
                             os.path.join(ROOT, "tests", "test_gpu_loss.py"), os.path.join(ROOT, "tests", "test_gpu_domain.py"),
                             os.path.join(ROOT, "tests", "test_gpu_trainer.py"), os.path.join(ROOT, "tests", "test_launcher_validation.py")],
                            cwd=ROOT, env=environment, capture_output=True, text=True, timeout=900)
    assert result.returncode == 0, result.stdout[-4000:] + result.stderr[-2000:]
    assert " passed" in result.stdout and "out-of-range" not in result.stdout
