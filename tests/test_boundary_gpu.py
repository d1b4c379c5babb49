"""The drop-in boundary against the real thing: the unmodified reference's own inferbit_load and
inferbit_forward with the GPU entries installed into its exported kernel table ib_kern
(src/kernels/scalar.c:185), one thread and four (the reference's pool then calls the table concurrently
with row slices, src/threading.c:220-241), FP32-activation and W4A8 routes. Each case runs in a child
process because the reference reads IB_W4A8 once per process."""
import json
import os
import subprocess
import sys

import pytest

from tests import _cpu

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("threads,w4a8", [(1, "0"), (4, "0"), (1, "1"), (4, "1")])
def test_reference_forward_runs_on_the_gpu_table(threads, w4a8):
    if not os.path.exists(_cpu.REF_SO):
        pytest.skip("the unmodified reference was not built here (oracle/_ref)")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_boundary_worker.py"), str(threads), w4a8],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])
    assert out["status"] == 0, out
    assert out["launches"] > 100, out                 # the forward pass really went through the GPU entries
    assert out["finite"] and out["close"], out
