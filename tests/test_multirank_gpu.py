"""Two ranks on two GPUs (skipped where fewer are visible): the decode step with every linear row-sharded and the slices
gathered - over the peer window (push over NVLink) and over NCCL - reproduces the logits the unmodified reference
recorded for the seeded mini model, on every rank. One process per GPU, as in the benchmark."""
import json
import os
import subprocess
import sys
import tempfile

import pytest

from libinferbit_b200 import _ffi

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("transport", ["push", "nccl"])
def test_two_ranks_reproduce_reference_logits(transport):
    if _ffi.load_ibcu().ibcu_device_count() < 2:
        pytest.skip("needs two GPUs")
    with tempfile.TemporaryDirectory() as d:
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "_tworank_worker.py"), str(r), "2", d, transport],
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
        outs = []
        for pr in procs:
            try:
                o, e = pr.communicate(timeout=300)
            except subprocess.TimeoutExpired:
                for q in procs:
                    q.kill()
                raise
            assert pr.returncode == 0, e[-2000:]
            outs.append(json.loads(o.strip().splitlines()[-1]))
    for o in outs:
        assert o["ok"], o
        assert o["launches"] > 50, o
