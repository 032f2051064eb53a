"""Numerical parity with the reference implementation itself: its unmodified model code runs on CPU as
the oracle (device lookups pointed at the CPU, Gloo world of one) next to this package's CPU path with the
reference's weights loaded through the checkpoint loader. Skipped when the reference tree is not installed
under `baseline/_ref`."""
import json
import os
import subprocess
import sys

import pytest

from dist_utils import ROOT, free_port

REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.parametrize("mode", ["dense", "moe"])
def test_loss_and_gradients_match_the_reference_model(mode):
    if not os.path.isfile(os.path.join(REF, "model", "gpt.py")):
        pytest.skip("reference tree not present under baseline/_ref")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    env.pop("PYTHONPATH", None)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_reference_worker.py"), REF, ROOT, mode,
                        str(free_port())], env=env, capture_output=True, text=True, timeout=600, cwd="/tmp")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["same_keys"], "state-dict keys / order differ from the reference"
    assert abs(res["loss_ref"] - res["loss_ours"]) < 2e-5 * abs(res["loss_ref"]), res
    assert abs(res["log_ref"] - res["log_ours"]) < 2e-5 * abs(res["log_ref"]), res
    assert res["worst_grad_rel"] < 2e-4, res
