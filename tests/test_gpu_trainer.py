"""The training loop on real GPUs: the recorded (CUDA-graph) step against the ordinary step, and
save -> resume -> loss parity with the recorded step on, at 1 and 2 GPUs."""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

from dist_utils import ROOT, free_port

pytestmark = pytest.mark.gpu

FLAGS = ("--use_mock_data --mock_data_num_samples 256 --seq_len 256 --max_epochs 1 --warmup_steps 4 "
         "--tied_lm_head --num_layer 2 --hidden_size 256 --num_attention_heads 4 --num_key_value_heads 2 "
         "--intermediate_size 512 --vocab_size 8192 --max_lr 1e-3 --min_lr 1e-4 --total_batch_size 4096 "
         "--batch_size 2 --use_distributed_optimizer --sep_size 1").split()


def _run(world, env_extra, flags, log_dir=None):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = tempfile.mktemp(suffix=".json")
    log_dir = log_dir or tempfile.mkdtemp(prefix="tlm_gpu_")
    env = dict(os.environ, TLM_TEST_OUT=out, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0", TLM_NVLS="0")
    env.update(env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "_trainer_worker.py")] + flags + ["--log_dir", log_dir]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    with open(out) as f:
        return json.load(f)


def _close(a, b, tol, keys=None):
    for k in (keys if keys is not None else a):
        assert abs(a[k] - b[k]) <= tol * max(1.0, abs(a[k])), (k, a[k], b[k])


@pytest.mark.parametrize("world", [1, 2])
def test_recorded_step_equals_ordinary_step_through_the_warmup_boundary(world):
    """Steps 0-1 run eagerly, step 2 is recorded, steps 3.. replay it; the learning-rate warm-up ends at step
    4, so both schedule branches reach the kernels through the device-side hyper-parameter buffer. Atomic
    reductions (split-K weight gradients, dQ) make the two runs agree to rounding, not bit for bit."""
    eager = _run(world, {"TLM_CUDA_GRAPH": "0"}, FLAGS)
    graph = _run(world, {"TLM_CUDA_GRAPH": "1"}, FLAGS)
    assert len(graph["losses"]) >= 6
    _close(eager["losses"], graph["losses"], 2e-3)
    _close(eager["norms"], graph["norms"], 2e-2)
    assert abs(eager["wsum"] - graph["wsum"]) < 0.5


@pytest.mark.parametrize("world", [1, 2])
def test_save_resume_loss_parity_with_recorded_step(world):
    """An interrupted run (checkpoint at step 4, stop after step 5) continued by a second job must follow
    the uninterrupted run: parameters come back from the fp32 master shards into the (symmetric) bf16 buffer,
    Adam moments and the step counter from the sharded optimizer state, the data position from the sampler."""
    whole = _run(world, {}, FLAGS)
    d = tempfile.mkdtemp(prefix="tlm_gpu_resume_")
    first = _run(world, {"TLM_STOP_AFTER": "6"}, FLAGS + ["--do_save", "--save_every_steps", "4"], log_dir=d)
    assert first["start_step"] == 0
    second = _run(world, {}, FLAGS + ["--do_save", "--save_every_steps", "400"], log_dir=d)
    assert second["start_step"] == 5
    later = [k for k in whole["losses"] if int(k) >= 5]
    assert len(later) >= 3
    _close(whole["losses"], second["losses"], 3e-3, later)
    _close(whole["norms"], second["norms"], 3e-2, later)
