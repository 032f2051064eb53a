"""Helpers to run a function on N Gloo ranks (CPU) as child processes."""
import json
import os
import socket
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TINY = ("--use_mock_data --mock_data_num_samples 64 --seq_len 64 --max_epochs 1 --warmup_steps 2 "
        "--tied_lm_head --num_layer 2 --hidden_size 64 --num_attention_heads 4 --num_key_value_heads 2 "
        "--intermediate_size 128 --max_lr 3e-3 --min_lr 3e-4 --precision fp32 --backend gloo").split()


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_trainer(world: int, flags: list[str], steps_env: dict | None = None, timeout: int = 600,
                script: str | None = None, expect_fail: bool = False):
    """Launch `tests/_trainer_worker.py` on `world` ranks; returns rank 0's JSON result."""
    port = free_port()
    out = tempfile.mktemp(suffix=".json")
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), TLM_TEST_OUT=out, PYTHONPATH=ROOT, OMP_NUM_THREADS="2",
                   CUDA_VISIBLE_DEVICES="")
        env.update(steps_env or {})
        procs.append(subprocess.Popen([sys.executable, script or os.path.join(ROOT, "tests", "_trainer_worker.py")] + flags,
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    codes, logs = [], []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        codes.append(p.returncode)
        logs.append(o)
    if expect_fail:
        return codes, logs
    assert all(c == 0 for c in codes), "\n".join(l[-3000:] for l in logs)
    with open(out) as f:
        res = json.load(f)
    os.remove(out)
    return res
