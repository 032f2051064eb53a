"""Multi-GPU paths (need >= 2 GPUs): peer-memory optimizer collectives against the
NCCL path, and layout invariance of the loss curve on real GPUs."""
import os
import sys

import pytest
import torch

from dist_utils import ROOT, free_port

pytestmark = pytest.mark.gpu

FLAGS = ("--use_mock_data --mock_data_num_samples 256 --seq_len 256 --max_epochs 1 --warmup_steps 2 "
         "--tied_lm_head --num_layer 2 --hidden_size 256 --num_attention_heads 4 --num_key_value_heads 2 "
         "--intermediate_size 512 --vocab_size 8192 --max_lr 1e-3 --min_lr 1e-4 --total_batch_size 4096 "
         "--batch_size 2 --debug --use_distributed_optimizer").split()


def _run(world, env_extra, flags):
    import json
    import subprocess
    import tempfile
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = tempfile.mktemp(suffix=".json")
    log_dir = tempfile.mkdtemp(prefix="tlm_gpu_")
    env = dict(os.environ, TLM_TEST_OUT=out, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    env.update(env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "_trainer_worker.py")] + flags + ["--log_dir", log_dir]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    with open(out) as f:
        return json.load(f)


def _close(a, b, tol):
    for k in a:
        assert abs(a[k] - b[k]) <= tol * max(1.0, abs(a[k])), (k, a[k], b[k])


def test_peer_collectives_match_nccl():
    ref = _run(2, {"TLM_COMM": "nccl"}, FLAGS + ["--sep_size", "1"])
    p2p = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, FLAGS + ["--sep_size", "1"])
    _close(ref["losses"], p2p["losses"], 2e-3)
    _close(ref["norms"], p2p["norms"], 2e-2)
    assert abs(ref["wsum"] - p2p["wsum"]) < 0.5


def test_peer_collectives_multimem():
    ref = _run(2, {"TLM_COMM": "nccl"}, FLAGS + ["--sep_size", "1"])
    mc = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "1"}, FLAGS + ["--sep_size", "1"])
    _close(ref["losses"], mc["losses"], 2e-3)
    _close(ref["norms"], mc["norms"], 2e-2)


def test_bf16_gradient_wire_tracks_fp32_wire():
    ref = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, FLAGS + ["--sep_size", "1"])
    for nvls in ("0", "1"):
        bf = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": nvls}, FLAGS + ["--sep_size", "1", "--grad_wire_dtype", "bf16"])
        _close(ref["losses"], bf["losses"], 3e-3)
        _close(ref["norms"], bf["norms"], 2e-2)


def test_sequence_parallel_matches_data_parallel_on_gpu():
    dp = _run(2, {}, FLAGS + ["--sep_size", "1"])
    sp = _run(2, {}, [f if f != "2" or FLAGS[i - 1] != "--batch_size" else "4" for i, f in enumerate(FLAGS)] + ["--sep_size", "2"])
    _close(dp["losses"], sp["losses"], 5e-3)


MOE = ["--use_moe", "--num_experts", "8", "--num_experts_per_tok", "2", "--moe_intermediate_size", "256"]


def test_ulysses_peer_path_matches_nccl_path():
    flags = [f if f != "2" or FLAGS[i - 1] != "--batch_size" else "4" for i, f in enumerate(FLAGS)] + ["--sep_size", "2"]
    ref = _run(2, {"TLM_COMM": "nccl"}, flags)
    peer = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, flags)                       # exchanges inside GEMM / attention epilogues
    _close(ref["losses"], peer["losses"], 2e-3)
    _close(ref["norms"], peer["norms"], 2e-2)
    plain = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0", "TLM_SP_FUSED": "0"}, flags)   # stand-alone scatter kernels
    _close(ref["losses"], plain["losses"], 2e-3)
    _close(ref["norms"], plain["norms"], 2e-2)


def test_ulysses_with_fewer_kv_heads_than_ranks_matches_nccl_path():
    """One KV head shared by both ranks' query heads (4 query heads, 1 KV head, sep 2): the QKV epilogue replicates
    the head to both owners and the sequence owners sum the replicas' dK / dV; against the library-collective path
    and against plain data parallelism."""
    one_kv = [f if FLAGS[i - 1] != "--num_key_value_heads" else "1" for i, f in enumerate(FLAGS)]
    flags = [f if FLAGS[i - 1] != "--batch_size" else "4" for i, f in enumerate(one_kv)] + ["--sep_size", "2"]
    ref = _run(2, {"TLM_COMM": "nccl"}, flags)
    peer = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, flags)
    _close(ref["losses"], peer["losses"], 2e-3)
    _close(ref["norms"], peer["norms"], 2e-2)
    dp = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, one_kv + ["--sep_size", "1"])
    _close(dp["losses"], peer["losses"], 5e-3)


def test_expert_parallel_peer_path_matches_nccl_path_and_single_group():
    flags4 = [f if f != "2" or FLAGS[i - 1] != "--batch_size" else "4" for i, f in enumerate(FLAGS)]
    ref = _run(2, {"TLM_COMM": "nccl"}, flags4 + MOE + ["--sep_size", "2"])
    peer = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, flags4 + MOE + ["--sep_size", "2"])
    dp = _run(2, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, FLAGS + MOE + ["--sep_size", "1"])
    _close(ref["losses"], peer["losses"], 3e-3)
    _close(ref["losses"], dp["losses"], 5e-3)
    _close(ref["norms"], peer["norms"], 3e-2)


WIDE = [f if FLAGS[i - 1] not in ("--num_attention_heads", "--num_key_value_heads") else "8" for i, f in enumerate(FLAGS)]


@pytest.mark.parametrize("world,sep,batch", [(4, 4, 4), (4, 2, 2), (8, 8, 8), (8, 2, 2)])
def test_larger_groups_match_the_nccl_path(world, sep, batch):
    """The peer-memory paths (optimizer collectives, Ulysses exchanges in the GEMM / attention epilogues) at
    4 and 8 ranks, pure sequence parallelism and DP x SEP grids, against the library-collective path with the
    same layout. 8 query / 8 KV heads so that every rank owns whole heads at sep = 8."""
    flags = [f if FLAGS[i - 1] != "--batch_size" else str(batch) for i, f in enumerate(WIDE)] + ["--sep_size", str(sep)]
    ref = _run(world, {"TLM_COMM": "nccl"}, flags)
    peer = _run(world, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, flags)
    _close(ref["losses"], peer["losses"], 3e-3)
    _close(ref["norms"], peer["norms"], 3e-2)


@pytest.mark.parametrize("world", [4, 8])
def test_expert_parallel_at_larger_groups(world):
    flags = [f if FLAGS[i - 1] != "--batch_size" else str(world) for i, f in enumerate(WIDE)]
    ref = _run(world, {"TLM_COMM": "nccl"}, flags + MOE + ["--sep_size", str(world)])
    peer = _run(world, {"TLM_COMM": "symm", "TLM_NVLS": "0"}, flags + MOE + ["--sep_size", str(world)])
    _close(ref["losses"], peer["losses"], 3e-3)
    _close(ref["norms"], peer["norms"], 3e-2)


@pytest.mark.parametrize("kind", ["dense_dp", "ulysses", "moe"])
def test_guard_bands_stay_intact_and_results_do_not_depend_on_epoch_parity(kind):
    """Stand-ins for a device-side memory / race checker on the peer-memory paths: (1) every symmetric buffer
    between guard bands that no peer store may touch; (2) the same job with all flag epochs started at an odd value
    (every double-buffered slot swaps parity) and just below 2^31 (the counters wrap within the run): losses and
    norms must not move."""
    flags4 = [f if f != "2" or FLAGS[i - 1] != "--batch_size" else "4" for i, f in enumerate(FLAGS)]
    flags = {"dense_dp": FLAGS + ["--sep_size", "1"], "ulysses": flags4 + ["--sep_size", "2"],
             "moe": flags4 + MOE + ["--sep_size", "2"]}[kind]
    env = {"TLM_COMM": "symm", "TLM_NVLS": "0"}
    base = _run(2, env, flags)
    guarded = _run(2, dict(env, TLM_SYMM_CANARY="1"), flags)
    assert guarded["guards"] == [], guarded["guards"]
    _close(base["losses"], guarded["losses"], 2e-3)
    for e0 in ("1", "2147483600"):
        other = _run(2, dict(env, TLM_EPOCH0=e0), flags)
        _close(base["losses"], other["losses"], 2e-3)
        _close(base["norms"], other["norms"], 2e-2)
