"""Multi-rank plumbing on CPU/Gloo: group layout, layout invariance of the loss
curve (DP, ZeRO-1, Ulysses SP, EP), checkpoint save -> resume parity, commit
marker atomicity."""
import os
import shutil
import tempfile

import pytest

from dist_utils import TINY, run_trainer
from train_large_model_from_scratch_b200.parallel.parallel_state import group_layout
from train_large_model_from_scratch_b200.parallel.sequence_parallel.ulysses import head_plan


def test_group_layout_matches_reference_rule():
    sep, dp = group_layout(8, 4)
    assert sep == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert dp == [[0, 4], [1, 5], [2, 6], [3, 7]]
    sep, dp = group_layout(8, 1)
    assert sep == [[i] for i in range(8)] and dp == [list(range(8))]
    with pytest.raises(AssertionError):
        group_layout(8, 3)


def test_head_plan():
    plans, q_l, kv_l = head_plan(16, 8, 8)            # 2 q heads / rank share one kv head
    assert (q_l, kv_l) == (2, 1) and plans[3] == [6, 7, 16 + 3, 24 + 3]
    plans, q_l, kv_l = head_plan(8, 2, 4)             # kv head replicated to two ranks
    assert (q_l, kv_l) == (2, 1) and plans[1] == [2, 3, 8 + 0, 10 + 0] and plans[2] == [4, 5, 8 + 1, 10 + 1]
    plans, q_l, kv_l = head_plan(8, 4, 2)
    assert (q_l, kv_l) == (4, 2) and plans[1] == [4, 5, 6, 7, 8 + 2, 8 + 3, 12 + 2, 12 + 3]
    with pytest.raises(ValueError):
        head_plan(6, 2, 4)


def _flags(tmp, extra):
    return TINY + ["--log_dir", tmp, "--total_batch_size", "512", "--debug"] + extra


def _close(a, b, tol):
    assert a.keys() == b.keys()
    for k in a:
        assert abs(a[k] - b[k]) <= tol * max(1.0, abs(a[k])), (k, a[k], b[k])


@pytest.fixture()
def tmp():
    d = tempfile.mkdtemp(prefix="tlm_test_")
    yield d
    shutil.rmtree(d, ignore_errors=True)


def test_dense_layout_invariance(tmp):
    """dp=1 vs dp=2 (ZeRO-1) vs sep=2: same losses and grad norms."""
    base = run_trainer(1, _flags(tmp, ["--batch_size", "4", "--sep_size", "1", "--use_distributed_optimizer"]))
    dp2 = run_trainer(2, _flags(tmp, ["--batch_size", "2", "--sep_size", "1", "--use_distributed_optimizer"]))
    dp2_plain = run_trainer(2, _flags(tmp, ["--batch_size", "2", "--sep_size", "1"]))
    sp2 = run_trainer(2, _flags(tmp, ["--batch_size", "4", "--sep_size", "2", "--use_distributed_optimizer"]))
    assert len(base["losses"]) == 8
    for other in (dp2, dp2_plain, sp2):
        _close(base["losses"], other["losses"], 2e-5)
        _close(base["norms"], other["norms"], 1e-3)
        assert abs(base["wsum"] - other["wsum"]) < 1e-2


MOE = ["--use_moe", "--num_experts", "4", "--num_experts_per_tok", "2", "--moe_intermediate_size", "32"]


def test_moe_layout_invariance(tmp):
    base = run_trainer(1, _flags(tmp, MOE + ["--batch_size", "4", "--sep_size", "1", "--use_distributed_optimizer"]))
    ep2 = run_trainer(2, _flags(tmp, MOE + ["--batch_size", "4", "--sep_size", "2", "--use_distributed_optimizer"]))
    dp2 = run_trainer(2, _flags(tmp, MOE + ["--batch_size", "2", "--sep_size", "1", "--use_distributed_optimizer"]))
    _close(base["losses"], ep2["losses"], 2e-5)
    _close(base["losses"], dp2["losses"], 2e-5)
    _close(base["norms"], ep2["norms"], 1e-3)


def test_four_ranks_dp2_sep2(tmp):
    base = run_trainer(1, _flags(tmp, MOE + ["--batch_size", "4", "--sep_size", "1", "--use_distributed_optimizer"]))
    grid = run_trainer(4, _flags(tmp, MOE + ["--batch_size", "2", "--sep_size", "2", "--use_distributed_optimizer"]))
    _close(base["losses"], grid["losses"], 2e-5)
    _close(base["norms"], grid["norms"], 1e-3)


@pytest.mark.parametrize("extra,world", [([], 2), (MOE + ["--sep_size", "2"], 2)])
def test_save_resume_parity(tmp, extra, world):
    """Train 8 steps straight vs 5 steps + save + new process resumes to 8."""
    sep = [] if "--sep_size" in extra else ["--sep_size", "1"]
    common = TINY + ["--log_dir", tmp, "--total_batch_size", "512", "--batch_size", "2",
                     "--use_distributed_optimizer", "--do_save", "--save_every_steps", "4"] + sep + extra
    straight = run_trainer(world, common + ["--exp_name", "a"])
    first = run_trainer(world, common + ["--exp_name", "b"], {"TLM_STOP_AFTER": "5"})
    files = os.listdir(first["log_dir"])
    for suffix in ("00004_model.pt", "00004_meta.pt", "00004_opt", "00004_rng_rank0.pt", f"00004_rng_rank{world - 1}.pt"):
        assert suffix in files, files
    second = run_trainer(world, common + ["--exp_name", "b"])
    assert second["start_step"] == 5
    for k in ("5", "6", "7"):
        assert abs(straight["losses"][k] - second["losses"][k]) < 2e-5, (k, straight["losses"][k], second["losses"][k])
    assert abs(straight["wsum"] - second["wsum"]) < 1e-3


def test_incomplete_checkpoint_is_ignored(tmp):
    common = TINY + ["--log_dir", tmp, "--total_batch_size", "512", "--batch_size", "4", "--sep_size", "1",
                     "--use_distributed_optimizer", "--do_save", "--save_every_steps", "2"]
    first = run_trainer(1, common, {"TLM_STOP_AFTER": "4", "TLM_CRASH_IN_SAVE": "1"})
    files = os.listdir(first["log_dir"])
    assert "00103_model.pt" in files and "00103_meta.pt" not in files      # crashed before the commit marker
    second = run_trainer(1, common, {"TLM_STOP_AFTER": "5"})
    assert second["start_step"] == 3                                         # resumed from step 2, not 103
