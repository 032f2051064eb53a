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


@pytest.mark.parametrize("extra", [[], MOE], ids=["dense", "moe"])
def test_bucketed_optimizer_step_equals_single_bucket_and_checkpoints_interchange(tmp, extra):
    """The sharded optimizer step cut into one bucket per layer (every rank owns the r-th 1/n of EVERY bucket)
    against the step over a single bucket: same losses, norms and weights; and a checkpoint written under one
    cut is resumed under the other (the on-disk format does not depend on how the state is sharded at run time)."""
    common = TINY + ["--log_dir", tmp, "--total_batch_size", "512", "--batch_size", "2", "--sep_size", "1",
                     "--use_distributed_optimizer", "--do_save", "--save_every_steps", "4"] + extra
    one = run_trainer(2, common + ["--exp_name", "one"], {"TLM_ZERO1_BUCKET_MB": "100000"})
    per_layer = run_trainer(2, common + ["--exp_name", "layers"], {"TLM_ZERO1_BUCKET_MB": "0.0001"})
    _close(one["losses"], per_layer["losses"], 2e-6)
    _close(one["norms"], per_layer["norms"], 1e-5)
    assert abs(one["wsum"] - per_layer["wsum"]) < 1e-3
    first = run_trainer(2, common + ["--exp_name", "mix"], {"TLM_STOP_AFTER": "5", "TLM_ZERO1_BUCKET_MB": "0.0001"})
    assert first["start_step"] == 0
    second = run_trainer(2, common + ["--exp_name", "mix"], {"TLM_ZERO1_BUCKET_MB": "100000"})
    assert second["start_step"] == 5
    for k in ("5", "6", "7"):
        assert abs(one["losses"][k] - second["losses"][k]) < 2e-5, (k, one["losses"][k], second["losses"][k])
    assert abs(one["wsum"] - second["wsum"]) < 1e-3


def test_bucket_plan_and_shard_pieces():
    """Pure layout arithmetic: cuts fall on `q_proj` of the blocks that open a group, every boundary is a multiple
    of 8 * shard count, and the local pieces of all ranks tile the buffer exactly once."""
    import torch
    from train_large_model_from_scratch_b200.models import GPT
    from train_large_model_from_scratch_b200.parallel.zero1.distributed_optimizer import _Shard
    from train_large_model_from_scratch_b200.training.config import ModelConfig
    cfg = ModelConfig(num_layer=4, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                      vocab_size=512, block_size=64)
    model = GPT(cfg, device="cpu", compute_dtype=torch.float32, shard_world=4)
    layer_bytes = 4 * (model.dense_buf.layout["blocks.1.attn.q_proj.weight"][0]
                       - model.dense_buf.layout["blocks.0.attn.q_proj.weight"][0])
    cuts, groups = model.plan_buckets(target_bytes=2 * layer_bytes)          # two layers per group
    assert cuts[0] == [model.dense_buf.layout["blocks.0.attn.q_proj.weight"][0],
                       model.dense_buf.layout["blocks.2.attn.q_proj.weight"][0]]
    assert groups[0] == [0, 1, 2] and model._group_of_block == {0: 1, 2: 2}
    assert all(c % 32 == 0 for c in cuts[0]) and model.dense_buf.padded % (1024 * 4) == 0

    class _G:                                                               # stands in for a 4-rank process group
        pass
    import torch.distributed as dist
    covered = torch.zeros(model.dense_buf.padded, dtype=torch.int32)
    init = model.dense_buf.init_fp32.clone()
    for r in range(4):
        model.dense_buf.init_fp32 = init.clone()
        s = _Shard.__new__(_Shard)
        # build the shard by hand for rank r of 4 (no process group needed for the arithmetic)
        real_ws, real_rank = dist.get_world_size, dist.get_rank
        dist.get_world_size, dist.get_rank = (lambda g=None: 4), (lambda g=None, r=r: r)
        try:
            s.__init__(model.dense_buf, _G(), True, cuts[0], groups[0])
        finally:
            dist.get_world_size, dist.get_rank = real_ws, real_rank
        assert s.len == model.dense_buf.padded // 4 and [b.group for b in s.buckets] == [0, 1, 2]
        for b in s.buckets:
            covered[b.seg_lo:b.seg_lo + b.seg] += 1
            assert b.seg_lo % 8 == 0 and b.lo <= b.seg_lo and b.seg_lo + b.seg <= b.hi
        torch.testing.assert_close(s.master, s.take_local(init))
        full = torch.zeros_like(init)
        s.put_local(full, s.master)
        assert torch.equal(full[covered.bool() & (full != 0)], init[covered.bool() & (full != 0)])
    assert bool((covered == 1).all())


def test_bucket_plan_never_exceeds_the_flag_array():
    """The "parameters ready" flag array has room for 16 buckets per flat buffer: with many layers and a small bucket
    target the plan merges layers evenly instead of making more groups (dense: bucket 0 + at most 15 groups)."""
    import torch
    from train_large_model_from_scratch_b200.models import GPT
    from train_large_model_from_scratch_b200.training.config import ModelConfig
    cfg = ModelConfig(num_layer=40, hidden_size=32, num_attention_heads=2, num_key_value_heads=1, intermediate_size=64,
                      vocab_size=128, block_size=32)
    model = GPT(cfg, device="cpu", compute_dtype=torch.float32, shard_world=2)
    cuts, groups = model.plan_buckets(target_bytes=1)                        # would be one group per layer
    assert len(groups[0]) <= 16 and groups[0][0] == 0 and groups[0] == list(range(len(groups[0])))
    assert len(cuts[0]) == len(groups[0]) - 1 and cuts[0] == sorted(set(cuts[0]))
    starts = sorted(model._group_of_block)
    assert starts[0] == 0 and max(b - a for a, b in zip(starts, starts[1:] + [40])) <= 3     # 40 layers in <= 15 groups
