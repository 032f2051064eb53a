"""CLI / config surface: defaults table, CLI-overrides-dataclass quirks, validation."""
import pytest

from train_large_model_from_scratch_b200.training import build_config, parse_args
from train_large_model_from_scratch_b200.training.config import ModelConfig, ParallelConfig, DataConfig
from train_large_model_from_scratch_b200.utils import get_training_info, lr_schedule


def test_cli_defaults_match_reference_table():
    a = parse_args([])
    assert (a.total_batch_size, a.batch_size, a.seq_len) == (524288, 8, 4096)
    assert a.max_steps is None and a.max_epochs == 1
    assert a.precision == "bf16" and a.steps_to_profile == [15, 20]
    assert (a.max_lr, a.min_lr, a.warmup_steps, a.weight_decay) == (4e-3, 3e-5, 1000, 0.1)
    assert (a.adam_beta1, a.adam_beta2, a.adam_eps) == (0.9, 0.95, 1e-8)
    assert a.sep_size == 8 and a.backend == "nccl" and a.init_method == "env://"
    assert (a.num_layer, a.num_attention_heads, a.num_key_value_heads, a.hidden_size) == (32, 128, 8, 1024)
    assert (a.num_experts, a.num_experts_per_tok, a.moe_intermediate_size) == (128, 8, 256)
    assert a.init_std == 0.013 and a.vocab_size == 50304 and a.block_size == 4096


def test_cli_overrides_dataclass_defaults():
    # dataclass defaults differ from the CLI defaults for these; the CLI wins
    assert ParallelConfig().sep_size == 1 and ParallelConfig().use_distributed_optimizer is True
    assert DataConfig().pin_memory is True and ModelConfig().tied_lm_head is True
    cfg = build_config(parse_args(["--warmup_steps", "1", "--max_steps", "5"]))
    assert cfg.parallel.sep_size == 8
    assert cfg.parallel.use_distributed_optimizer is False
    assert cfg.data.pin_memory is False and cfg.model.tied_lm_head is False
    assert cfg.parallel.ddp_gradient_as_bucket_view is False


def test_seed_not_forwarded_to_model_and_split_rate():
    cfg = build_config(parse_args(["--seed", "7"]))
    assert cfg.seed.seed == 7 and cfg.model.seed == 1337
    assert cfg.train.split_rate == 1.0
    assert build_config(parse_args(["--do_val"])).train.split_rate == 0.99
    d = cfg.as_dict()
    assert set(d) == {"logging", "seed", "data", "train", "optim", "ckpt", "parallel", "model"}
    assert cfg.model.as_dict()["hidden_size"] == 1024


def test_no_abbreviations_and_validation():
    with pytest.raises(SystemExit):
        parse_args(["--seq", "128"])
    with pytest.raises(ValueError):
        build_config(parse_args(["--hidden_size", "100", "--num_attention_heads", "3"]))
    with pytest.raises(ValueError):
        build_config(parse_args(["--max_steps", "10", "--warmup_steps", "10"]))
    with pytest.raises(ValueError):
        build_config(parse_args(["--num_attention_heads", "12", "--num_key_value_heads", "8", "--hidden_size", "768"]))


def test_training_info():
    info = get_training_info(1280, 4096, 524288, 8, 8, None, 1)
    assert info == {"epochs": 1, "max_steps": 10, "grad_accum_steps": 2, "total_tokens_per_step": 262144}
    info = get_training_info(1280, 4096, 524288, 8, 1, 5, None)
    assert info["grad_accum_steps"] == 16 and info["epochs"] == 0.5
    with pytest.raises(ValueError):
        get_training_info(1280, 4096, 524288, 8, 8, 7, 1)
    with pytest.raises(ValueError):
        get_training_info(1280, 4096, 524288, 8, 8, None, None)


def test_lr_schedule():
    assert lr_schedule(0, 100, 10, 1.0, 0.1) == pytest.approx(0.1)
    assert lr_schedule(9, 100, 10, 1.0, 0.1) == pytest.approx(1.0)
    assert lr_schedule(10, 100, 10, 1.0, 0.1) == pytest.approx(1.0)
    assert lr_schedule(55, 100, 10, 1.0, 0.1) == pytest.approx(0.55)
    assert lr_schedule(100, 100, 10, 1.0, 0.1) == pytest.approx(0.1)
    assert lr_schedule(101, 100, 10, 1.0, 0.1) == 0.1
