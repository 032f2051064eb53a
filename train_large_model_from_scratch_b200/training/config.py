"""Frozen configuration dataclasses. This module is a leaf: it imports nothing
from the rest of the package, so models, parallel state and utils can all
depend on it without an import cycle.

Field names, defaults and the CLI-overrides-dataclass behaviour follow the
reference's `training/config.py:6-234` (e.g. `--pin_memory`, `--sep_size`,
`--tied_lm_head`, `--use_distributed_optimizer` have CLI defaults that differ
from the dataclass defaults; `build_config` always takes the CLI value).

Differences, all deliberate:
  * `ModelConfig.as_dict()` exists (the reference's `save()` calls it and
    crashes because it is missing, `training/trainer.py:398`).
  * Extra optional knobs with reference-parity defaults: `moe_aux_loss_coef`
    (0.0 = no auxiliary loss, as in the reference), `moe_capacity_factor`
    (0.0 = dropless), `rope_variant` ("reference"), `grad_wire_dtype`,
    `heartbeat_timeout_s` (0 = off), `dist_timeout_s`.
"""
from __future__ import annotations

import argparse
from dataclasses import asdict, dataclass, field, fields
from typing import Any


@dataclass(frozen=True)
class TrainingConfig:
    total_batch_size: int = 524288      # tokens per optimizer step, whole job
    batch_size: int = 8                 # micro-batch (sequences) per DP rank
    seq_len: int = 4096                 # full sequence; each SP rank sees seq_len / sep
    max_steps: int | None = None
    max_epochs: int | None = 1
    do_val: bool = False
    val_every_steps: int = 250
    split_rate: float | None = None
    grad_clip_value: float = 1.0
    debug: bool = False
    precision: str = "bf16"
    use_compile: bool = False
    use_profiler: bool = False
    steps_to_profile: list[int] = field(default_factory=lambda: [15, 20])

    def with_derived(self) -> "TrainingConfig":
        """Fill `split_rate` (0.99 with validation, else 1.0) when unset."""
        if self.split_rate is not None:
            return self
        values = {f.name: getattr(self, f.name) for f in fields(self)}
        values["split_rate"] = 0.99 if self.do_val else 1.0
        return TrainingConfig(**values)


@dataclass(frozen=True)
class LoggingConfig:
    exp_name: str = "gpt"
    log_dir: str = "./log/"
    log_every: int = 10
    print_config: bool = False


@dataclass(frozen=True)
class SeedConfig:
    seed: int = 1337
    deterministic: bool = False


@dataclass(frozen=True)
class DataConfig:
    dataset_path: str = ""
    use_mock_data: bool = False
    mock_data_num_samples: int = 1280
    num_workers: int = 0
    pin_memory: bool = True


@dataclass(frozen=True)
class OptimConfig:
    max_lr: float = 4e-3
    min_lr: float = 3e-5
    warmup_steps: int = 1000
    weight_decay: float = 0.1
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8


@dataclass(frozen=True)
class CheckpointConfig:
    do_save: bool = False
    save_every_steps: int = 5000
    resume_path: str | None = None


@dataclass(frozen=True)
class ParallelConfig:
    backend: str = "nccl"
    init_method: str = "env://"
    sep_size: int = 1
    ddp_find_unused_parameters: bool = False
    ddp_gradient_as_bucket_view: bool = True
    use_distributed_optimizer: bool = True
    # "bf16": gradients cross NVLink as bf16 and are summed in fp32;
    # "fp32": full-precision wire, used for parity runs.
    grad_wire_dtype: str = "fp32"
    # > 0: host-side heartbeats between steps (`utils.health`); a peer silent for this long fails the job
    heartbeat_timeout_s: float = 0.0
    dist_timeout_s: float = 1800.0


@dataclass(frozen=True)
class ModelConfig:
    seed: int = 1337
    block_size: int = 4096
    vocab_size: int = 50304
    num_layer: int = 32
    num_attention_heads: int = 128
    num_key_value_heads: int = 8
    hidden_size: int = 1024
    intermediate_size: int = 4096
    dropout: float = 0.0
    init_std: float = 0.013
    tied_lm_head: bool = True
    use_moe: bool = False
    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 256
    # additions (defaults reproduce the reference's behaviour)
    moe_aux_loss_coef: float = 0.0
    moe_capacity_factor: float = 0.0
    rope_variant: str = "reference"     # "reference" | "standard"
    rope_theta: float = 10000.0

    def as_dict(self) -> dict[str, Any]:
        return asdict(self)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


@dataclass(frozen=True)
class Config:
    logging: LoggingConfig
    seed: SeedConfig
    data: DataConfig
    train: TrainingConfig
    optim: OptimConfig
    ckpt: CheckpointConfig
    parallel: ParallelConfig
    model: ModelConfig

    def as_dict(self) -> dict[str, Any]:
        return {f.name: asdict(getattr(self, f.name)) for f in fields(self)}


def _pick(cls, args: argparse.Namespace, **overrides):
    """Build dataclass `cls` from the Namespace attributes of the same name."""
    values = {}
    for f in fields(cls):
        if f.name in overrides:
            values[f.name] = overrides[f.name]
        elif hasattr(args, f.name):
            values[f.name] = getattr(args, f.name)
    return cls(**values)


def build_config(args: argparse.Namespace) -> Config:
    """Namespace -> frozen Config. As in the reference
    (`training/config.py:184-199`) the global `--seed` is NOT forwarded to
    `ModelConfig.seed`, which stays at its default so that weight init does not
    depend on the data seed."""
    cfg = Config(
        logging=_pick(LoggingConfig, args),
        seed=_pick(SeedConfig, args),
        data=_pick(DataConfig, args),
        train=_pick(TrainingConfig, args).with_derived(),
        optim=_pick(OptimConfig, args),
        ckpt=_pick(CheckpointConfig, args),
        parallel=_pick(ParallelConfig, args),
        model=_pick(ModelConfig, args, seed=ModelConfig.seed),
    )
    validate_static(cfg)
    return cfg


def validate_static(cfg: Config) -> None:
    """Checks that need no process group (reference: `training/config.py:214-234`)."""
    t, m = cfg.train, cfg.model
    if t.seq_len <= 0:
        raise ValueError("seq_len must be positive.")
    if t.batch_size <= 0:
        raise ValueError("batch_size (micro batch) must be positive.")
    if t.total_batch_size <= 0:
        raise ValueError("total_batch_size must be positive (tokens).")
    if cfg.parallel.sep_size <= 0:
        raise ValueError("sep_size must be positive.")
    if t.precision not in ("bf16", "fp16", "fp32"):
        raise ValueError(f"Unsupported precision: {t.precision}")
    if t.max_steps is not None and cfg.optim.warmup_steps >= t.max_steps:
        raise ValueError("warmup_steps must be < max_steps when max_steps is set.")
    if m.hidden_size % m.num_attention_heads != 0:
        raise ValueError("hidden_size must be divisible by num_attention_heads.")
    if m.num_attention_heads % m.num_key_value_heads != 0:
        raise ValueError("num_attention_heads must be divisible by num_key_value_heads (GQA).")
    if m.use_moe and m.num_experts_per_tok <= 0:
        raise ValueError("num_experts_per_tok must be positive when use_moe is enabled.")
    if m.use_moe and m.num_experts_per_tok > m.num_experts:
        raise ValueError("num_experts_per_tok must be <= num_experts.")
    if m.rope_variant not in ("reference", "standard"):
        raise ValueError(f"Unknown rope_variant: {m.rope_variant}")
    if cfg.parallel.grad_wire_dtype not in ("bf16", "fp32"):
        raise ValueError(f"Unknown grad_wire_dtype: {cfg.parallel.grad_wire_dtype}")
