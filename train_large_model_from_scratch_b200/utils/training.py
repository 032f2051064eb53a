"""Schedule arithmetic, seeding and capability probes.

Semantics follow the reference's `utils/training.py:10-91`: gradient-accumulation
steps are `total_batch / (seq_len * micro_batch * dp)`, `max_steps` is derived
from epochs when unset, and the two are cross-checked when both are given.
"""
from __future__ import annotations

import random
from typing import Any

import numpy as np
import torch
from packaging import version


def get_training_info(
    num_samples: int,
    tokens_per_sample: int,
    global_token_batch_size: int,
    samples_per_device_per_step: int,
    num_devices: int,
    max_steps: int | None = None,
    max_epochs: float | None = None,
) -> dict[str, Any]:
    """Return `{epochs, max_steps, grad_accum_steps, total_tokens_per_step}`.

    `total_tokens_per_step` is the token count of ONE micro-step over all DP
    ranks (the reference's naming, `utils/training.py:40-41`)."""
    if max_steps is None and max_epochs is None:
        raise ValueError("At least one of max_steps or max_epochs must be provided.")
    micro_tokens = tokens_per_sample * samples_per_device_per_step * num_devices
    grad_accum_steps = int(global_token_batch_size / micro_tokens)
    dataset_tokens = num_samples * tokens_per_sample
    steps_from_epochs = (
        int(max_epochs * dataset_tokens / global_token_batch_size) if max_epochs is not None else None)
    epochs_from_steps = (
        max_steps * global_token_batch_size / dataset_tokens if max_steps is not None else None)
    if max_steps is not None and max_epochs is not None:
        if steps_from_epochs != max_steps or int(epochs_from_steps) != int(max_epochs):
            raise ValueError(
                "Inconsistent max_steps and max_epochs for this dataset/configuration: "
                f"max_epochs={max_epochs} gives {steps_from_epochs} steps but max_steps={max_steps}; "
                f"max_steps gives {int(epochs_from_steps)} epochs.")
    elif max_steps is None:
        max_steps = steps_from_epochs
    else:
        max_epochs = epochs_from_steps
    return {
        "epochs": max_epochs,
        "max_steps": max_steps,
        "grad_accum_steps": grad_accum_steps,
        "total_tokens_per_step": micro_tokens,
    }


def set_seed(seed: int, deterministic: bool = False) -> None:
    """Seed python, numpy and torch (CPU + all CUDA devices)."""
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)
        from ..ops import native
        if native.available():
            native.set_deterministic(True)            # no split-K atomics in the weight-gradient GEMMs


def torch_version_ge(torch_version: str = "2.10") -> bool:
    """True when the running torch is at least `torch_version` (the reference's
    helper of the same name compares with a strict `>`, `utils/training.py:85-87`;
    this one means what its name says)."""
    return version.parse(torch.__version__.split("+")[0]) >= version.parse(torch_version)


def sm_ge(device: torch.device | int | None = None, sm: int = 80) -> bool:
    """True when the CUDA device's compute capability is >= `sm` (e.g. 100)."""
    if not torch.cuda.is_available():
        return False
    major, minor = torch.cuda.get_device_capability(device)
    return major * 10 + minor >= sm


def lr_schedule(it: int, max_steps: int, warmup_steps: int, max_lr: float, min_lr: float) -> float:
    """Linear warm-up then cosine decay to `min_lr`
    (reference: `training/trainer.py:196-207`)."""
    import math
    if it < warmup_steps:
        return max_lr * (it + 1) / warmup_steps
    if it > max_steps:
        return min_lr
    ratio = (it - warmup_steps) / (max_steps - warmup_steps)
    return min_lr + 0.5 * (1.0 + math.cos(math.pi * ratio)) * (max_lr - min_lr)
