"""Sequence-parallel-aware cross-entropy (reference: `model/modules/loss.py:14-42`).

Each SP rank holds a slice of the sequence. The loss that is back-propagated
is `local CE sum / number of valid targets over the whole SP group`, so that
summing gradients over the SP group gives the gradient of the mean loss; the
logged loss is the SP-global mean. The valid-target count depends on the
targets only, so it is reduced once up front; the count and both loss scalars
travel in one small all-reduce instead of two per micro-step.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ...ops import functional as F_ops
from ...parallel import parallel_state


def sp_valid_count(targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Number of non-ignored targets over the SP group, clamped to >= 1 (fp32, 0-d)."""
    cnt = (targets != ignore_index).sum().float()
    if parallel_state.get_sp_world_size() > 1:
        from ...parallel.symm import scalar_all_reduce
        cnt = scalar_all_reduce(cnt, parallel_state.get_sp_group())
    return cnt.clamp(min=1.0)


def sp_sum(x: torch.Tensor) -> torch.Tensor:
    if parallel_state.get_sp_world_size() > 1:
        from ...parallel.symm import scalar_all_reduce
        x = scalar_all_reduce(x, parallel_state.get_sp_group())
    return x


class CrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index: int = -100):
        super().__init__()
        self.ignore_index = ignore_index

    def forward(self, logits: torch.Tensor, targets: torch.Tensor):
        """From materialised logits `[B, T_local, V]` -> (loss, logging_loss)."""
        local_sum, _ = F_ops.cross_entropy_from_logits(
            logits.reshape(-1, logits.size(-1)), targets, self.ignore_index)
        count = sp_valid_count(targets, self.ignore_index)
        loss = local_sum / count
        with torch.no_grad():
            logging_loss = sp_sum(local_sum.detach()) / count
        return loss, logging_loss

    def fused(self, h: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, loss_scale: float = 1.0):
        """LM head + CE without materialising logits.
        Returns (loss * loss_scale, logging_loss * loss_scale)."""
        count = sp_valid_count(targets, self.ignore_index)
        grad_scale = loss_scale / count
        local_sum = F_ops.linear_cross_entropy(h, weight, targets, grad_scale, self.ignore_index)
        loss = local_sum * grad_scale
        with torch.no_grad():
            logging_loss = sp_sum(local_sum.detach()) * grad_scale
        return loss, logging_loss
