"""RMSNorm. The class keeps the reference's name `LayerNorm` and state-dict key
(`ln_1.weight`, ...) although it normalises by the root mean square only: no
mean subtraction, no bias, eps 1e-6, statistics in fp32
(reference: `model/modules/norm.py:6-19`)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import functional as F_ops


class LayerNorm(nn.Module):
    def __init__(self, config, device=None):
        super().__init__()
        self.variance_epsilon = 1e-6
        self.hidden_size = config.hidden_size
        self.weight = nn.Parameter(torch.ones(self.hidden_size, device=device))

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None = None):
        """Standalone use: returns the normalised tensor. Inside the blocks the
        fused form `add_norm` is used instead."""
        shape = x.shape
        _, h = F_ops.add_rmsnorm(x.reshape(-1, shape[-1]).float(), delta, self.weight, self.variance_epsilon)
        return h.view(shape)

    def add_norm(self, x: torch.Tensor, delta: torch.Tensor | None):
        """(x + delta, norm(x + delta)) in one pass over the residual stream."""
        return F_ops.add_rmsnorm(x, delta, self.weight, self.variance_epsilon)


RMSNorm = LayerNorm
