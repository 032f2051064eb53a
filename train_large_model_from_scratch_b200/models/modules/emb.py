"""Embedding tables (reference: `model/modules/emb.py:1-5`, where
`TextEmbedding` aliases `nn.Embedding` and `ImgEmbedding` is a placeholder)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import functional as F_ops


class TextEmbedding(nn.Module):
    """Token embedding whose output is the fp32 residual stream `[B*T, D]`."""

    def __init__(self, num_embeddings: int, embedding_dim: int, device=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim, device=device))

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        return F_ops.embedding(idx, self.weight)


class ImgEmbedding(nn.Module):
    """Placeholder kept for import compatibility; the reference defines no
    image embedding either."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        raise NotImplementedError("image embeddings are not part of this model family")
