"""Dense SwiGLU MLP and dropless top-k mixture of experts with expert parallelism.

Reference: `model/modules/mlp.py:16-169`. Same parameters and state-dict keys
(`gate_proj/up_proj/down_proj.weight`; `router.weight`, `experts_gate_weights
[E_local, I, D]`, `experts_up_weights [E_local, I, D]`, `experts_down_weights
[E_local, D, I]`), same routing rule (top-k on raw logits, softmax over the k
winners, no token dropping), same seeding (`seed + global expert index`).

Differences in how it is computed:
  * gate and up are one GEMM against the fused `[2I, D]` weight;
  * expert math is `x @ W^T` for any `I` (the reference's grouped path only
    type-checks for `I == D`, its padded-bmm path has this meaning);
  * tokens are sorted by global expert id once; per-(destination, expert)
    counts are exchanged so the receiver derives its regrouping from counts
    and never receives expert ids; no `repeat_interleave` copy of the tokens;
  * optional load-balance auxiliary loss (`moe_aux_loss_coef`, default 0 like
    the reference, which has none) and optional capacity limit.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import functional as F_ops
from ...ops import moe_ops
from ...parallel import parallel_state
from ...parallel.flat import fuse_adjacent
from .attn import _Proj
from .init import seeded_normal


class MLP(nn.Module):
    """`down(silu(gate(x)) * up(x))`"""

    def __init__(self, config, use_moe: bool = False, device=None):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.moe_intermediate_size if use_moe else config.intermediate_size
        self.use_moe = use_moe
        D, I = self.hidden_size, self.intermediate_size
        self.gate_proj = _Proj(I, D, config.init_std, config.seed, device)
        self.up_proj = _Proj(I, D, config.init_std, config.seed, device)
        self.down_proj = _Proj(D, I, config.init_std, config.seed, device)
        self._gate_up_weight = None

    def _post_flatten(self) -> None:
        self._gate_up_weight = fuse_adjacent([self.gate_proj.weight, self.up_proj.weight])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x = x.reshape(-1, shape[-1]).to(self.gate_proj.weight.dtype)
        if F_ops.swiglu_mlp_fused_ok(x, self._gate_up_weight):
            return F_ops.swiglu_mlp(x, self._gate_up_weight, self.down_proj.weight).view(shape)
        if self._gate_up_weight is not None:
            gu = F_ops.linear(x, self._gate_up_weight)
        else:
            gu = torch.cat([F_ops.linear(x, self.gate_proj.weight), F_ops.linear(x, self.up_proj.weight)], dim=-1)
        return F_ops.linear(F_ops.swiglu(gu), self.down_proj.weight).view(shape)


class MoE(nn.Module):
    def __init__(self, config, top_k: int | None = None, device=None):
        super().__init__()
        self.config = config
        self.num_experts = config.num_experts
        self.top_k = top_k if top_k is not None else config.num_experts_per_tok
        assert self.top_k <= self.num_experts, \
            f"top_k must be <= num_experts, got {self.top_k} and {self.num_experts}"
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.moe_intermediate_size
        self.ep_size = parallel_state.get_ep_world_size()
        assert self.num_experts % self.ep_size == 0
        self.num_local_experts = self.num_experts // self.ep_size
        D, I, El = self.hidden_size, self.intermediate_size, self.num_local_experts
        self.router = _Proj(self.num_experts, D, config.init_std, config.seed, device)
        first = parallel_state.get_ep_rank() * El
        # The three matrices of expert e come from ONE generator stream seeded with
        # `seed + global index of e` (gate, up, down in this order), as in the reference.
        g, u, d = [], [], []
        for e in range(El):
            gen = torch.Generator(device=torch.device(device) if device is not None else torch.device("cpu"))
            gen.manual_seed(config.seed + first + e)
            dev = gen.device
            g.append(torch.empty(I, D, device=dev).normal_(0.0, config.init_std, generator=gen))
            u.append(torch.empty(I, D, device=dev).normal_(0.0, config.init_std, generator=gen))
            d.append(torch.empty(D, I, device=dev).normal_(0.0, config.init_std, generator=gen))
        self.experts_gate_weights = nn.Parameter(torch.stack(g))
        self.experts_up_weights = nn.Parameter(torch.stack(u))
        self.experts_down_weights = nn.Parameter(torch.stack(d))
        self.aux_loss = None
        self._pair_weight = None

    def _post_flatten(self) -> None:
        # gate and up matrices of all local experts as one [2 E_local, I, D] operand (a view: the two parameters
        # are adjacent in the flat expert buffer)
        g, u = self.experts_gate_weights, self.experts_up_weights
        buf = getattr(g, "flat_buffer", None)
        if buf is not None and getattr(u, "flat_buffer", None) is buf and u.flat_offset == g.flat_offset + g.numel():
            w, mg = buf.view(g.flat_offset, (2 * g.shape[0], g.shape[1], g.shape[2]))
            w = w.detach()
            w.requires_grad_(g.requires_grad)
            w.main_grad = mg
            self._pair_weight = w

    def forward(self, x: torch.Tensor):
        """x `[..., D]` -> (output of the same shape, router logits `[M, E]`)."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(self.router.weight.dtype)
        logits = F_ops.linear(x2, self.router.weight)
        out, aux = moe_ops.moe_forward(
            x2, logits, self.experts_gate_weights, self.experts_up_weights, self.experts_down_weights,
            self.top_k, self.num_experts, parallel_state.get_ep_group(), self.ep_size,
            aux_coef=self.config.moe_aux_loss_coef, capacity_factor=self.config.moe_capacity_factor,
            layer_key=id(self), w_pair=self._pair_weight)
        self.aux_loss = aux
        return out.view(shape), logits
