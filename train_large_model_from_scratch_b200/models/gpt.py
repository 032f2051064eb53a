"""Decoder-only GPT: token embedding -> `num_layer` pre-norm blocks (GQA
attention with RoPE, SwiGLU MLP or top-k MoE) -> final norm -> (tied) LM head
-> sequence-parallel-aware cross-entropy.

Same modules, parameter names and FLOP model as the reference
(`model/gpt.py:19-98`). The blocks hand the un-added branch output to the next
norm so that `residual add + RMSNorm` is one pass, and in training the LM head
and the loss are one fused op that never materialises `[B*T, V]` logits.

Numerical conventions kept from the reference: fp32 residual stream, RMSNorm
statistics in fp32, GEMM inputs in the compute dtype (bf16 on the GPU), fp32
cross-entropy.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as F_ops
from ..parallel import parallel_state
from ..parallel.flat import EXPERT_LOCAL_PARAM_SUFFIXES, flatten_model
from ..training.config import ModelConfig
from .modules.attn import Attention
from .modules.emb import TextEmbedding
from .modules.init import seeded_normal
from .modules.loss import CrossEntropyLoss
from .modules.mlp import MLP, MoE
from .modules.norm import LayerNorm

__all__ = ["GPT", "Block", "EXPERT_LOCAL_PARAM_SUFFIXES"]


def _default_device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


class Block(nn.Module):
    def __init__(self, config: ModelConfig, use_moe: bool = True, top_k: int | None = None, device=None):
        super().__init__()
        self.use_moe = use_moe
        self.ln_1 = LayerNorm(config, device)
        self.attn = Attention(config, device)
        self.ln_2 = LayerNorm(config, device)
        self.mlp = MoE(config, top_k, device) if use_moe else MLP(config, device=device)

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None, B: int, T: int):
        """x: fp32 residual `[B*T, D]`; delta: branch output not yet added.
        Returns (residual, pending branch output)."""
        x, h = self.ln_1.add_norm(x, delta)
        a = self.attn(h, B, T)
        x, h = self.ln_2.add_norm(x, a)
        m = self.mlp(h)
        if self.use_moe:
            m = m[0]
        return x, m


class _GroupBoundary(torch.autograd.Function):
    """Identity on the residual stream at the entry of a layer group. Its backward runs right after the
    backward of the group's first block, i.e. when every gradient of the group's parameters has been produced,
    and tells the optimizer so (`hooks.group_backward_done(g)`), which may then start reducing that bucket."""

    @staticmethod
    def forward(ctx, x, delta, hooks, g):
        ctx.hooks, ctx.g = hooks, g
        return x.view_as(x), (delta.view_as(delta) if delta is not None else None)

    @staticmethod
    def backward(ctx, gx, gd):
        ctx.hooks.group_backward_done(ctx.g)
        return gx, gd, None, None


class GPT(nn.Module):
    def __init__(self, config: ModelConfig, device=None, compute_dtype: torch.dtype | None = None,
                 flatten: bool = True, shard_world: int = 1, alloc=None):
        super().__init__()
        self.config = config
        self.device = torch.device(device) if device is not None else _default_device()
        if compute_dtype is None:
            compute_dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.compute_dtype = compute_dtype
        self.use_moe = config.use_moe
        dev = self.device
        self.wte = TextEmbedding(config.vocab_size, config.hidden_size, device=dev)
        self.blocks = nn.ModuleList([Block(config, self.use_moe, device=dev) for _ in range(config.num_layer)])
        self.lnf = LayerNorm(config, dev)
        self.lm_head = nn.Module()
        self.lm_head.weight = nn.Parameter(torch.empty(0, device=dev))
        with torch.no_grad():
            self.wte.weight.copy_(seeded_normal((config.vocab_size, config.hidden_size), config.init_std,
                                                config.seed, dev, cache=not config.tied_lm_head))
        if config.tied_lm_head:
            self.lm_head.weight = self.wte.weight
        else:
            self.lm_head.weight = nn.Parameter(
                seeded_normal((config.vocab_size, config.hidden_size), config.init_std, config.seed, dev))
        self.loss_fn = CrossEntropyLoss()
        self.dense_buf = self.expert_buf = None
        # communication hooks of the sharded optimizer step (set by the trainer on the peer-memory path): an object
        # with before_forward(), before_group(g) and group_backward_done(g); `_group_of_block[i] = g` for the
        # blocks that open a layer group (see `plan_buckets`)
        self.comm_hooks = None
        self._group_of_block: dict = {}
        if flatten:
            pad = 1024 * max(1, shard_world)
            # every parameter starts at a multiple of 8 * shard count, so that any parameter boundary can be
            # a bucket boundary of the optimizer step
            self.dense_buf, self.expert_buf = flatten_model(self, compute_dtype, dev, pad, pad, alloc,
                                                            align=8 * max(1, shard_world))

    # ------------------------------------------------------------------ optimizer buckets
    def plan_buckets(self, target_bytes: int = 192 << 20, max_groups: int = 15):
        """Cut the flat buffers at layer-group boundaries for the bucketed optimizer step.

        Consecutive blocks form a group until the group holds `target_bytes` of fp32 gradients (at most
        `max_groups` groups). Group g >= 1 starts at block s_g; the dense buffer is cut at the offset of
        `blocks[s_g].attn.q_proj.weight` (a group's FIRST norm weight stays in the bucket before it: it is read
        before the group's first GEMM, which is where the group's parameters are waited for), the expert buffer
        at `blocks[s_g].mlp.experts_gate_weights`. Bucket 0 of the dense buffer (embedding, first norm) belongs
        to group 0, whose gradients are only final at the end of the backward pass.
        Returns `(cuts, bucket_groups)`, each a list with one entry per flat buffer (dense, then expert if
        present), and records which block opens which group."""
        dl = self.dense_buf.layout
        offs = [dl[f"blocks.{i}.attn.q_proj.weight"][0] for i in range(len(self.blocks))] + [self.dense_buf.padded]
        el = self.expert_buf.layout if self.expert_buf is not None else None
        starts, acc = [0], 0
        for i in range(len(self.blocks)):
            layer = offs[i + 1] - offs[i]
            if el is not None:
                nxt = el[f"blocks.{i + 1}.mlp.experts_gate_weights"][0] if i + 1 < len(self.blocks) else self.expert_buf.padded
                layer += nxt - el[f"blocks.{i}.mlp.experts_gate_weights"][0]
            acc += 4 * layer
            if acc >= target_bytes and i + 1 < len(self.blocks):
                starts.append(i + 1)
                acc = 0
        if len(starts) > max_groups:                       # merge evenly
            per = -(-len(self.blocks) // max_groups)
            starts = list(range(0, len(self.blocks), per))
        self._group_of_block = {s: g + 1 for g, s in enumerate(starts)}
        cuts = [[offs[s] for s in starts]]
        groups = [[0] + [g + 1 for g in range(len(starts))]]
        if el is not None:
            cuts.append([el[f"blocks.{s}.mlp.experts_gate_weights"][0] for s in starts if s > 0])
            groups.append([g + 1 for g in range(len(starts))])
        return cuts, groups

    # ------------------------------------------------------------------ forward
    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None, loss_scale: float = 1.0,
                return_logits: bool | None = None):
        """idx, targets: `[B, T_local]` (this SP rank's slice of the sequence).
        Returns `(logits, loss, logging_loss)` like the reference
        (`model/gpt.py:64-73`); both losses are multiplied by `loss_scale`
        (pass `1 / grad_accum_steps`, then call `loss.backward()` directly).
        Logits are only materialised when there are no targets or when
        `return_logits=True`."""
        B, T = idx.size()
        sp = parallel_state.get_sp_world_size()
        assert T * sp <= self.config.block_size * sp and T <= self.config.block_size, \
            f"Cannot forward sequence of length {T}, block size is only {self.config.block_size}"
        hooks = self.comm_hooks
        if hooks is not None:
            hooks.before_forward()                      # embedding and first norm: wait for their bucket
        x = self.wte(idx)
        delta = None
        aux_total = None
        for i, block in enumerate(self.blocks):
            g = self._group_of_block.get(i) if hooks is not None else None
            if g is not None:
                hooks.before_group(g)                   # the group's first GEMM waits for the group's parameters
                if torch.is_grad_enabled():
                    x, delta = _GroupBoundary.apply(x, delta, hooks, g)
            x, delta = block(x, delta, B, T)
            if self.use_moe and block.mlp.aux_loss is not None:
                aux_total = block.mlp.aux_loss if aux_total is None else aux_total + block.mlp.aux_loss
        _, h = self.lnf.add_norm(x, delta)
        if return_logits is None:
            return_logits = targets is None
        logits = None
        if return_logits:
            logits = F_ops.linear(h, self.lm_head.weight).view(B, T, -1)
        if targets is None:
            return logits, None, None
        if return_logits:
            loss, logging_loss = self.loss_fn(logits, targets)
            loss, logging_loss = loss * loss_scale, logging_loss * loss_scale
        else:
            loss, logging_loss = self.loss_fn.fused(h, self.lm_head.weight, targets, loss_scale)
        if aux_total is not None:
            loss = loss + aux_total * (loss_scale / sp)
        return logits, loss, logging_loss

    # ------------------------------------------------------------------ bookkeeping
    def zero_grad_buffers(self) -> None:
        for buf in (self.dense_buf, self.expert_buf):
            if buf is not None:
                buf.zero_grad()

    def get_flops_per_fwd_bwd(self, batch_size: int, seq_len: int) -> float:
        """Reference FLOP model (`model/gpt.py:75-98`), kept verbatim in meaning
        so that MFU figures are comparable: 8BTD^2 for the four projections
        (GQA ignored), 4BT^2D for attention (causality ignored), SwiGLU FFN, no
        LM head; x3 for forward+backward; divided by the SP / EP sizes."""
        c = self.config
        sp, ep = parallel_state.get_sp_world_size(), parallel_state.get_ep_world_size()
        B, T, D = batch_size, seq_len, c.hidden_size
        attn = 8 * B * T * D * D + 4 * B * T * T * D
        inter = c.moe_intermediate_size if self.use_moe else c.intermediate_size
        ffn = 6 * B * T * D * inter + B * T * inter
        if self.use_moe:
            per_layer = (attn + 2 * B * T * D * c.num_experts) / sp + c.num_experts_per_tok * ffn / ep
        else:
            per_layer = (attn + ffn) / sp
        return 3 * c.num_layer * per_layer

    def get_exact_flops_per_fwd_bwd(self, batch_size: int, seq_len: int) -> float:
        """Corrected count per device: GQA projection sizes, causal attention
        (half the score matrix), LM head included."""
        c = self.config
        sp, ep = parallel_state.get_sp_world_size(), parallel_state.get_ep_world_size()
        B, T, D = batch_size, seq_len, c.hidden_size
        hd = D // c.num_attention_heads
        proj = 2 * B * T * D * (c.num_attention_heads * hd + 2 * c.num_key_value_heads * hd + D)
        attn = 4 * B * T * T * D / 2
        if self.use_moe:
            ffn = 2 * B * T * D * c.num_experts + c.num_experts_per_tok * 6 * B * T * D * c.moe_intermediate_size
        else:
            ffn = 6 * B * T * D * c.intermediate_size
        head = 2 * B * T * D * c.vocab_size
        # backward = 2x forward for GEMMs, 2.5x for attention (recomputed scores)
        return (3 * c.num_layer * (proj + ffn) + 3.5 * c.num_layer * attn + 3 * head) / sp
