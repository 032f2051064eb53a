"""GQA causal self-attention with RoPE and optional Ulysses sequence parallelism.

What the reference does in `model/modules/attn.py:126-176` with three GEMMs, a
K/V expansion to Hq heads, a freshly built fp32 RoPE table per call, stack /
transpose copies around two all-to-alls and a library SDPA call is done here as:

  one GEMM against the fused `[Hq*hd + 2*Hkv*hd, D]` weight (q|k|v are adjacent
  in the flat parameter buffer) -> RoPE on the q and k heads of the packed
  `[B, T, Hq+2Hkv, hd]` tensor (table cached per position range) -> (SP only)
  seq->head exchange of un-expanded heads -> flash attention that reads KV head
  `h // (Hq/Hkv)` directly -> (SP only) head->seq exchange -> output GEMM.

State-dict keys (`q_proj.weight`, `k_proj.weight`, `v_proj.weight`,
`c_proj.weight`) and shapes equal the reference's.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import functional as F_ops
from ...ops import oracle
from ...parallel import parallel_state
from ...parallel.flat import fuse_adjacent
from ...parallel.sequence_parallel import ulysses
from .init import seeded_normal


def rope_impl(q: torch.Tensor, k: torch.Tensor, position_ids: torch.Tensor, rope_theta: float = 10000.0,
              variant: str = "reference"):
    """Functional RoPE on `[B, H, T, hd]` tensors (API of the reference's
    `rope_impl`, `attn.py:12-68`); fp32 result."""
    pos = position_ids[0] if position_ids.dim() > 1 else position_ids
    cos, sin = oracle.rope_tables(pos, q.shape[-1], rope_theta, variant)
    qe = oracle.rope(q.transpose(1, 2), cos, sin).transpose(1, 2)
    ke = oracle.rope(k.transpose(1, 2), cos, sin).transpose(1, 2)
    return qe, ke


def gqa_impl(k: torch.Tensor, v: torch.Tensor, num_key_value_heads: int, num_attention_heads: int):
    """Expand `[B, Hkv, T, hd]` to Hq heads. Provided for API parity
    (`attn.py:71-88`); the attention op never needs it."""
    if num_attention_heads % num_key_value_heads:
        raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
    rep = num_attention_heads // num_key_value_heads
    if rep == 1:
        return k, v
    return k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)


class _Proj(nn.Module):
    """Holder of one bias-free weight so that keys read `<name>.weight`."""

    def __init__(self, out_features: int, in_features: int, std: float, seed: int, device):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(seeded_normal((out_features, in_features), std, seed, device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        y = F_ops.linear(x.reshape(-1, shape[-1]).to(self.weight.dtype), self.weight)
        return y.view(*shape[:-1], self.out_features)


class Attention(nn.Module):
    def __init__(self, config, device=None):
        super().__init__()
        assert config.hidden_size % config.num_attention_heads == 0
        self.config = config
        self.num_attention_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.n_embd = config.hidden_size
        self.dropout = config.dropout           # > 0: training steps take the library attention path (see forward)
        hd, D = self.head_dim, config.hidden_size
        self.q_proj = _Proj(self.num_attention_heads * hd, D, config.init_std, config.seed, device)
        self.k_proj = _Proj(self.num_key_value_heads * hd, D, config.init_std, config.seed, device)
        self.v_proj = _Proj(self.num_key_value_heads * hd, D, config.init_std, config.seed, device)
        self.c_proj = _Proj(D, D, config.init_std, config.seed, device)
        self._qkv_weight = None
        self._rope_cache: dict = {}
        self._rope_cache_full: dict = {}
        self._rope_cache_fp16: dict = {}

    def _post_flatten(self) -> None:
        self._qkv_weight = fuse_adjacent([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight])

    def _rope(self, T_local: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        start = parallel_state.get_sep_rank() * T_local
        key = (start, T_local, str(device))
        if key not in self._rope_cache:
            pos = torch.arange(start, start + T_local, device=device)
            self._rope_cache = {key: oracle.rope_tables(pos, self.head_dim, self.config.rope_theta,
                                                        self.config.rope_variant)}
        return self._rope_cache[key]

    def _rope_fp16(self, T_local: int, device) -> torch.Tensor:
        """(cos, sin) pairs in fp16 for the fused projection epilogue."""
        from ...ops import native
        key = (parallel_state.get_sep_rank() * T_local, T_local, str(device))
        if key not in self._rope_cache_fp16:
            self._rope_cache_fp16 = {key: native.rope_table_fp16(*self._rope(T_local, device))}
        return self._rope_cache_fp16[key]

    def _rope_full(self, T_full: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        key = ("full", T_full, str(device))
        if key not in self._rope_cache_full:
            pos = torch.arange(0, T_full, device=device)
            self._rope_cache_full = {key: oracle.rope_tables(pos, self.head_dim, self.config.rope_theta,
                                                             self.config.rope_variant)}
        return self._rope_cache_full[key]

    def _symm_ok(self, x: torch.Tensor) -> bool:
        if not (x.is_cuda and x.dtype == torch.bfloat16):
            return False
        from ...parallel import symm
        return symm.use_symm()

    def _peer_path(self, qkv: torch.Tensor, sp: int) -> bool:
        from ...parallel.sequence_parallel import ulysses_peer
        return self._symm_ok(qkv) and ulysses_peer.supported(self.num_attention_heads, self.num_key_value_heads, sp,
                                                             self.head_dim)

    def forward(self, h: torch.Tensor, B: int | None = None, T_local: int | None = None) -> torch.Tensor:
        """h: `[B*T_local, D]` (or `[B, T_local, D]`) in the compute dtype -> same shape."""
        shape = h.shape
        if h.dim() == 3:
            B, T_local = shape[0], shape[1]
            h = h.reshape(-1, shape[-1])
        Hq, Hkv, hd = self.num_attention_heads, self.num_key_value_heads, self.head_dim
        h = h.to(self.q_proj.weight.dtype)
        sp = parallel_state.get_sep_world_size()
        group = parallel_state.get_sep_group()
        cos, sin = self._rope(T_local, h.device)
        dropout_p = self.dropout if self.training else 0.0      # reference: attn.py:159
        if dropout_p > 0.0:
            return self._forward_with_dropout(h, B, T_local, cos, sin, dropout_p, sp, group).view(shape)
        if F_ops.qkv_project_fused_ok(h, self._qkv_weight, hd, T_local):
            # CUDA: projection + RoPE (+ the seq->head exchange) are one GEMM with a head-scatter epilogue
            if sp == 1:
                o = F_ops.qkv_attention(h, self._qkv_weight, cos, sin, self._rope_fp16(T_local, h.device), B, T_local,
                                        Hq, Hkv, hd)
                y = F_ops.linear(o.reshape(B * T_local, Hq * hd), self.c_proj.weight)
                return y.view(shape)
            from ...parallel.sequence_parallel import ulysses_peer
            if self._symm_ok(h) and ulysses_peer.fused_ok(Hq, Hkv, sp, hd, T_local):      # incl. Hkv < sp (replicated KV heads)
                cos_f, sin_f = self._rope_full(T_local * sp, h.device)
                y = ulysses_peer.attention_block(h, self._qkv_weight, self.c_proj.weight, Hq, Hkv, hd, B, T_local,
                                                 self._rope_fp16(T_local, h.device), cos_f, sin_f, id(self), group)
                return y.view(shape)
        if self._qkv_weight is not None:
            qkv = F_ops.linear(h, self._qkv_weight)
        else:
            qkv = torch.cat([F_ops.linear(h, self.q_proj.weight), F_ops.linear(h, self.k_proj.weight),
                             F_ops.linear(h, self.v_proj.weight)], dim=-1)
        qkv = qkv.view(B, T_local, Hq + 2 * Hkv, hd)
        if sp > 1 and self._peer_path(qkv, sp):
            # RoPE + seq->head exchange in one kernel writing into the head owners' memory,
            # attention, then the head->seq exchange; see parallel/sequence_parallel/ulysses_peer.py
            from ...parallel.sequence_parallel import ulysses_peer
            cos_f, sin_f = self._rope_full(T_local * sp, h.device)
            qkv_l = ulysses_peer.seq_to_head(qkv, Hq, Hkv, cos, sin, cos_f, sin_f, id(self), group)
            o = F_ops.attention_packed(qkv_l, Hq // sp, Hkv // sp, True)
            o = ulysses_peer.head_to_seq(o, Hq, id(self), group)
            y = F_ops.linear(o.reshape(B * T_local, Hq * hd), self.c_proj.weight)
            return y.view(shape)
        qkv = F_ops.rope_qk(qkv, cos, sin, Hq + Hkv)
        if sp > 1:
            qkv_l, q_l, kv_l = ulysses.seq_to_head(qkv, Hq, Hkv, group)
            o = F_ops.attention_packed(qkv_l.contiguous(), q_l, kv_l, True)
            o = ulysses.head_to_seq(o, group)
        else:
            o = F_ops.attention_packed(qkv, Hq, Hkv, True)
        y = F_ops.linear(o.reshape(B * T_local, Hq * hd), self.c_proj.weight)
        return y.view(shape)

    def _forward_with_dropout(self, h, B, T_local, cos, sin, dropout_p, sp, group) -> torch.Tensor:
        """Attention-probability dropout (`--dropout > 0`, training mode). The flash kernels of this package carry no
        dropout mask, so this configuration runs projection, RoPE and the Ulysses exchanges as separate ops and the
        library's scaled-dot-product attention with `dropout_p` (what the reference calls, `attn.py:159-163`); every
        reference script trains with 0.0, which takes the fused path."""
        import warnings
        Hq, Hkv, hd = self.num_attention_heads, self.num_key_value_heads, self.head_dim
        warnings.warn("attention dropout > 0: using the library attention kernel instead of the sm_100a flash kernels",
                      stacklevel=2)
        if self._qkv_weight is not None:
            qkv = F_ops.linear(h, self._qkv_weight)
        else:
            qkv = torch.cat([F_ops.linear(h, self.q_proj.weight), F_ops.linear(h, self.k_proj.weight),
                             F_ops.linear(h, self.v_proj.weight)], dim=-1)
        qkv = F_ops.rope_qk(qkv.view(B, T_local, Hq + 2 * Hkv, hd), cos, sin, Hq + Hkv)
        q_l, kv_l = Hq, Hkv
        if sp > 1:
            qkv, q_l, kv_l = ulysses.seq_to_head(qkv, Hq, Hkv, group)
        q, k, v = qkv.split([q_l, kv_l, kv_l], dim=2)
        o = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=dropout_p, is_causal=True,
            enable_gqa=q_l != kv_l).transpose(1, 2).contiguous()
        if sp > 1:
            o = ulysses.head_to_seq(o, group)
        return F_ops.linear(o.reshape(B * T_local, Hq * hd), self.c_proj.weight)
