"""Plain-PyTorch definitions of every op in the model, written for clarity.

These are the numerical oracle for the CUDA kernels (tests compare a kernel
with the function here evaluated in fp32) and the execution path on CPU
(Gloo runs, fp32). They restate the math of the reference modules:
RMSNorm `model/modules/norm.py:14-19`, the RoPE variant of
`model/modules/attn.py:12-68`, GQA causal attention `attn.py:71-88,160-163`,
SwiGLU `model/modules/mlp.py:44`, top-k-then-softmax routing `mlp.py:100-103`,
and the masked-sum cross-entropy of `model/modules/loss.py:19-36`.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight.float() * (xf * rstd)


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float = 10000.0,
                variant: str = "reference") -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables `[T, head_dim]` in fp32.

    variant "reference": frequency i occupies ADJACENT slots (2i, 2i+1) —
    `[c0,c0,c1,c1,...]` — while the rotation still pairs slot j with j +- hd/2.
    That is what the reference computes; it is a fixed linear map per position
    but not the usual norm-preserving rotation.
    variant "standard": frequency i occupies slots i and i + hd/2.
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    freqs = torch.outer(positions.float(), inv_freq)            # [T, hd/2]
    if variant == "reference":
        full = freqs.repeat_interleave(2, dim=-1)                # c0,c0,c1,c1,...
    else:
        full = torch.cat([freqs, freqs], dim=-1)                 # c0..c_{hd/2-1}, c0..
    return full.cos(), full.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def rotate_half_t(x: torch.Tensor) -> torch.Tensor:
    """Transpose of `rotate_half` (used by the RoPE backward)."""
    h = x.shape[-1] // 2
    return torch.cat((x[..., h:], -x[..., :h]), dim=-1)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, T, H, hd]; cos/sin: [T, hd]. fp32 math, fp32 result."""
    xf = x.float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return xf * c + rotate_half(xf) * s


def rope_bwd(dy: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    df = dy.float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return df * c + rotate_half_t(df * s)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              q_offset: int = 0) -> torch.Tensor:
    """q: [B, Tq, Hq, hd], k/v: [B, Tk, Hkv, hd] -> [B, Tq, Hq, hd].
    Query row i sits at absolute position `q_offset + i`; key j at j."""
    B, Tq, Hq, hd = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)                                   # B,Hq,Tq,hd
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(hd)
    if causal:
        qi = torch.arange(Tq, device=q.device)[:, None] + q_offset
        kj = torch.arange(Tk, device=q.device)[None, :]
        s = s.masked_fill(kj > qi, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).permute(0, 2, 1, 3)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up: [..., 2I] with gate in the first half -> silu(gate) * up."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return F.silu(g) * u


def mlp(x, w_gate, w_up, w_down):
    xf = x.float()
    return (F.silu(xf @ w_gate.float().t()) * (xf @ w_up.float().t())) @ w_down.float().t()


def router_topk(logits: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """top-k on raw logits, THEN softmax over the k winners."""
    vals, idx = torch.topk(logits.float(), k, dim=-1)
    return torch.softmax(vals, dim=-1), idx


def moe(x: torch.Tensor, w_router, w_gate, w_up, w_down, k: int) -> torch.Tensor:
    """Dropless MoE, all experts local. x: [M, D]; w_gate/up: [E, I, D]; w_down: [E, D, I]."""
    xf = x.float()
    weights, experts = router_topk(xf @ w_router.float().t(), k)
    out = torch.zeros_like(xf)
    for e in range(w_gate.shape[0]):
        tok, slot = (experts == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        y = mlp(xf[tok], w_gate[e], w_up[e], w_down[e])
        out.index_add_(0, tok, y * weights[tok, slot, None])
    return out


def moe_aux_stats(logits: torch.Tensor, experts: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Switch-style load-balance term  E * sum_e f_e * p_e  with f_e the fraction
    of routed slots that chose e and p_e the mean full-softmax probability."""
    probs = torch.softmax(logits.float(), dim=-1).mean(0)
    frac = torch.bincount(experts.reshape(-1), minlength=num_experts).float() / experts.numel()
    return num_experts * (frac * probs).sum()


def cross_entropy_sum(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100):
    """(sum of per-token CE over valid targets, number of valid targets), fp32."""
    per_tok = F.cross_entropy(logits.float(), targets, ignore_index=ignore_index, reduction="none")
    valid = targets != ignore_index
    return (per_tok * valid).sum(), valid.sum().float()


def adamw_step(p, g, m, v, step: int, lr: float, beta1: float, beta2: float, eps: float, wd: float,
               grad_scale: float = 1.0):
    """One decoupled-weight-decay Adam step on fp32 tensors, in place.
    Same update as `torch.optim.AdamW` (non-amsgrad)."""
    g = g * grad_scale
    p.mul_(1.0 - lr * wd)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
