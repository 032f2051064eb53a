"""CUDA attention entry points used by `ops.native`.

INTERIM: until the tcgen05 flash-attention kernels land, the forward and
backward call the library SDPA kernels through ATen (a library call, like a
cuBLAS GEMM). Signature and tensor layouts are those of the final kernels.
"""
from __future__ import annotations

import torch


def fwd(qkv: torch.Tensor, n_q: int, n_kv: int, causal: bool):
    q = qkv[:, :, :n_q].transpose(1, 2)
    k = qkv[:, :, n_q:n_q + n_kv].transpose(1, 2)
    v = qkv[:, :, n_q + n_kv:].transpose(1, 2)
    rep = n_q // n_kv
    if rep > 1:
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    out = torch.ops.aten._scaled_dot_product_flash_attention(q, k, v, 0.0, causal, False)
    o, lse = out[0], out[1]
    fwd._ctx = None
    return o.transpose(1, 2).contiguous(), (lse, out[6], out[7])


def bwd(do, qkv, o, lse_pack, n_q: int, n_kv: int, causal: bool):
    lse, seed, offset = lse_pack
    B, T, _, hd = qkv.shape
    rep = n_q // n_kv
    q = qkv[:, :, :n_q].transpose(1, 2)
    k = qkv[:, :, n_q:n_q + n_kv].transpose(1, 2)
    v = qkv[:, :, n_q + n_kv:].transpose(1, 2)
    if rep > 1:
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
        do.transpose(1, 2), q, k, v, o.transpose(1, 2), lse, None, None, T, T, 0.0, causal, seed, offset)
    if rep > 1:
        dk = dk.reshape(B, n_kv, rep, T, hd).sum(2)
        dv = dv.reshape(B, n_kv, rep, T, hd).sum(2)
    return torch.cat([dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)], dim=2).contiguous()
