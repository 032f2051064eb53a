"""CUDA attention entry points used by `ops.native`: the tcgen05 flash-attention
kernels for head dims 32, 64 and 128 (32 runs on the 64-wide kernel with
zero-filled upper columns).

Other head dims (and non-causal calls) go to the library SDPA kernels through
ATen (a library call, like a cuBLAS GEMM).
"""
from __future__ import annotations

import math

import torch

from . import native


def _native_ok(hd: int) -> bool:
    return hd in (32, 64, 128)


_WARNED: set = set()


def _warn_library_path(hd: int, causal: bool) -> None:
    """Said once per shape class: a configuration must never be measured on the library kernels unnoticed."""
    key = (hd, causal)
    if key not in _WARNED:
        _WARNED.add(key)
        import warnings
        warnings.warn(f"attention with head dim {hd}, causal={causal} is outside the tcgen05 kernels "
                      f"(head dims 32 / 64 / 128, causal): running the library SDPA kernels instead",
                      RuntimeWarning, stacklevel=3)


def fwd(qkv: torch.Tensor, n_q: int, n_kv: int, causal: bool):
    """qkv `[B, T, n_q + 2 n_kv, hd]` bf16 -> (o `[B, T, n_q, hd]` bf16, lse `[B, n_q, T]` fp32)."""
    B, T, _, hd = qkv.shape
    if causal and _native_ok(hd):
        assert qkv.is_contiguous()
        o = torch.empty(B, T, n_q, hd, dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty(B, n_q, T, dtype=torch.float32, device=qkv.device)
        native._check(native.lib().tlm_attn_fwd(qkv.data_ptr(), o.data_ptr(), lse.data_ptr(), B, T, n_q, n_kv, hd,
                                                1.0 / math.sqrt(hd), native._stream()), "attn_fwd")
        return o, lse
    _warn_library_path(hd, causal)
    q, k, v = _split(qkv, n_q, n_kv)
    out = torch.ops.aten._scaled_dot_product_flash_attention(q, k, v, 0.0, causal, False)
    return out[0].transpose(1, 2).contiguous(), out[1]


def fwd_scatter(qkv: torch.Tensor, n_q: int, n_kv: int, dst_ptrs, n_dst: int, dst_rows: int, dst_heads: int,
                dst_head0: int):
    """Causal attention (head dims 64 / 128) whose epilogue also stores each output row into
    `dst[t // dst_rows][b, t % dst_rows, dst_head0 + h, :]` (`dst_ptrs`: ctypes array of device addresses of
    bf16 `[B, dst_rows, dst_heads, hd]` tensors, typically peers' symmetric buffers)."""
    B, T, _, hd = qkv.shape
    assert _native_ok(hd) and qkv.is_contiguous()
    o = torch.empty(B, T, n_q, hd, dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty(B, n_q, T, dtype=torch.float32, device=qkv.device)
    native._check(native.lib().tlm_attn_fwd_scatter(qkv.data_ptr(), o.data_ptr(), lse.data_ptr(), B, T, n_q, n_kv, hd,
                                                    1.0 / math.sqrt(hd), dst_ptrs, n_dst, dst_rows, dst_heads,
                                                    dst_head0, native._stream()), "attn_fwd_scatter")
    return o, lse


def bwd_scatter(do, qkv, o, lse, n_q: int, n_kv: int, rope, dst_ptrs, n_dst: int, dst_rows: int, dst_heads: int,
                dst_q0: int, dst_k0: int, dst_v0: int) -> None:
    """Causal attention backward (head dims 32 / 64 / 128) whose gradient rows are stored straight into the sequence
    owners' packed gradient tensors: row t of local q head s -> `dst[t // dst_rows][b, t % dst_rows, dst_q0 + s]`,
    k -> `dst_k0 + s`, v -> `dst_v0 + s` (`dst_ptrs`: ctypes array of device addresses of bf16
    `[B, dst_rows, dst_heads, hd]` tensors, typically peers' symmetric buffers). `rope = (cos, sin)` fp32 `[T, hd]`
    or None: transposed rotation of dQ / dK on the way."""
    B, T, _, hd = qkv.shape
    assert _native_ok(hd) and qkv.is_contiguous()
    do, o = do.contiguous(), o.contiguous()
    dq_acc = torch.empty(B, n_q, T, hd, dtype=torch.float32, device=qkv.device)
    delta = torch.empty(B, n_q, T, dtype=torch.float32, device=qkv.device)
    cos, sin = rope if rope is not None else (None, None)
    native._check(native.lib().tlm_attn_bwd_scatter(
        qkv.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), dq_acc.data_ptr(), delta.data_ptr(), B, T, n_q, n_kv,
        hd, 1.0 / math.sqrt(hd), native._ptr(cos), native._ptr(sin), dst_ptrs, n_dst, dst_rows, dst_heads, dst_q0, dst_k0,
        dst_v0, native._stream()), "attn_bwd_scatter")


def _split(qkv, n_q, n_kv):
    q = qkv[:, :, :n_q].transpose(1, 2)
    k = qkv[:, :, n_q:n_q + n_kv].transpose(1, 2)
    v = qkv[:, :, n_q + n_kv:].transpose(1, 2)
    rep = n_q // n_kv
    if rep > 1:
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    return q, k, v


def bwd(do, qkv, o, lse, n_q: int, n_kv: int, causal: bool, rope=None):
    """-> dqkv `[B, T, n_q + 2 n_kv, hd]` bf16 (gradient of the packed input). With `rope = (cos, sin)` (fp32
    `[T, hd]`) the q and k parts are the gradient of the UN-rotated heads (transposed RoPE applied in the kernels)."""
    B, T, _, hd = qkv.shape
    if causal and _native_ok(hd):
        do, o = do.contiguous(), o.contiguous()
        dqkv = torch.empty_like(qkv)
        dq_acc = torch.empty(B, n_q, T, hd, dtype=torch.float32, device=qkv.device)
        delta = torch.empty(B, n_q, T, dtype=torch.float32, device=qkv.device)
        cos, sin = rope if rope is not None else (None, None)
        if cos is not None:
            assert cos.dtype == torch.float32 and cos.shape == (T, hd) and cos.is_contiguous() and sin.is_contiguous()
        native._check(native.lib().tlm_attn_bwd(qkv.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                                dqkv.data_ptr(), dq_acc.data_ptr(), delta.data_ptr(), B, T, n_q, n_kv,
                                                hd, 1.0 / math.sqrt(hd), native._ptr(cos), native._ptr(sin),
                                                native._stream()), "attn_bwd")
        return dqkv
    assert rope is None, "the transposed rotation is part of the tcgen05 kernels only"
    _warn_library_path(hd, causal)
    rep = n_q // n_kv
    q, k, v = _split(qkv, n_q, n_kv)
    zero = torch.zeros((), dtype=torch.int64, device=qkv.device)
    dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
        do.transpose(1, 2), q, k, v, o.transpose(1, 2), lse, None, None, T, T, 0.0, causal, zero, zero)
    if rep > 1:
        dk = dk.reshape(B, n_kv, rep, T, hd).sum(2)
        dv = dv.reshape(B, n_kv, rep, T, hd).sum(2)
    return torch.cat([dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)], dim=2).contiguous()
