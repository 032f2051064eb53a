"""ctypes binding of the sm_100a kernel library (`libtlm_b200.so`, built in-tree
by `build_ext.py` from `csrc/*.cu`).

The library exports plain C launchers that take device pointers, sizes and a
CUDA stream; this module wraps them into functions on torch tensors. Nothing
here falls back to another implementation: on a machine with a GPU a missing
or unloadable library is an error.
"""
from __future__ import annotations

import ctypes
import os

import torch

_LIB = None
# the in-tree build; TLM_LIB names another build of the same sources (A/B comparisons of kernel changes)
_LIB_PATH = os.environ.get("TLM_LIB") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                      "libtlm_b200.so")


class NativeError(RuntimeError):
    pass


def lib_path() -> str:
    return _LIB_PATH


def available() -> bool:
    return torch.cuda.is_available() and os.path.exists(_LIB_PATH)


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(_LIB_PATH):
            raise NativeError(
                f"{_LIB_PATH} not found: build it with `python -m train_large_model_from_scratch_b200.build_ext`")
        _LIB = ctypes.CDLL(_LIB_PATH)
        _declare(_LIB)
    return _LIB


_c = ctypes
_P, _I, _LL, _F = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_float

_SIGS = {
    "tlm_launch_count": (_c.c_ulonglong, []),
    "tlm_reset_launch_count": (None, []),
    "tlm_add_launch_count": (None, [_c.c_ulonglong]),
    "tlm_take_device_status": (_c.c_uint, []),
    "tlm_num_sms": (_I, []),
    "tlm_set_deterministic": (None, [_I]),
    "tlm_get_deterministic": (_I, []),
    "tlm_gemm_set_pair": (_I, [_I]),
    "tlm_gemm": (_I, [_P, _P, _P, _I, _I, _I, _LL, _LL, _LL, _I, _I, _I, _P]),
    "tlm_gemm_heads": (_I, [_P, _P, _I, _I, _I, _LL, _LL, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P]),
    "tlm_gemm_swiglu": (_I, [_P, _P, _P, _P, _I, _I, _I, _LL, _LL, _P]),
    "tlm_gemm_swiglu_bwd": (_I, [_P, _P, _P, _P, _I, _I, _I, _LL, _LL, _P]),
    "tlm_gemm_swiglu_grouped": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _I, _P]),
    "tlm_gemm_swiglu_bwd_grouped": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _I, _P]),
    "tlm_gemm_grouped_rows": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _LL, _LL, _I, _I, _I, _P]),
    "tlm_gemm_grouped_k": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _LL, _LL, _I, _P]),
    "tlm_embedding_fwd": (_I, [_P, _P, _P, _I, _I, _LL, _P]),
    "tlm_embedding_bwd": (_I, [_P, _P, _P, _I, _I, _LL, _P]),
    "tlm_add_rmsnorm_fwd": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _P]),
    "tlm_add_rmsnorm_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P]),
    "tlm_rope": (_I, [_P, _P, _P, _LL, _I, _I, _I, _I, _I, _P]),
    "tlm_swiglu_fwd": (_I, [_P, _P, _LL, _I, _P, _P]),
    "tlm_swiglu_bwd": (_I, [_P, _P, _P, _LL, _I, _P, _P]),
    "tlm_gemm_grouped_pair": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _LL, _LL, _LL, _I, _I, _P]),
    "tlm_ce_inplace": (_I, [_P, _P, _P, _P, _I, _I, _LL, _LL, _I, _P]),
    "tlm_sumsq_scratch_floats": (_I, []),
    "tlm_sumsq": (_I, [_P, _LL, _P, _P, _P]),
    "tlm_attn_fwd": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _F, _P]),
    "tlm_attn_fwd_scatter": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _I, _I, _I, _I, _P]),
    "tlm_attn_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P, _P]),
    "tlm_attn_bwd_scatter": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "tlm_peer_barrier": (_I, [_P, _I, _I, _I, _P]),
    "tlm_wait_flag": (_I, [_P, _I, _c.c_ulonglong, _P]),
    "tlm_reduce_scatter_blocks": (_I, []),
    "tlm_reduce_scatter": (_I, [_P, _P, _P, _P, _P, _P, _LL, _LL, _I, _I, _I, _I, _P]),
    "tlm_reduce_scatter_bf16": (_I, [_P, _P, _LL, _LL, _P, _P, _P, _P, _P, _P, _LL, _LL, _I, _I, _I, _I, _P]),
    "tlm_adamw_gather": (_I, [_P, _P, _P, _P, _P, _P, _P, _LL, _LL, _I, _I, _F, _F, _F, _F, _F, _F, _F, _P, _P, _I, _P]),
    "tlm_ready_ints": (_I, []),
    "tlm_ready_max_buckets": (_I, []),
    "tlm_wait_params_ready": (_I, [_P, _I, _I, _P]),
    "tlm_gemm_arm_param_wait": (_I, [_P, _I, _I]),
    "tlm_gemm_clear_param_waits": (None, []),
    "tlm_gemm_flush_param_waits": (_I, [_P]),
    "tlm_peer_allreduce_scalar": (_I, [_P, _P, _P, _P, _F, _I, _I, _I, _P]),
    "tlm_peer_scatter_heads": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P]),
    "tlm_peer_put_i32": (_I, [_P, _I, _P, _I, _LL, _P]),
    "tlm_peer_scatter_rows": (_I, [_P, _P, _I, _P, _P, _P, _P, _I, _I, _P, _LL, _LL, _P]),
    "tlm_moe_route_blocks": (_I, [_I]),
    "tlm_moe_route": (_I, [_P, _LL, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P]),
    "tlm_moe_plan": (_I, [_P, _I, _I, _I, _P, _P, _P, _I, _LL, _P, _P, _P, _P, _P, _P, _P]),
    "tlm_moe_route_bwd": (_I, [_P, _P, _P, _P, _LL, _I, _I, _P]),
    "tlm_moe_gather": (_I, [_P, _P, _I, _P, _P, _LL, _I, _P]),
    "tlm_moe_combine": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "tlm_moe_pair_dot": (_I, [_P, _P, _P, _P, _LL, _I, _I, _P]),
    "tlm_gemm_grouped_rows_scatter": (_I, [_P, _P, _P, _I, _I, _I, _I, _LL, _LL, _LL, _LL, _I, _I, _P, _P, _P, _I, _LL, _P]),
    "tlm_adamw": (_I, [_P, _P, _P, _P, _P, _P, _LL, _F, _F, _F, _F, _F, _F, _F, _P, _P]),
    "tlm_expect_close": (_I, [_P, _P, _F, _I, _P]),
    "tlm_gemm_lse": (_I, [_P, _P, _I, _I, _I, _LL, _LL, _P, _P, _P, _P]),
    "tlm_gemm_dlogits": (_I, [_P, _P, _P, _I, _I, _I, _LL, _LL, _LL, _P, _P, _P, _LL, _P]),
    "tlm_lse_finish": (_I, [_P, _I, _P, _P, _LL, _LL, _P, _P, _I, _P]),
}


def _declare(l) -> None:
    for name, (res, args) in _SIGS.items():
        fn = getattr(l, name, None)
        if fn is None:
            continue
        fn.restype, fn.argtypes = res, args


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str) -> None:
    if code != 0:
        raise NativeError(f"{what} failed with code {code}"
                          + (f" ({torch.cuda.get_device_name()})" if torch.cuda.is_available() else ""))


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def launch_count() -> int:
    return int(lib().tlm_launch_count())


def reset_launch_count() -> None:
    lib().tlm_reset_launch_count()


def add_launch_count(n: int) -> None:
    """Account for kernels launched by replaying a recorded CUDA graph."""
    lib().tlm_add_launch_count(int(n))


def set_deterministic(on: bool) -> None:
    """Deterministic kernels: the split-K weight-gradient GEMM (fp32 `red.global`, order-dependent rounding) is
    replaced by the single-pass accumulate. The attention backward's dQ reduction and the MoE / embedding
    scatter-adds still sum in hardware order."""
    lib().tlm_set_deterministic(int(bool(on)))


def set_gemm_pairs(mode) -> int:
    """Plain GEMMs of at least 256 rows, and row-grouped GEMMs with large groups, run as CTA pairs (`cta_group::2`, one
    256 x 256 tile per two SMs). `mode`: 0 / False off (also `TLM_GEMM_PAIR=0`), 1 / True on (the default), 2 on and
    also for row-grouped GEMMs with small groups. Returns the previous mode. For tests and A/B measurements."""
    return int(lib().tlm_gemm_set_pair(int(mode)))


def take_device_status() -> int:
    """Nonzero when a kernel gave up on a bounded wait since the last call
    (`site << 8 | detail`). Call after synchronising."""
    return int(lib().tlm_take_device_status())


def raise_on_device_status() -> None:
    torch.cuda.synchronize()
    st = take_device_status()
    if st:
        raise NativeError(describe_status(st))


def describe_status(st: int) -> str:
    site, detail = st >> 8, st & 0xff
    if site == SITE_CE_UPSTREAM_GRAD:
        return ("linear_cross_entropy: the gradient that reached the fused LM-head loss differs from the "
                "grad_scale it was given (the loss was rescaled after the op); its gradients are wrong")
    return f"a kernel timed out waiting at site {site} (detail {detail})"


SITE_CE_UPSTREAM_GRAD = 70


def expect_close(a: torch.Tensor, b: torch.Tensor, rel_tol: float, site: int) -> None:
    """Device-side contract check of two 0-d fp32 CUDA tensors (no host sync): if they differ by more than
    `rel_tol` relatively, the device status word gets `site << 8 | 2`, which `take_device_status()` (and the
    trainer after each step) reports."""
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_cuda and b.is_cuda
    _check(lib().tlm_expect_close(a.data_ptr(), b.data_ptr(), float(rel_tol), int(site), _stream()), "expect_close")


def wait_flag(flag: torch.Tensor, expect: int, limit_s: float) -> None:
    """Queue a bounded device-side wait for `flag[0] >= expect` (int32 tensor) on the current stream.
    If the limit passes first the kernel returns anyway and `take_device_status()` reports site 42."""
    assert flag.dtype == torch.int32 and flag.is_cuda
    _check(lib().tlm_wait_flag(flag.data_ptr(), expect, int(limit_s * 1e9), _stream()), "wait_flag")


# --------------------------------------------------------------------------- GEMM
EPI_BF16, EPI_F32_ACC, EPI_F32 = 0, 1, 2


def _rows(t: torch.Tensor) -> tuple[int, int, int]:
    assert t.dim() == 2 and t.stride(1) == 1, "2-D tensor with contiguous rows expected"
    return t.shape[0], t.shape[1], t.stride(0)


def _pad8(t: torch.Tensor, dim: int) -> torch.Tensor:
    """Zero-pad `dim` to a multiple of 8 elements (TMA needs 16-byte row pitches).
    Only tiny operands ever need it (e.g. a router with a number of experts that
    is not a multiple of 8)."""
    n = t.shape[dim]
    if n % 8 == 0:
        return t
    pad = list(t.shape)
    pad[dim] = 8 - n % 8
    return torch.cat([t, t.new_zeros(pad)], dim=dim)


def gemm_nt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M,N] = x[M,K] @ w[N,K]^T (bf16)."""
    if w.shape[0] % 8 and out is None:
        return gemm_nt(x, _pad8(w, 0))[:, :w.shape[0]].contiguous()
    M, K, lda = _rows(x)
    N, K2, ldb = _rows(w)
    assert K == K2
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    _check(lib().tlm_gemm(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, lda, ldb, out.stride(0),
                          0, 0, EPI_BF16, _stream()), "gemm_nt")
    return out


def gemm_nn(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M,K] = dy[M,N] @ w[N,K] (bf16): the data-gradient GEMM. `w` is read in
    place as an MN-major operand, no transpose is materialised."""
    if dy.shape[1] % 8:
        dy, w = _pad8(dy, 1), _pad8(w, 0)
    M, N, lda = _rows(dy)
    N2, K, ldb = _rows(w)
    assert N == N2
    if out is None:
        out = torch.empty(M, K, dtype=torch.bfloat16, device=dy.device)
    _check(lib().tlm_gemm(dy.data_ptr(), w.data_ptr(), out.data_ptr(), M, K, N, lda, ldb, out.stride(0),
                          0, 1, EPI_BF16, _stream()), "gemm_nn")
    return out


def gemm_tn_accum(dy: torch.Tensor, x: torch.Tensor, acc: torch.Tensor) -> None:
    """acc[N,K] (fp32) += dy[M,N]^T @ x[M,K]: the weight-gradient GEMM, both
    operands MN-major, accumulated into the fp32 gradient buffer."""
    if dy.shape[1] % 8:                      # output rows beyond acc.shape[0] are masked by the kernel (M = N rows)
        dy = _pad8(dy, 1)
    M, N, lda = _rows(dy)
    M2, K, ldb = _rows(x)
    N = acc.shape[0]
    assert M == M2 and acc.dtype == torch.float32 and acc.shape[1] == K
    _check(lib().tlm_gemm(dy.data_ptr(), x.data_ptr(), acc.data_ptr(), N, K, M, lda, ldb, acc.stride(0),
                          1, 1, EPI_F32_ACC, _stream()), "gemm_tn_accum")


def heads_epilogue_ok(hd: int, rows_per_batch: int, n_dst: int = 1) -> bool:
    """Shapes the head-scatter GEMM epilogue supports."""
    # head dim 32 only without an exchange (one destination): the attention kernels' scatter forms take 64 / 128
    return (hd in (64, 128) or (hd == 32 and n_dst == 1)) and rows_per_batch % 32 == 0 and 1 <= n_dst <= 8


def rope_table_fp16(cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """`[T, hd]` fp32 cos / sin tables -> `[T, hd, 2]` fp16 (cos, sin) pairs, the table format of the
    head-scatter GEMM epilogue."""
    return torch.stack([cos, sin], dim=-1).to(torch.float16).contiguous()


def gemm_heads(x: torch.Tensor, w: torch.Tensor, b_mn: bool, dst_ptrs, n_dst: int, batch: int, rows_per_batch: int,
               dst_rows: int, dst_heads: int, row_off: int, n_q: int, n_kv: int, q_l: int, kv_l: int, hd: int,
               n_rot: int, cs: torch.Tensor | None, kv_rep: int = 1) -> None:
    """Projection GEMM with the head-scatter epilogue (`csrc/gemm.cu`, `tlm_gemm_heads`):
    `x [batch*rows_per_batch, K]` times `w` (`[N, K]`, or `[K, N]` when `b_mn`), N = (n_q + 2 n_kv) * hd;
    head h of row (b, t) -> RoPE (heads < n_rot, table `cs` from `rope_table_fp16`) ->
    `dst[owner(h)][b, row_off + t, slot(h), :]`.
    `dst_ptrs` is a ctypes array of `n_dst` device addresses (this rank's own tensor or peers' buffers).
    `kv_rep > 1` (fewer KV heads than destinations): k / v head j goes to the `kv_rep` destinations
    `j * kv_rep .. j * kv_rep + kv_rep - 1`, slots `q_l` and `q_l + 1`."""
    M, K, lda = _rows(x)
    if b_mn:
        K2, N, ldb = _rows(w)
    else:
        N, K2, ldb = _rows(w)
    assert K == K2 and M == batch * rows_per_batch
    assert cs is None or (cs.dtype == torch.float16 and cs.shape == (rows_per_batch, hd, 2) and cs.is_contiguous())
    _check(lib().tlm_gemm_heads(x.data_ptr(), w.data_ptr(), M, N, K, lda, ldb, int(b_mn), dst_ptrs, n_dst, batch,
                                rows_per_batch, dst_rows, dst_heads, row_off, n_q, n_kv, q_l, kv_l, hd, n_rot,
                                _ptr(cs), int(kv_rep), _stream()), "gemm_heads")


def swiglu_epilogue_ok(I: int) -> bool:
    return I % 128 == 0


def gemm_swiglu(x: torch.Tensor, w_gu: torch.Tensor):
    """`gate_up = x @ w_gu^T` (`w_gu` = `[2 I, K]`, gate rows then up rows) and `act = silu(gate) * up`
    from one kernel. Returns `(gate_up [M, 2 I], act [M, I])`, both bf16."""
    M, K, lda = _rows(x)
    N2, K2, ldb = _rows(w_gu)
    I = N2 // 2
    assert K == K2 and N2 % 2 == 0 and swiglu_epilogue_ok(I)
    gu = torch.empty(M, N2, dtype=torch.bfloat16, device=x.device)
    act = torch.empty(M, I, dtype=torch.bfloat16, device=x.device)
    _check(lib().tlm_gemm_swiglu(x.data_ptr(), w_gu.data_ptr(), gu.data_ptr(), act.data_ptr(), M, I, K, lda, ldb,
                                 _stream()), "gemm_swiglu")
    return gu, act


def gemm_swiglu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    """`d(gate_up) [M, 2 I]` from `dy [M, D]`, `w_down [D, I]` and the saved `gate_up`: the data-gradient
    GEMM `dy @ w_down` with the SwiGLU derivative in its epilogue."""
    M, D, lda = _rows(dy)
    D2, I, ldb = _rows(w_down)
    assert D == D2 and gu.shape == (M, 2 * I) and gu.is_contiguous() and gu.dtype == torch.bfloat16
    dgu = torch.empty_like(gu)
    _check(lib().tlm_gemm_swiglu_bwd(dy.data_ptr(), w_down.data_ptr(), gu.data_ptr(), dgu.data_ptr(), M, I, D, lda, ldb,
                                     _stream()), "gemm_swiglu_bwd")
    return dgu


def gemm_raw(a, b, c, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi) -> None:
    _check(lib().tlm_gemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, lda, ldb, ldc, a_mn, b_mn, epi,
                          _stream()), "gemm")


# --------------------------------------------------------------------------- elementwise
def embedding_fwd(idx: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    idx = idx.reshape(-1).contiguous()
    rows, D = idx.numel(), weight.shape[1]
    out = torch.empty(rows, D, dtype=torch.float32, device=weight.device)
    _check(lib().tlm_embedding_fwd(idx.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, D, weight.shape[0], _stream()), "embedding_fwd")
    return out


def embedding_bwd(idx: torch.Tensor, dx: torch.Tensor, main_grad: torch.Tensor) -> None:
    idx = idx.reshape(-1).contiguous()
    rows, D = dx.shape
    _check(lib().tlm_embedding_bwd(idx.data_ptr(), dx.data_ptr(), main_grad.data_ptr(), rows, D, main_grad.shape[0], _stream()), "embedding_bwd")


def add_rmsnorm_fwd(x: torch.Tensor, delta: torch.Tensor | None, w: torch.Tensor, eps: float):
    rows, D = x.shape
    x = x.contiguous()
    x_new = torch.empty_like(x) if delta is not None else x
    h = torch.empty(rows, D, dtype=torch.bfloat16, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    if delta is not None:
        delta = delta.contiguous()
    _check(lib().tlm_add_rmsnorm_fwd(x.data_ptr(), _ptr(delta), w.data_ptr(), x_new.data_ptr(), h.data_ptr(),
                                     rstd.data_ptr(), rows, D, eps, _stream()), "add_rmsnorm_fwd")
    return x_new, h, rstd


def add_rmsnorm_bwd(g_xnew, g_h, x_new, rstd, w, main_grad, has_delta: bool):
    rows, D = x_new.shape
    if g_h is None:
        g_h = torch.zeros(rows, D, dtype=torch.bfloat16, device=x_new.device)
    g_h = g_h.contiguous()
    if g_xnew is not None:
        g_xnew = g_xnew.contiguous()
    g_x = torch.empty(rows, D, dtype=torch.float32, device=x_new.device)
    g_delta = torch.empty(rows, D, dtype=torch.bfloat16, device=x_new.device) if has_delta else None
    _check(lib().tlm_add_rmsnorm_bwd(_ptr(g_xnew), g_h.data_ptr(), x_new.data_ptr(), rstd.data_ptr(), w.data_ptr(),
                                     g_x.data_ptr(), _ptr(g_delta), main_grad.data_ptr(), rows, D, _stream()),
           "add_rmsnorm_bwd")
    return g_x, g_delta


def rope_qk(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot: int, inverse: bool) -> torch.Tensor:
    """In place on a contiguous `[B, T, H, hd]` bf16 tensor."""
    assert qkv.is_contiguous()
    B, T, H, hd = qkv.shape
    _check(lib().tlm_rope(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), B * T, T, H, n_rot, hd, int(inverse),
                          _stream()), "rope")
    return qkv


def swiglu_fwd(gu: torch.Tensor, valid_rows: torch.Tensor | None = None) -> torch.Tensor:
    """`valid_rows` (optional 1-element int64 device tensor): only that many leading rows are computed."""
    gu = gu.contiguous()
    rows, two_i = gu.shape
    act = torch.empty(rows, two_i // 2, dtype=torch.bfloat16, device=gu.device)
    _check(lib().tlm_swiglu_fwd(gu.data_ptr(), act.data_ptr(), rows, two_i // 2, _ptr(valid_rows), _stream()), "swiglu_fwd")
    return act


def swiglu_bwd(dact: torch.Tensor, gu: torch.Tensor, valid_rows: torch.Tensor | None = None) -> torch.Tensor:
    rows, two_i = gu.shape
    dgu = torch.empty_like(gu)
    _check(lib().tlm_swiglu_bwd(dact.data_ptr(), gu.data_ptr(), dgu.data_ptr(), rows, two_i // 2, _ptr(valid_rows),
                                _stream()), "swiglu_bwd")
    return dgu


def ce_fwd_bwd_inplace(logits, targets, grad_scale, loss_sum, ignore_index: int, write_grad: bool) -> None:
    rows, V = logits.shape
    if not torch.is_tensor(grad_scale):
        grad_scale = torch.tensor(float(grad_scale), dtype=torch.float32, device=logits.device)
    _check(lib().tlm_ce_inplace(logits.data_ptr(), targets.data_ptr(), grad_scale.data_ptr(), loss_sum.data_ptr(),
                                rows, V, logits.stride(0), ignore_index, int(write_grad), _stream()), "ce_inplace")


def linear_cross_entropy_sum(h: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100,
                             want_lse: bool = False):
    """`sum_i CE(h_i @ weight^T, target_i)` over the valid rows WITHOUT logits in memory: the logits GEMM's epilogue
    keeps a (max, sum-of-exp) pair per row and 256-column tile plus the target logit, a second kernel folds them
    (`csrc/gemm.cu` EPI_LSE, `csrc/elementwise.cu` lse_finish_kernel). Side buffers: 8 bytes per row and tile
    (V = 50304: 1.6 KB per row instead of 100 KB of logits). Returns the loss sum (0-d fp32) and, with `want_lse`,
    the per-row log-sum-exp. Forward only (evaluation, or the first pass of a recomputing backward)."""
    M, K, lda = _rows(h)
    V, K2, ldb = _rows(weight)
    assert K == K2 and targets.numel() == M and targets.dtype == torch.int64
    tiles = (V + 255) // 256
    part = torch.empty(M, tiles, 2, dtype=torch.float32, device=h.device)
    tgt = torch.zeros(M, dtype=torch.float32, device=h.device)
    loss = torch.zeros((), dtype=torch.float32, device=h.device)
    lse = torch.empty(M, dtype=torch.float32, device=h.device) if want_lse else None
    t = targets.contiguous()
    _check(lib().tlm_gemm_lse(h.data_ptr(), weight.data_ptr(), M, V, K, lda, ldb, part.data_ptr(), t.data_ptr(),
                              tgt.data_ptr(), _stream()), "gemm_lse")
    _check(lib().tlm_lse_finish(part.data_ptr(), tiles, tgt.data_ptr(), t.data_ptr(), ignore_index, V, _ptr(lse),
                                loss.data_ptr(), M, _stream()), "lse_finish")
    return (loss, lse) if want_lse else loss


def gemm_dlogits(h: torch.Tensor, weight: torch.Tensor, lse: torch.Tensor, targets: torch.Tensor, scale: torch.Tensor,
                 ignore_index: int = -100, out: torch.Tensor | None = None) -> torch.Tensor:
    """`scale * (softmax(h @ weight^T) - onehot(targets))` as bf16 `[M, V]` from the rows' log-sum-exp: the logits
    are recomputed by the GEMM and turned into their gradient in its epilogue (rows with an ignored target give 0)."""
    M, K, lda = _rows(h)
    V, K2, ldb = _rows(weight)
    assert K == K2 and V % 8 == 0 and lse.dtype == torch.float32 and lse.numel() == M and scale.dtype == torch.float32
    if out is None:
        out = torch.empty(M, V, dtype=torch.bfloat16, device=h.device)
    _check(lib().tlm_gemm_dlogits(h.data_ptr(), weight.data_ptr(), out.data_ptr(), M, V, K, lda, ldb, out.stride(0),
                                  lse.data_ptr(), targets.data_ptr(), scale.data_ptr(), ignore_index, _stream()),
           "gemm_dlogits")
    return out


_SUMSQ_SCRATCH: dict = {}


def sumsq(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    dev = x.device
    if dev not in _SUMSQ_SCRATCH:
        _SUMSQ_SCRATCH[dev] = torch.empty(lib().tlm_sumsq_scratch_floats(), dtype=torch.float32, device=dev)
    out = torch.empty((), dtype=torch.float32, device=dev)
    _check(lib().tlm_sumsq(x.data_ptr(), x.numel(), _SUMSQ_SCRATCH[dev].data_ptr(), out.data_ptr(), _stream()), "sumsq")
    return out


def adam_hyper(step: int, lr: float, beta1: float, beta2: float) -> tuple[float, float, float]:
    """(lr, 1/(1-beta1^t), 1/sqrt(1-beta2^t)): the per-step scalars of the AdamW kernels."""
    import math
    return float(lr), 1.0 / (1.0 - beta1 ** step), 1.0 / math.sqrt(1.0 - beta2 ** step)


def adamw_step(master, exp_avg, exp_avg_sq, grad, param_out, scale, step: int, lr, beta1, beta2, eps, wd,
               hyper: torch.Tensor | None = None) -> None:
    """`hyper` (3 fp32 on the device, see `adam_hyper`) replaces lr and the bias corrections when given."""
    lr_, inv_bc1, inv_sqrt_bc2 = adam_hyper(max(step, 1), lr, beta1, beta2)
    _check(lib().tlm_adamw(master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad.data_ptr(),
                           param_out.data_ptr(), scale.data_ptr(), master.numel(), lr_, beta1, beta2, eps, wd,
                           inv_bc1, inv_sqrt_bc2, _ptr(hyper), _stream()), "adamw")


# --------------------------------------------------------------------------- attention
def flash_attn_fwd(qkv: torch.Tensor, n_q: int, n_kv: int, causal: bool):
    from . import attention_cuda
    return attention_cuda.fwd(qkv, n_q, n_kv, causal)


def flash_attn_bwd(do, qkv, o, lse, n_q: int, n_kv: int, causal: bool, rope=None):
    """`rope = (cos, sin)` (fp32 `[T, hd]` tables): also apply the transposed rotation to dQ and dK, i.e. return
    the gradient of the un-rotated q and k (done in fp32 as the gradients leave the kernels)."""
    from . import attention_cuda
    return attention_cuda.bwd(do, qkv, o, lse, n_q, n_kv, causal, rope)


# --------------------------------------------------------------------------- grouped GEMMs (MoE experts)
class DeviceCounts:
    """Row grouping known only on the device: `row_start` int32 `[groups + 1]`
    plus a host-side upper bound of the rows of any one group."""

    def __init__(self, row_start: torch.Tensor, max_rows: int):
        self.row_start, self.max_rows = row_start, int(max_rows)


def _grouping(counts, device):
    if isinstance(counts, DeviceCounts):
        return counts.row_start, counts.max_rows
    return _row_start(counts, device), max(int(c) for c in counts)


def _row_start(counts, device) -> torch.Tensor:
    acc, out = 0, [0]
    for c in counts:
        acc += int(c)
        out.append(acc)
    return torch.tensor(out, dtype=torch.int32, device=device)


def grouped_gemm_nt(x: torch.Tensor, weight: torch.Tensor, counts) -> torch.Tensor:
    """rows of `x [R,K]` grouped by expert (`counts`); out[rows_e] = x[rows_e] @ weight[e]^T, weight `[E,N,K]`."""
    R, K, lda = _rows(x)
    E, N, K2 = weight.shape
    assert K == K2 and weight.is_contiguous()
    out = torch.empty(R, N, dtype=torch.bfloat16, device=x.device)
    if R == 0:
        return out
    rs, bound = _grouping(counts, x.device)
    _check(lib().tlm_gemm_grouped_rows(x.data_ptr(), weight.data_ptr(), out.data_ptr(), rs.data_ptr(), E, R, N, K,
                                       lda, K, N * K, N, 0, EPI_BF16, bound, _stream()),
           "grouped_gemm_nt")
    return out


def grouped_gemm_nn(dy: torch.Tensor, weight: torch.Tensor, counts) -> torch.Tensor:
    """dx[rows_e] = dy[rows_e] @ weight[e]  (dy `[R,N]`, weight `[E,N,K]` -> `[R,K]`)."""
    R, N, lda = _rows(dy)
    E, N2, K = weight.shape
    assert N == N2 and weight.is_contiguous()
    out = torch.empty(R, K, dtype=torch.bfloat16, device=dy.device)
    if R == 0:
        return out
    rs, bound = _grouping(counts, dy.device)
    _check(lib().tlm_gemm_grouped_rows(dy.data_ptr(), weight.data_ptr(), out.data_ptr(), rs.data_ptr(), E, R, K, N,
                                       lda, K, N * K, K, 1, EPI_BF16, bound, _stream()),
           "grouped_gemm_nn")
    return out


def grouped_gemm_tn_accum(dy: torch.Tensor, x: torch.Tensor, acc: torch.Tensor, counts) -> None:
    """acc[e] (`[E,N,K]` fp32) += dy[rows_e]^T @ x[rows_e]."""
    R, N, lda = _rows(dy)
    R2, K, ldb = _rows(x)
    E = acc.shape[0]
    assert R == R2 and acc.shape == (E, N, K) and acc.dtype == torch.float32 and acc.is_contiguous()
    if R == 0:
        return
    rs, _ = _grouping(counts, dy.device)
    _check(lib().tlm_gemm_grouped_k(dy.data_ptr(), x.data_ptr(), acc.data_ptr(), rs.data_ptr(), E, R, N, K, lda, ldb,
                                    K, N * K, EPI_F32_ACC, _stream()), "grouped_gemm_tn_accum")


def grouped_gemm_nt_scatter(x: torch.Tensor, weight: torch.Tensor, counts, dest_rank: torch.Tensor,
                            dest_row: torch.Tensor, dst_ptrs, n_dst: int, dst_rows: int) -> None:
    """Like `grouped_gemm_nt`, but output row r is stored into `dst[dest_rank[r]][dest_row[r], :]`
    (bf16 `[dst_rows, N]` buffers given by device address; rows with `dest_rank < 0` are dropped)."""
    R, K, lda = _rows(x)
    E, N, K2 = weight.shape
    assert K == K2 and weight.is_contiguous() and dest_rank.dtype == torch.int32 and dest_row.dtype == torch.int64
    if R == 0:
        return
    rs, bound = _grouping(counts, x.device)
    _check(lib().tlm_gemm_grouped_rows_scatter(x.data_ptr(), weight.data_ptr(), rs.data_ptr(), E, R, N, K, lda, K, N * K,
                                               N, 0, bound, dest_rank.data_ptr(), dest_row.data_ptr(), dst_ptrs, n_dst,
                                               dst_rows, _stream()), "grouped_gemm_nt_scatter")


# --------------------------------------------------------------------------- MoE routing and row movement
def moe_route(logits: torch.Tensor, k: int):
    """Top-k routing of `[M, E]` bf16 logits on the device. Returns
    `(weights [M,k] fp32, experts [M,k] int32, counts [E] int32, base [E+1] int32, pos [M*k] int32,
    order [M*k] int32)`: `pos[p]` is the place of pair p = token*k + slot in expert-major / token-minor
    order, `order` its inverse, `base[e]` the first place of expert e."""
    M, E = logits.shape
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    dev = logits.device
    i32 = dict(dtype=torch.int32, device=dev)
    weights = torch.empty(M, k, dtype=torch.float32, device=dev)
    experts = torch.empty(M, k, **i32)
    hist = torch.empty(max(1, lib().tlm_moe_route_blocks(M)) * E, **i32)
    counts, base = torch.empty(E, **i32), torch.empty(E + 1, **i32)
    pos, order = torch.empty(M * k, **i32), torch.empty(M * k, **i32)
    _check(lib().tlm_moe_route(logits.data_ptr(), logits.stride(0), M, E, k, weights.data_ptr(), experts.data_ptr(),
                               hist.data_ptr(), counts.data_ptr(), base.data_ptr(), pos.data_ptr(), order.data_ptr(),
                               _stream()), "moe_route")
    return weights, experts, counts, base, pos, order


def moe_plan(table: torch.Tensor, ep: int, me: int, experts: torch.Tensor, order: torch.Tensor, my_start: torch.Tensor):
    """Expert-parallel routing plan from the all-ranks count table `[ep, E]` int32 (`csrc/moe.cu`,
    `moe_plan_kernel`). Returns a dict: `send_rank [P]` int32, `send_row [P]` int64 (where each of this rank's
    sorted pairs lands), `row_start [E/ep + 1]` int32 and `n_recv [1]` int64 (row ranges of this rank's experts in
    its receive buffer), `back_rank [R]` int32 / `back_row [R]` int64 (the way back of every received row,
    `R = ep * P`, rank -1 past `n_recv`)."""
    E = table.numel() // ep
    P = order.numel()
    R = ep * P
    dev = table.device
    out = {"send_rank": torch.empty(P, dtype=torch.int32, device=dev), "send_row": torch.empty(P, dtype=torch.int64, device=dev),
           "row_start": torch.empty(E // ep + 1, dtype=torch.int32, device=dev), "n_recv": torch.empty(1, dtype=torch.int64, device=dev),
           "back_rank": torch.empty(R, dtype=torch.int32, device=dev), "back_row": torch.empty(R, dtype=torch.int64, device=dev),
           "P": P, "R": R}
    _check(lib().tlm_moe_plan(table.data_ptr(), ep, E, me, experts.data_ptr(), order.data_ptr(), my_start.data_ptr(), P, R,
                              out["send_rank"].data_ptr(), out["send_row"].data_ptr(), out["row_start"].data_ptr(),
                              out["n_recv"].data_ptr(), out["back_rank"].data_ptr(), out["back_row"].data_ptr(), _stream()),
           "moe_plan")
    return out


def moe_route_bwd(dw: torch.Tensor, w: torch.Tensor, experts: torch.Tensor, M: int, E: int) -> torch.Tensor:
    d_logits = torch.zeros(M, E, dtype=torch.bfloat16, device=w.device)
    _check(lib().tlm_moe_route_bwd(dw.contiguous().data_ptr(), w.data_ptr(), experts.data_ptr(), d_logits.data_ptr(), E, M,
                                   w.shape[1], _stream()), "moe_route_bwd")
    return d_logits


def moe_gather(x: torch.Tensor, order: torch.Tensor, k: int, scale: torch.Tensor | None = None) -> torch.Tensor:
    """`out[i] = scale[order[i]] * x[order[i] // k]` (bf16 rows)."""
    P, D = order.numel(), x.shape[1]
    out = torch.empty(P, D, dtype=torch.bfloat16, device=x.device)
    _check(lib().tlm_moe_gather(x.data_ptr(), order.data_ptr(), k, _ptr(scale), out.data_ptr(), P, D, _stream()), "moe_gather")
    return out


def moe_combine(y: torch.Tensor, pos: torch.Tensor, w: torch.Tensor | None, M: int, k: int) -> torch.Tensor:
    """`out[t] = sum_s w[t,s] * y[pos[t*k+s]]` (`w=None`: plain sum)."""
    D = y.shape[1]
    out = torch.empty(M, D, dtype=torch.bfloat16, device=y.device)
    _check(lib().tlm_moe_combine(y.data_ptr(), pos.data_ptr(), _ptr(w), out.data_ptr(), M, D, k, _stream()), "moe_combine")
    return out


def moe_pair_dot(d_out: torch.Tensor, y: torch.Tensor, pos: torch.Tensor, k: int) -> torch.Tensor:
    """`dw[p] = <d_out[p // k], y[pos[p]]>` -> `[P]` fp32."""
    P, D = pos.numel(), y.shape[1]
    dw = torch.empty(P, dtype=torch.float32, device=y.device)
    _check(lib().tlm_moe_pair_dot(d_out.data_ptr(), y.data_ptr(), pos.data_ptr(), dw.data_ptr(), P, D, k, _stream()),
           "moe_pair_dot")
    return dw


def grouped_swiglu_ok(I: int) -> bool:
    return I % 128 == 0


def grouped_gemm_swiglu(x: torch.Tensor, w_pair: torch.Tensor, counts):
    """MoE gate | up + SwiGLU in one grouped GEMM: `w_pair [2E, I, D]` (gate matrices, then up matrices); for the rows
    of group e, `gate_up = [x @ w_pair[e]^T | x @ w_pair[E + e]^T]` and `act = silu(gate) * up`.
    Returns `(gate_up [R, 2 I], act [R, I])`; rows outside every group are left untouched."""
    R, D, lda = _rows(x)
    E2, I, D2 = w_pair.shape
    assert D == D2 and E2 % 2 == 0 and w_pair.is_contiguous() and grouped_swiglu_ok(I)
    gu = torch.empty(R, 2 * I, dtype=torch.bfloat16, device=x.device)
    act = torch.empty(R, I, dtype=torch.bfloat16, device=x.device)
    if R == 0:
        return gu, act
    rs, bound = _grouping(counts, x.device)
    _check(lib().tlm_gemm_swiglu_grouped(x.data_ptr(), w_pair.data_ptr(), gu.data_ptr(), act.data_ptr(), rs.data_ptr(),
                                         E2 // 2, R, I, D, lda, I * D, bound, _stream()), "grouped_gemm_swiglu")
    return gu, act


def grouped_gemm_swiglu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor, counts) -> torch.Tensor:
    """`d(gate_up) [R, 2 I]` for the rows of each group e from `dy [R, D]`, `w_down [E, D, I]` and the saved `gate_up`:
    the grouped data-gradient GEMM `dy @ w_down[e]` with the SwiGLU derivative in its epilogue."""
    R, D, lda = _rows(dy)
    E, D2, I = w_down.shape
    assert D == D2 and w_down.is_contiguous() and gu.shape == (R, 2 * I) and gu.is_contiguous()
    dgu = torch.empty_like(gu)
    if R == 0:
        return dgu
    rs, bound = _grouping(counts, dy.device)
    _check(lib().tlm_gemm_swiglu_bwd_grouped(dy.data_ptr(), w_down.data_ptr(), gu.data_ptr(), dgu.data_ptr(), rs.data_ptr(),
                                             E, R, I, D, lda, D * I, bound, _stream()), "grouped_gemm_swiglu_bwd")
    return dgu


def grouped_pair_ok(I: int) -> bool:
    return I % 256 == 0


def grouped_gemm_pair_fwd(x: torch.Tensor, w_pair: torch.Tensor, counts) -> torch.Tensor:
    """MoE gate | up in one grouped GEMM: `w_pair [2E, I, D]` (gate matrices, then up matrices);
    rows of group e -> `[x @ w_pair[e]^T | x @ w_pair[E + e]^T]`, result `[R, 2 I]`."""
    R, D, lda = _rows(x)
    E2, I, D2 = w_pair.shape
    assert D == D2 and E2 % 2 == 0 and w_pair.is_contiguous() and grouped_pair_ok(I)
    out = torch.empty(R, 2 * I, dtype=torch.bfloat16, device=x.device)
    if R == 0:
        return out
    rs, bound = _grouping(counts, x.device)
    _check(lib().tlm_gemm_grouped_pair(x.data_ptr(), w_pair.data_ptr(), out.data_ptr(), rs.data_ptr(), E2 // 2, R, I, D, lda,
                                       I * D, 2 * I, 0, bound, _stream()), "grouped_gemm_pair_fwd")
    return out


def grouped_gemm_pair_dgrad(dgu: torch.Tensor, w_pair: torch.Tensor, counts) -> torch.Tensor:
    """`dx [R, D] = dgu[:, :I] @ w_pair[e] + dgu[:, I:] @ w_pair[E + e]` for the rows of each group e."""
    R, I2, lda = _rows(dgu)
    E2, I, D = w_pair.shape
    assert I2 == 2 * I and w_pair.is_contiguous()
    out = torch.empty(R, D, dtype=torch.bfloat16, device=dgu.device)
    if R == 0:
        return out
    rs, bound = _grouping(counts, dgu.device)
    _check(lib().tlm_gemm_grouped_pair(dgu.data_ptr(), w_pair.data_ptr(), out.data_ptr(), rs.data_ptr(), E2 // 2, R, I, D, lda,
                                       I * D, D, 1, bound, _stream()), "grouped_gemm_pair_dgrad")
    return out
