"""Differentiable ops used by the model. Each op is a `torch.autograd.Function`
with a hand-written backward, so the same graph runs on both execution paths:

  * CUDA + bf16 parameters  -> the sm_100a kernels in `ops.native`
    (one implementation per op; a missing extension raises);
  * everything else (CPU / fp32) -> the torch expressions written here, which
    restate exactly what the kernels compute and double as their test oracle.

Weight gradients are not returned through autograd. Every parameter carries a
`main_grad` fp32 view into the flat gradient buffer (see `parallel.flat`), and
the backward of an op ACCUMULATES into it (`+=`), which is what the wgrad GEMM
epilogue does on the GPU. Gradient accumulation over micro-steps and the tied
embedding / LM-head weight therefore need no extra pass.
"""
from __future__ import annotations

import math

import torch

from . import oracle
from . import native


def _use_native(x: torch.Tensor, w: torch.Tensor | None = None) -> bool:
    if not x.is_cuda:
        return False
    ref = w if w is not None else x
    return ref.dtype == torch.bfloat16


def _main_grad(p: torch.Tensor) -> torch.Tensor:
    mg = getattr(p, "main_grad", None)
    if mg is None:
        mg = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        p.main_grad = mg
    return mg


# --------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight):
        ctx.save_for_backward(idx)
        ctx.weight = weight
        if _use_native(weight):
            return native.embedding_fwd(idx, weight)
        return weight[idx.reshape(-1)].float()

    @staticmethod
    def backward(ctx, dx):
        (idx,) = ctx.saved_tensors
        mg = _main_grad(ctx.weight)
        if _use_native(ctx.weight):
            native.embedding_bwd(idx, dx.contiguous(), mg)
        else:
            mg.index_add_(0, idx.reshape(-1), dx.float())
        return None, None


def embedding(idx: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Token embedding -> fp32 residual stream `[B*T, D]`."""
    return _Embedding.apply(idx, weight)


# --------------------------------------------------------------------------- residual add + RMSNorm
class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        if _use_native(x, weight):
            x_new, h, rstd = native.add_rmsnorm_fwd(x, delta, weight, eps)
        else:
            x_new = x if delta is None else x + delta.float()
            rstd = torch.rsqrt(x_new.pow(2).mean(-1, keepdim=True) + eps)
            h = (weight.float() * (x_new * rstd)).to(weight.dtype)
        ctx.save_for_backward(x_new, rstd)
        ctx.weight = weight
        ctx.has_delta = delta is not None
        ctx.delta_dtype = delta.dtype if delta is not None else None
        return x_new, h

    @staticmethod
    def backward(ctx, g_xnew, g_h):
        x_new, rstd = ctx.saved_tensors
        w = ctx.weight
        mg = _main_grad(w)
        if _use_native(x_new, w):
            g_x, g_delta = native.add_rmsnorm_bwd(
                g_xnew, g_h, x_new, rstd, w, mg, ctx.has_delta)
        else:
            xhat = x_new * rstd
            gh = g_h.float() if g_h is not None else torch.zeros_like(x_new)
            mg.add_((gh * xhat).sum(0))
            gxh = gh * w.float()
            dx = rstd * (gxh - xhat * (gxh * xhat).mean(-1, keepdim=True))
            g_x = dx if g_xnew is None else g_xnew + dx
            g_delta = g_x.to(ctx.delta_dtype) if ctx.has_delta else None
        return g_x, g_delta, None, None


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float = 1e-6):
    """`x_new = x + delta` (fp32 residual stream), `h = rmsnorm(x_new) * weight`
    in the compute dtype. Returns `(x_new, h)`."""
    return _AddRMSNorm.apply(x, delta, weight, eps)


# --------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x)
        ctx.weight = weight
        if _use_native(x, weight):
            return native.gemm_nt(x, weight)                    # x[M,K] @ weight[N,K]^T
        return (x.to(weight.dtype) @ weight.t())

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        w = ctx.weight
        mg = _main_grad(w)
        dy = dy.contiguous()
        if _use_native(x, w):
            native.gemm_tn_accum(dy, x, mg)                     # mg[N,K] += dy[M,N]^T @ x[M,K]
            dx = native.gemm_nn(dy, w) if ctx.needs_input_grad[0] else None
        else:
            mg.add_((dy.float().t() @ x.float()))
            dx = (dy.to(w.dtype) @ w) if ctx.needs_input_grad[0] else None
        return dx, None


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Bias-free `x @ weight.T` on 2-D `x`."""
    return _Linear.apply(x, weight)


# --------------------------------------------------------------------------- RoPE on the packed qkv tensor
class _RopeQK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, n_rot_heads):
        # qkv: [B, T, H_total, hd]; rotate the first n_rot_heads heads (q and k).
        ctx.save_for_backward(cos, sin)
        ctx.n = n_rot_heads
        if _use_native(qkv):
            ctx.mark_dirty(qkv)
            return native.rope_qk(qkv, cos, sin, n_rot_heads, False)
        out = qkv.clone()
        out[:, :, :n_rot_heads] = oracle.rope(qkv[:, :, :n_rot_heads], cos, sin).to(qkv.dtype)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        if _use_native(dy):
            return native.rope_qk(dy.contiguous(), cos, sin, ctx.n, True), None, None, None
        dx = dy.clone()
        dx[:, :, :ctx.n] = oracle.rope_bwd(dy[:, :, :ctx.n], cos, sin).to(dy.dtype)
        return dx, None, None, None


def rope_qk(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int) -> torch.Tensor:
    return _RopeQK.apply(qkv, cos, sin, n_rot_heads)


# --------------------------------------------------------------------------- fused QKV projection + RoPE
class _QKVProject(torch.autograd.Function):
    """`h [B*T, D]` -> packed, rotated `[B, T, n_q + 2 n_kv, hd]` in one GEMM:
    the epilogue applies RoPE to the q and k heads while the accumulator is
    still in registers and writes the packed layout that attention reads. The
    backward applies the transposed rotation in place to the incoming gradient
    and runs the weight- and data-gradient GEMMs on it."""

    @staticmethod
    def forward(ctx, h, weight, cos, sin, cs, B, T, n_q, n_kv, hd):
        ctx.save_for_backward(h, cos, sin)
        ctx.weight, ctx.n_rot = weight, n_q + n_kv
        Ht = n_q + 2 * n_kv
        out = torch.empty(B, T, Ht, hd, dtype=torch.bfloat16, device=h.device)
        import ctypes
        dst = (ctypes.c_void_p * 1)(out.data_ptr())
        native.gemm_heads(h, weight, False, dst, 1, B, T, T, Ht, 0, n_q, n_kv, n_q, max(n_kv, 1), hd,
                          n_q + n_kv, cs)
        return out

    @staticmethod
    def backward(ctx, d_rot):
        h, cos, sin = ctx.saved_tensors
        w = ctx.weight
        d = native.rope_qk(d_rot.contiguous(), cos, sin, ctx.n_rot, True)      # in place: the gradient is ours
        d2 = d.view(h.shape[0], -1)
        native.gemm_tn_accum(d2, h, _main_grad(w))
        dh = native.gemm_nn(d2, w) if ctx.needs_input_grad[0] else None
        return dh, None, None, None, None, None, None, None, None, None


class _QKVAttention(torch.autograd.Function):
    """`h [B*T, D]` -> causal GQA attention output `[B, T, n_q, hd]`: the QKV projection with RoPE and the packed
    layout in its epilogue (`_QKVProject`), then flash attention, as ONE autograd node, so that the backward can
    hand the transposed rotation to the attention-backward kernels (dQ is rotated while it is converted from its
    fp32 accumulator, dK as it leaves tensor memory) instead of running a separate pass over the packed gradient."""

    @staticmethod
    def forward(ctx, h, weight, cos, sin, cs, B, T, n_q, n_kv, hd):
        Ht = n_q + 2 * n_kv
        qkv = torch.empty(B, T, Ht, hd, dtype=torch.bfloat16, device=h.device)
        import ctypes
        dst = (ctypes.c_void_p * 1)(qkv.data_ptr())
        native.gemm_heads(h, weight, False, dst, 1, B, T, T, Ht, 0, n_q, n_kv, n_q, max(n_kv, 1), hd, n_q + n_kv, cs)
        o, lse = native.flash_attn_fwd(qkv, n_q, n_kv, True)
        ctx.save_for_backward(h, qkv, o, lse, cos, sin)
        ctx.weight, ctx.meta = weight, (n_q, n_kv)
        return o

    @staticmethod
    def backward(ctx, do):
        h, qkv, o, lse, cos, sin = ctx.saved_tensors
        n_q, n_kv = ctx.meta
        w = ctx.weight
        d = native.flash_attn_bwd(do.contiguous(), qkv, o, lse, n_q, n_kv, True, rope=(cos, sin))
        d2 = d.view(h.shape[0], -1)
        native.gemm_tn_accum(d2, h, _main_grad(w))
        dh = native.gemm_nn(d2, w) if ctx.needs_input_grad[0] else None
        return dh, None, None, None, None, None, None, None, None, None


def qkv_attention(h, weight, cos, sin, cs, B: int, T: int, n_q: int, n_kv: int, hd: int) -> torch.Tensor:
    """CUDA only (same conditions as `qkv_project`): projection + RoPE + causal attention -> `[B, T, n_q, hd]`."""
    return _QKVAttention.apply(h, weight, cos.contiguous(), sin.contiguous(), cs, B, T, n_q, n_kv, hd)


def qkv_project_fused_ok(h: torch.Tensor, weight: torch.Tensor | None, hd: int, T: int) -> bool:
    return weight is not None and _use_native(h, weight) and native.heads_epilogue_ok(hd, T)


def qkv_project(h, weight, cos, sin, cs, B: int, T: int, n_q: int, n_kv: int, hd: int) -> torch.Tensor:
    """CUDA only (check `qkv_project_fused_ok` first). `cs` = `native.rope_table_fp16(cos, sin)`."""
    return _QKVProject.apply(h, weight, cos, sin, cs, B, T, n_q, n_kv, hd)


# --------------------------------------------------------------------------- attention
def _attn_fwd_ref(q, k, v, causal):
    """Returns (out, lse) with fp32 math. q [B,T,Hq,hd], k/v [B,T,Hkv,hd]."""
    B, Tq, Hq, hd = q.shape
    rep = Hq // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(hd)
    if causal:
        mask = torch.ones(Tq, k.shape[1], dtype=torch.bool, device=q.device).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                              # B,Hq,Tq
    p = torch.exp(s - lse[..., None])
    o = (p @ vf).permute(0, 2, 1, 3)
    return o, lse, p, qf, kf, vf


class _Attention(torch.autograd.Function):
    """Causal GQA attention on a packed `[B, T, Hq + 2*Hkv, hd]` tensor."""

    @staticmethod
    def forward(ctx, qkv, n_q, n_kv, causal):
        ctx.n_q, ctx.n_kv, ctx.causal = n_q, n_kv, causal
        if _use_native(qkv):
            o, lse = native.flash_attn_fwd(qkv, n_q, n_kv, causal)
            ctx.save_for_backward(qkv, o)
            ctx.lse = lse
            return o
        q, k, v = qkv[:, :, :n_q], qkv[:, :, n_q:n_q + n_kv], qkv[:, :, n_q + n_kv:]
        o, lse, *_ = _attn_fwd_ref(q, k, v, causal)
        o = o.to(qkv.dtype).contiguous()
        ctx.save_for_backward(qkv, o)
        ctx.lse = lse
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o = ctx.saved_tensors
        lse = ctx.lse
        n_q, n_kv = ctx.n_q, ctx.n_kv
        if _use_native(qkv):
            return native.flash_attn_bwd(do.contiguous(), qkv, o, lse, n_q, n_kv, ctx.causal), None, None, None
        q, k, v = qkv[:, :, :n_q], qkv[:, :, n_q:n_q + n_kv], qkv[:, :, n_q + n_kv:]
        B, T, _, hd = q.shape
        rep = n_q // n_kv
        _, _, p, qf, kf, vf = _attn_fwd_ref(q, k, v, ctx.causal)
        dof = do.float().permute(0, 2, 1, 3)                       # B,Hq,T,hd
        of = o.float().permute(0, 2, 1, 3)
        dv = p.transpose(-1, -2) @ dof
        dp = dof @ vf.transpose(-1, -2)
        delta = (dof * of).sum(-1, keepdim=True)
        ds = p * (dp - delta) / math.sqrt(hd)
        dq = ds @ kf
        dk = ds.transpose(-1, -2) @ qf
        dk = dk.view(B, n_kv, rep, -1, hd).sum(2)
        dv = dv.view(B, n_kv, rep, -1, hd).sum(2)
        dqkv = torch.cat([dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3)], dim=2)
        return dqkv.to(qkv.dtype), None, None, None


def attention_packed(qkv: torch.Tensor, n_q: int, n_kv: int, causal: bool = True) -> torch.Tensor:
    """-> `[B, T, Hq, hd]`"""
    return _Attention.apply(qkv, n_q, n_kv, causal)


# --------------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, valid_rows):
        ctx.save_for_backward(gu)
        ctx.valid_rows = valid_rows
        if _use_native(gu):
            return native.swiglu_fwd(gu, valid_rows)
        return oracle.swiglu(gu).to(gu.dtype)

    @staticmethod
    def backward(ctx, dact):
        (gu,) = ctx.saved_tensors
        if _use_native(gu):
            return native.swiglu_bwd(dact.contiguous(), gu, ctx.valid_rows), None
        g, u = gu.float().chunk(2, dim=-1)
        sig = torch.sigmoid(g)
        d = dact.float()
        dg = d * u * sig * (1.0 + g * (1.0 - sig))
        du = d * g * sig
        return torch.cat([dg, du], dim=-1).to(gu.dtype), None


def swiglu(gate_up: torch.Tensor, valid_rows: torch.Tensor | None = None) -> torch.Tensor:
    """`[M, 2I]` (gate | up) -> `silu(gate) * up` `[M, I]`. `valid_rows` (CUDA only, 1-element int64 device
    tensor): rows past that count are neither read nor written (their content is undefined)."""
    return _SwiGLU.apply(gate_up, valid_rows)


class _SwiGLUMLP(torch.autograd.Function):
    """`down(silu(gate(x)) * up(x))` on CUDA with the SwiGLU math inside GEMM epilogues: the gate|up GEMM also
    emits `act`, and in backward the data-gradient GEMM of the down projection turns d(act) into d(gate|up)
    while the accumulator is still in registers. Five GEMMs forward + backward become the only kernels of the
    MLP (no separate SwiGLU passes, d(act) never reaches memory)."""

    @staticmethod
    def forward(ctx, x, w_gu, w_down):
        gu, act = native.gemm_swiglu(x, w_gu)
        ctx.save_for_backward(x, gu, act)
        ctx.w_gu, ctx.w_down = w_gu, w_down
        return native.gemm_nt(act, w_down)

    @staticmethod
    def backward(ctx, dy):
        x, gu, act = ctx.saved_tensors
        w_gu, w_down = ctx.w_gu, ctx.w_down
        dy = dy.contiguous()
        native.gemm_tn_accum(dy, act, _main_grad(w_down))
        dgu = native.gemm_swiglu_bwd(dy, w_down, gu)
        native.gemm_tn_accum(dgu, x, _main_grad(w_gu))
        dx = native.gemm_nn(dgu, w_gu) if ctx.needs_input_grad[0] else None
        return dx, None, None


def swiglu_mlp_fused_ok(x: torch.Tensor, w_gu: torch.Tensor | None) -> bool:
    return w_gu is not None and _use_native(x, w_gu) and native.swiglu_epilogue_ok(w_gu.shape[0] // 2)


def swiglu_mlp(x: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """CUDA only (check `swiglu_mlp_fused_ok` first). `w_gu` is the fused `[2 I, D]` gate|up weight."""
    return _SwiGLUMLP.apply(x, w_gu, w_down)


# --------------------------------------------------------------------------- fused LM head + cross-entropy
class _LinearCrossEntropy(torch.autograd.Function):
    """`sum_i CE(h_i @ W^T, target_i)` without keeping the `[M, V]` logits.

    The forward walks over row chunks (up to 32768 rows on the GPU: a 3.3 GB bf16 logits workspace for a 50k vocabulary, overwritten in place by its own gradient): logits chunk = GEMM, one kernel turns it
    in place into `grad_scale * (softmax - onehot)` while emitting the chunk's
    loss sum, then dgrad and wgrad GEMMs consume it. So the backward work is
    done during forward and `backward()` only hands out the stored `dh`.
    `grad_scale` (a 0-d fp32 tensor) must be the factor that the caller applies
    to the returned sum to form the final loss (e.g. 1 / (valid tokens * grad
    accumulation steps)); it stays on the device, no host sync is needed.
    Because the weight gradient has already been accumulated with that factor
    when `backward()` runs, the contract is CHECKED there: the incoming
    gradient must equal `grad_scale` (on the CPU path an exception; on CUDA a
    one-thread kernel that records status site 70 in the device status word,
    which the trainer turns into an error at the step's synchronize, without a
    host sync on the hot path).
    """

    RECOMPUTE_CHUNK_ROWS = 4096
    CHUNK_ROWS = 32768         # rows of logits alive at once on the GPU (3.3 GB of bf16 at V = 50304); measured on the
                               # headline step: 8192 rows 176.5 ms, 16384 rows 175.5 ms, 32768 rows 174.8 ms
    CHUNK_ROWS_CPU = 8192      # the fp32 path keeps its transient logits small

    @staticmethod
    def forward(ctx, h, weight, targets, grad_scale, ignore_index):
        M = h.shape[0]
        need_grad = bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])
        if not need_grad and _use_native(h, weight) and weight.shape[0] % 8 == 0:
            # evaluation: the loss needs no logits at all (statistics in the GEMM epilogue, see native)
            ctx.dh = None
            ctx.grad_scale = grad_scale
            return native.linear_cross_entropy_sum(h.contiguous(), weight, targets, ignore_index)
        mg = _main_grad(weight) if need_grad else None
        dh = torch.empty_like(h) if need_grad else None
        use_nat = _use_native(h, weight)
        if use_nat and _lm_head_recompute() and weight.shape[0] % 8 == 0:
            # Memory-lean variant: pass 1 keeps only per-tile statistics (no logits), pass 2 recomputes the logits a
            # chunk of rows at a time and stores them as their own gradient, which feeds the dgrad / wgrad GEMMs.
            # One extra logits GEMM per micro-step instead of the in-place softmax pass; the largest transient is
            # RECOMPUTE_CHUNK_ROWS x V bf16 instead of M x V.
            hc_all = h.contiguous()
            loss_sum, lse = native.linear_cross_entropy_sum(hc_all, weight, targets, ignore_index, want_lse=True)
            gs = grad_scale if torch.is_tensor(grad_scale) else torch.tensor(float(grad_scale), device=h.device)
            gs = gs.reshape(()).float().contiguous()
            step = _LinearCrossEntropy.RECOMPUTE_CHUNK_ROWS
            work = torch.empty(min(step, M), weight.shape[0], dtype=torch.bfloat16, device=h.device)
            for r0 in range(0, M, step):
                r1 = min(M, r0 + step)
                dl = native.gemm_dlogits(hc_all[r0:r1], weight, lse[r0:r1], targets[r0:r1].contiguous(), gs, ignore_index,
                                         out=work[:r1 - r0])
                native.gemm_nn(dl, weight, out=dh[r0:r1])
                native.gemm_tn_accum(dl, hc_all[r0:r1], mg)
            ctx.dh = dh
            ctx.grad_scale = grad_scale
            return loss_sum
        loss_sum = torch.zeros((), dtype=torch.float32, device=h.device)
        step = _LinearCrossEntropy.CHUNK_ROWS if use_nat else _LinearCrossEntropy.CHUNK_ROWS_CPU
        for r0 in range(0, M, step):
            r1 = min(M, r0 + step)
            hc, tc = h[r0:r1], targets[r0:r1]
            if use_nat:
                logits = native.gemm_nt(hc, weight)
                native.ce_fwd_bwd_inplace(logits, tc, grad_scale, loss_sum, ignore_index, need_grad)
                if need_grad:
                    native.gemm_nn(logits, weight, out=dh[r0:r1])
                    native.gemm_tn_accum(logits, hc, mg)
            else:
                logits = hc.to(weight.dtype) @ weight.t()
                lf = logits.float()
                lse = torch.logsumexp(lf, dim=-1)
                valid = tc != ignore_index
                safe_t = tc.clamp(min=0)
                tgt_logit = lf.gather(1, safe_t[:, None]).squeeze(1)
                loss_sum = loss_sum + ((lse - tgt_logit) * valid).sum()
                if need_grad:
                    p = torch.exp(lf - lse[:, None])
                    p[torch.arange(r1 - r0, device=h.device), safe_t] -= 1.0
                    dl = (p * valid[:, None] * grad_scale).to(weight.dtype)
                    dh[r0:r1] = dl @ weight
                    mg.add_(dl.float().t() @ hc.float())
        ctx.dh = dh
        ctx.grad_scale = grad_scale
        return loss_sum

    @staticmethod
    def backward(ctx, g):
        # dh and the accumulated weight gradient already carry grad_scale: the upstream gradient must be it
        dh, ctx.dh = ctx.dh, None
        gs = ctx.grad_scale
        if dh is not None:
            if g.is_cuda and native.available():
                gs_t = gs if torch.is_tensor(gs) else torch.full((), float(gs), dtype=torch.float32, device=g.device)
                native.expect_close(g.reshape(()).float(), gs_t.reshape(()).float().to(g.device), 1e-3,
                                    native.SITE_CE_UPSTREAM_GRAD)
            elif not torch.allclose(g.detach().float().reshape(()).cpu(), torch.as_tensor(gs).float().reshape(()).cpu(),
                                    rtol=1e-3, atol=0.0):
                raise RuntimeError("linear_cross_entropy: the upstream gradient differs from grad_scale; multiply "
                                   "the returned sum by exactly the grad_scale that was passed in")
        return dh, None, None, None, None


def _lm_head_recompute() -> bool:
    """`TLM_LM_HEAD=recompute`: the LM head never holds `[M, V]` logits in training either (see `_LinearCrossEntropy`).
    Default off: at 0.3 B parameters the extra logits GEMM costs more time than the softmax pass it replaces."""
    import os
    return os.environ.get("TLM_LM_HEAD", "inplace") == "recompute"


def linear_cross_entropy(h, weight, targets, grad_scale, ignore_index: int = -100) -> torch.Tensor:
    return _LinearCrossEntropy.apply(h, weight, targets.reshape(-1), grad_scale, ignore_index)


def cross_entropy_from_logits(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100):
    """Unfused path used for evaluation when logits are requested."""
    return oracle.cross_entropy_sum(logits, targets.reshape(-1), ignore_index)
