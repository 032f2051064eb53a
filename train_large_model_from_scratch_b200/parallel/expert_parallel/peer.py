"""Expert-parallel dispatch / combine as direct row stores into peer memory (CUDA).

The NCCL path (`comm.py`, and the reference's `model/modules/mlp.py:104-127,
160-167`) needs the per-rank split sizes on the HOST before it can call
`all_to_all_single`: two device->host syncs per MoE layer. Here nothing leaves
the device:

  1. every rank publishes its per-expert pair counts into all peers' count
     table (`[ep, E]`, symmetric memory) and a flag barrier follows;
  2. from that table each rank derives, with a few tiny device ops,
       - where each of ITS sorted (token, slot) pairs lands in the destination
         rank's receive buffer, which is laid out expert-major / source-minor,
         i.e. already grouped for the expert GEMMs,
       - the row ranges of its own experts (`row_start`, consumed by the grouped
         GEMM's device-side tile scheduler),
       - for every received row, which rank and which sorted-pair slot it came
         from (for the way back);
  3. one kernel stores the rows into the peers' buffers (dispatch); after the
     expert MLP the same kernel returns them (combine). Backward uses the same
     two routes in the opposite roles.

Receive buffers have the worst-case size (`ep * M * k` rows: dropless routing can
send every pair to one rank); rows past the real count are never read.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...ops import native
from ..sequence_parallel.ulysses_peer import _fresh


class PeerMoE:
    _instance = None

    def __init__(self, group, num_experts: int):
        from ..symm import alloc_flags, symm_alloc, _Peer
        self.group, self.ep, self.me = group, dist.get_world_size(group), dist.get_rank(group)
        self.E = num_experts
        self.E_l = num_experts // self.ep
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        self.flags = _Peer(alloc_flags(dev), group)
        self.counts_t = symm_alloc(self.ep * num_experts, torch.int32, dev)
        self.counts = _Peer(self.counts_t, group)
        self.buffers: dict = {}
        dist.barrier(group=group)

    @classmethod
    def get(cls, group, num_experts: int) -> "PeerMoE":
        if cls._instance is None or cls._instance.group is not group or cls._instance.E != num_experts:
            cls._instance = cls(group, num_experts)
        return cls._instance

    def barrier(self) -> None:
        f = self.flags
        native._check(native.lib().tlm_peer_barrier(f.ptr_array, f.rank, f.n, 0, native._stream()), "peer_barrier")

    def buffer(self, key, rows: int, D: int):
        """Receive buffer of `key` for this shape; cached per (key, shape) and never freed, because a recorded
        CUDA graph keeps writing to (and its peers keep addressing) the buffers of the shape it was recorded
        with, while a call with another shape (ragged last batch, evaluation) needs its own."""
        from ..symm import symm_alloc, _Peer
        key = (key, int(rows), int(D))
        b = self.buffers.get(key)
        if b is None:
            t = symm_alloc(rows * D, torch.bfloat16, self.dev).view(rows, D)
            b = (t, _Peer(t, self.group))
            self.buffers[key] = b
        return b

    # ------------------------------------------------------------------ routing
    def plan(self, my_counts: torch.Tensor, experts: torch.Tensor, order: torch.Tensor, my_start: torch.Tensor):
        """`my_counts [E]` int32 (pairs per expert on this rank), `experts [M*k]` / `order [P]` / `my_start [E+1]`
        int32 from `native.moe_route`. Publishes the counts to every peer, then one kernel derives both routes.
        Returns a dict of device tensors. No barrier is needed after the table has been read: the next write into
        it (the next layer's counts) can only happen after the dispatch exchange, which this rank completes after
        its plan kernel."""
        ep, E, E_l, me = self.ep, self.E, self.E_l, self.me
        c32 = my_counts.to(torch.int32).contiguous()
        native._check(native.lib().tlm_peer_put_i32(c32.data_ptr(), E, self.counts.ptr_array, ep, me * E,
                                                    native._stream()), "peer_put_i32")
        self.barrier()
        return native.moe_plan(self.counts_t, ep, me, experts, order, my_start)

    def scatter(self, src: torch.Tensor, dest_rank, dest_row, dst, n_ptr, n_max: int, src_idx=None, src_div: int = 1,
                row_scale=None) -> None:
        """Row i (< *n_ptr) of the route: `dst[dest_rank[i]][dest_row[i]] = scale * src[j // src_div]`,
        `j = src_idx[i]` (or i), `scale = row_scale[j]` (or 1); then the flag barrier."""
        t, peer = dst
        native._check(native.lib().tlm_peer_scatter_rows(
            src.data_ptr(), native._ptr(src_idx), src_div, native._ptr(row_scale), dest_rank.data_ptr(),
            dest_row.data_ptr(), peer.ptr_array, self.ep, src.shape[1], native._ptr(n_ptr), n_max, t.shape[0],
            native._stream()), "peer_scatter_rows")
        self.barrier()


class _Dispatch(torch.autograd.Function):
    """sorted pairs `[P, D]` -> expert-grouped rows on their owners `[R, D]`."""

    @staticmethod
    def forward(ctx, x_sorted, pm: PeerMoE, plan: dict, key):
        dst = pm.buffer((key, "disp"), plan["R"], x_sorted.shape[1])
        pm.scatter(x_sorted.contiguous(), plan["send_rank"], plan["send_row"], dst, None, plan["P"])
        ctx.pm, ctx.plan, ctx.key = pm, plan, key
        return _fresh(dst[0])

    @staticmethod
    def backward(ctx, d_local):
        pm, plan = ctx.pm, ctx.plan
        dst = pm.buffer((ctx.key, "disp_bwd"), plan["P"], d_local.shape[1])
        pm.scatter(d_local.contiguous(), plan["back_rank"], plan["back_row"], dst, plan["n_recv"], plan["R"])
        return _fresh(dst[0]), None, None, None


class _Combine(torch.autograd.Function):
    """expert outputs `[R, D]` -> back to the pairs' owners in sorted order `[P, D]`."""

    @staticmethod
    def forward(ctx, y_local, pm: PeerMoE, plan: dict, key):
        dst = pm.buffer((key, "comb"), plan["P"], y_local.shape[1])
        pm.scatter(y_local.contiguous(), plan["back_rank"], plan["back_row"], dst, plan["n_recv"], plan["R"])
        ctx.pm, ctx.plan, ctx.key = pm, plan, key
        return _fresh(dst[0])

    @staticmethod
    def backward(ctx, d_comb):
        pm, plan = ctx.pm, ctx.plan
        dst = pm.buffer((ctx.key, "comb_bwd"), plan["R"], d_comb.shape[1])
        pm.scatter(d_comb.contiguous(), plan["send_rank"], plan["send_row"], dst, None, plan["P"])
        return _fresh(dst[0]), None, None, None


def dispatch(x_sorted, pm, plan, key):
    return _Dispatch.apply(x_sorted, pm, plan, key)


def combine(y_local, pm, plan, key):
    return _Combine.apply(y_local, pm, plan, key)


class _DispatchTokens(torch.autograd.Function):
    """tokens `[M, D]` -> expert-grouped rows on the experts' owners `[R, D]` in one kernel: row
    `order[i] // k` of `x` is read and stored straight into the destination rank's buffer (no
    sorted copy of the tokens is made). Backward: the rows' gradients return to the token owner in
    sorted-pair order and are summed over each token's k slots."""

    @staticmethod
    def forward(ctx, x, pm: PeerMoE, plan: dict, order, pos, k: int, key):
        dst = pm.buffer((key, "disp"), plan["R"], x.shape[1])
        pm.scatter(x.contiguous(), plan["send_rank"], plan["send_row"], dst, None, plan["P"], src_idx=order, src_div=k)
        ctx.pm, ctx.plan, ctx.key, ctx.k, ctx.M = pm, plan, key, k, x.shape[0]
        ctx.save_for_backward(pos)
        return _fresh(dst[0])

    @staticmethod
    def backward(ctx, d_local):
        pm, plan = ctx.pm, ctx.plan
        (pos,) = ctx.saved_tensors
        dst = pm.buffer((ctx.key, "disp_bwd"), plan["P"], d_local.shape[1])
        pm.scatter(d_local.contiguous(), plan["back_rank"], plan["back_row"], dst, plan["n_recv"], plan["R"])
        return native.moe_combine(dst[0], pos, None, ctx.M, ctx.k), None, None, None, None, None, None


class _DownCombine(torch.autograd.Function):
    """Expert down-projection + combine: the grouped GEMM's epilogue stores every output row into the
    token owner's buffer (`csrc/gemm.cu`, row-scatter epilogue), then the owner forms
    `out[t] = sum_s w[t,s] * row(t,s)`. Backward: weight gradients from the received rows, and
    `w * d_out[token]` is pushed to the experts' owners, where the down-projection's own backward runs."""

    @staticmethod
    def forward(ctx, act, w_down, weights, pm: PeerMoE, plan: dict, per_expert, order, pos, k: int, key):
        D = w_down.shape[1]
        comb = pm.buffer((key, "comb"), plan["P"], D)
        native.grouped_gemm_nt_scatter(act, w_down, per_expert, plan["back_rank"], plan["back_row"],
                                       comb[1].ptr_array, pm.ep, plan["P"])
        pm.barrier()
        M = weights.shape[0]
        out = native.moe_combine(comb[0], pos, weights, M, k)
        ctx.pm, ctx.plan, ctx.key, ctx.k, ctx.per_expert, ctx.w_down = pm, plan, key, k, per_expert, w_down
        ctx.save_for_backward(act, weights, order, pos, comb[0])
        return out

    @staticmethod
    def backward(ctx, d_out):
        from ...ops.functional import _main_grad
        pm, plan, k = ctx.pm, ctx.plan, ctx.k
        act, weights, order, pos, comb = ctx.saved_tensors
        d_out = d_out.contiguous()
        dw = native.moe_pair_dot(d_out, comb, pos, k).view_as(weights)
        dst = pm.buffer((ctx.key, "comb_bwd"), plan["R"], d_out.shape[1])
        pm.scatter(d_out, plan["send_rank"], plan["send_row"], dst, None, plan["P"], src_idx=order, src_div=k,
                   row_scale=weights)
        d_y = dst[0]
        native.grouped_gemm_tn_accum(d_y, act, _main_grad(ctx.w_down), ctx.per_expert)
        d_act = native.grouped_gemm_nn(d_y, ctx.w_down, ctx.per_expert)
        return d_act, None, dw, None, None, None, None, None, None, None


class _ExpertMLPCombine(torch.autograd.Function):
    """Expert MLP + combine on the experts' owner: gate|up GEMM with the SwiGLU epilogue, then the down projection
    whose epilogue stores every output row into the token owner's buffer, where `out[t] = sum_s w[t,s] * row(t,s)` is
    formed. Backward: `w * d_out[token]` is pushed to the experts' owners, and the expert MLP's backward runs there
    with the SwiGLU derivative inside the down projection's data-gradient GEMM."""

    @staticmethod
    def forward(ctx, x_local, w_pair, w_down, weights, pm: PeerMoE, plan: dict, per_expert, order, pos, k: int, key):
        gu, act = native.grouped_gemm_swiglu(x_local, w_pair, per_expert)
        D = w_down.shape[1]
        comb = pm.buffer((key, "comb"), plan["P"], D)
        native.grouped_gemm_nt_scatter(act, w_down, per_expert, plan["back_rank"], plan["back_row"],
                                       comb[1].ptr_array, pm.ep, plan["P"])
        pm.barrier()
        M = weights.shape[0]
        out = native.moe_combine(comb[0], pos, weights, M, k)
        ctx.pm, ctx.plan, ctx.key, ctx.k, ctx.per_expert = pm, plan, key, k, per_expert
        ctx.w_pair, ctx.w_down = w_pair, w_down
        ctx.save_for_backward(x_local, gu, act, weights, order, pos, comb[0])
        return out

    @staticmethod
    def backward(ctx, d_out):
        from ...ops.moe_ops import expert_mlp_backward
        pm, plan, k = ctx.pm, ctx.plan, ctx.k
        x_local, gu, act, weights, order, pos, comb = ctx.saved_tensors
        d_out = d_out.contiguous()
        dw = native.moe_pair_dot(d_out, comb, pos, k).view_as(weights)
        dst = pm.buffer((ctx.key, "comb_bwd"), plan["R"], d_out.shape[1])
        pm.scatter(d_out, plan["send_rank"], plan["send_row"], dst, None, plan["P"], src_idx=order, src_div=k,
                   row_scale=weights)
        dx = expert_mlp_backward(dst[0], x_local, gu, act, ctx.w_pair, ctx.w_down, ctx.per_expert)
        return dx, None, None, dw, None, None, None, None, None, None, None


def expert_mlp_combine(x_local, w_pair, w_down, weights, pm, plan, per_expert, order, pos, k, key):
    return _ExpertMLPCombine.apply(x_local, w_pair, w_down, weights, pm, plan, per_expert, order, pos, k, key)


def dispatch_tokens(x, pm, plan, order, pos, k, key):
    return _DispatchTokens.apply(x, pm, plan, order, pos, k, key)


def down_combine(act, w_down, weights, pm, plan, per_expert, order, pos, k, key):
    return _DownCombine.apply(act, w_down, weights, pm, plan, per_expert, order, pos, k, key)
