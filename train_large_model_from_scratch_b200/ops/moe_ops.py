"""Mixture-of-experts data path: routing, dispatch, grouped expert MLP, combine.

The routing/dispatch bookkeeping is expressed once here in terms of small
building blocks; the CUDA path swaps the heavy blocks (grouped GEMM, SwiGLU,
gather/scatter) for kernels while the control flow stays the same.

Data flow for `M` local tokens, top-`k`, `E` experts over `ep` ranks
(reference: `model/modules/mlp.py:95-169`):

  1. `weights, experts = softmax(topk(logits))`                     [M, k]
  2. sort the M*k (token, slot) pairs by global expert id (stable); because
     experts are laid out rank-major this is also sorted by destination rank
  3. exchange per-(destination, local expert) counts; exchange rows
  4. receiver regroups rows from (source, expert) order to expert order using
     the counts only
  5. per-expert `down(silu(gate x) * up x)` as grouped GEMMs
  6. inverse regroup, rows travel back, un-sort, weighted sum over the k slots
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import functional as F_ops
from . import native
from . import oracle
from ..parallel.expert_parallel.comm import ep_all_to_all, exchange_counts


class _GroupedLinear(torch.autograd.Function):
    """rows of `x` are grouped by expert: rows [offs[e-1], offs[e]) use `weight[e]`
    (`[E, N, K]`, `y = x @ weight[e]^T`). `counts` is a host list."""

    @staticmethod
    def forward(ctx, x, weight, counts):
        ctx.counts = counts
        ctx.weight = weight
        ctx.save_for_backward(x)
        if F_ops._use_native(x, weight):
            return native.grouped_gemm_nt(x, weight, counts)
        out = x.new_empty((x.shape[0], weight.shape[1]), dtype=weight.dtype)
        r = 0
        for e, c in enumerate(counts):
            if c:
                out[r:r + c] = x[r:r + c].to(weight.dtype) @ weight[e].t()
            r += c
        return out

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        w, counts = ctx.weight, ctx.counts
        mg = F_ops._main_grad(w)
        dy = dy.contiguous()
        if F_ops._use_native(x, w):
            native.grouped_gemm_tn_accum(dy, x, mg, counts)
            return native.grouped_gemm_nn(dy, w, counts), None, None
        dx = torch.empty_like(x)
        r = 0
        for e, c in enumerate(counts):
            if c:
                dx[r:r + c] = (dy[r:r + c].to(w.dtype) @ w[e]).to(x.dtype)
                mg[e].add_(dy[r:r + c].float().t() @ x[r:r + c].float())
            r += c
        return dx, None, None


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, counts: list[int]) -> torch.Tensor:
    return _GroupedLinear.apply(x, weight, counts)


class _GroupedGateUp(torch.autograd.Function):
    """Gate and up projections of all local experts as ONE grouped GEMM writing `gate | up` side by side
    (`w_pair [2E, I, D]`: the gate matrices, then the up matrices; they are adjacent in the flat expert buffer).
    Backward: one grouped GEMM with the reduction running over both halves gives `dx` (no separate sum),
    two grouped wgrad GEMMs accumulate into the two halves of the gradient buffer."""

    @staticmethod
    def forward(ctx, x, w_pair, counts):
        ctx.counts, ctx.w_pair = counts, w_pair
        ctx.save_for_backward(x)
        return native.grouped_gemm_pair_fwd(x, w_pair, counts)

    @staticmethod
    def backward(ctx, dgu):
        (x,) = ctx.saved_tensors
        w, counts = ctx.w_pair, ctx.counts
        E, I = w.shape[0] // 2, w.shape[1]
        mg = F_ops._main_grad(w)
        dgu = dgu.contiguous()
        native.grouped_gemm_tn_accum(dgu[:, :I], x, mg[:E], counts)
        native.grouped_gemm_tn_accum(dgu[:, I:], x, mg[E:], counts)
        return native.grouped_gemm_pair_dgrad(dgu, w, counts), None, None


class _ExpertMLP(torch.autograd.Function):
    """The expert MLP on expert-grouped rows, `down_e(silu(gate_e x) * up_e x)`, with the SwiGLU math inside the
    grouped GEMMs' epilogues: forward = gate|up GEMM that also emits `act` + down GEMM; backward = two weight-gradient
    GEMMs, the down projection's data-gradient GEMM whose epilogue turns d(act) into d(gate|up), and one
    K-concatenated data-gradient GEMM for both projections. No stand-alone SwiGLU pass, d(act) never reaches memory."""

    @staticmethod
    def forward(ctx, x, w_pair, w_down, counts):
        gu, act = native.grouped_gemm_swiglu(x, w_pair, counts)
        ctx.save_for_backward(x, gu, act)
        ctx.w_pair, ctx.w_down, ctx.counts = w_pair, w_down, counts
        return native.grouped_gemm_nt(act, w_down, counts)

    @staticmethod
    def backward(ctx, dy):
        x, gu, act = ctx.saved_tensors
        dx = expert_mlp_backward(dy.contiguous(), x, gu, act, ctx.w_pair, ctx.w_down, ctx.counts)
        return dx, None, None, None


def expert_mlp_backward(dy, x, gu, act, w_pair, w_down, counts):
    """Shared by `_ExpertMLP` and the expert-parallel variant (`parallel.expert_parallel.peer`): accumulates the
    three weight gradients into their `main_grad` buffers and returns the gradient of the grouped input rows."""
    E, I = w_pair.shape[0] // 2, w_pair.shape[1]
    native.grouped_gemm_tn_accum(dy, act, F_ops._main_grad(w_down), counts)
    dgu = native.grouped_gemm_swiglu_bwd(dy, w_down, gu, counts)
    mg = F_ops._main_grad(w_pair)
    native.grouped_gemm_tn_accum(dgu[:, :I], x, mg[:E], counts)
    native.grouped_gemm_tn_accum(dgu[:, I:], x, mg[E:], counts)
    return native.grouped_gemm_pair_dgrad(dgu, w_pair, counts)


def route(logits: torch.Tensor, k: int):
    """(weights [M,k] fp32, experts [M,k] int64); differentiable w.r.t. logits."""
    vals, experts = torch.topk(logits.float(), k, dim=-1)
    return torch.softmax(vals, dim=-1), experts


def aux_loss(logits: torch.Tensor, experts: torch.Tensor, num_experts: int) -> torch.Tensor:
    probs = torch.softmax(logits.float(), dim=-1).mean(0)
    frac = _count(experts.reshape(-1), num_experts).float() / experts.numel()
    return num_experts * (frac.detach() * probs).sum()


# --------------------------------------------------------------------------- CUDA path: routing and row movement as kernels
class _RouteDevice(torch.autograd.Function):
    """Top-k routing on the device (`csrc/moe.cu`): no sort, no host sync."""

    @staticmethod
    def forward(ctx, logits, k):
        weights, experts, counts, base, pos, order = native.moe_route(logits, k)
        ctx.save_for_backward(weights, experts)
        ctx.shape = logits.shape
        for t in (experts, counts, base, pos, order):
            ctx.mark_non_differentiable(t)
        return weights, experts, counts, base, pos, order

    @staticmethod
    def backward(ctx, dw, *unused):
        weights, experts = ctx.saved_tensors
        return native.moe_route_bwd(dw, weights, experts, ctx.shape[0], ctx.shape[1]), None


class _GatherDevice(torch.autograd.Function):
    """tokens `[M, D]` -> expert-major pair rows `[M*k, D]`; backward sums each token's k rows."""

    @staticmethod
    def forward(ctx, x, order, pos, k):
        ctx.save_for_backward(pos)
        ctx.k, ctx.M = k, x.shape[0]
        return native.moe_gather(x.contiguous(), order, k)

    @staticmethod
    def backward(ctx, d_rows):
        (pos,) = ctx.saved_tensors
        return native.moe_combine(d_rows.contiguous(), pos, None, ctx.M, ctx.k), None, None, None


class _CombineDevice(torch.autograd.Function):
    """`out[t] = sum_s w[t,s] * y[pos[t,s]]`; backward gives `d_y` (expert-major rows) and `d_w`."""

    @staticmethod
    def forward(ctx, y, weights, order, pos, k):
        ctx.save_for_backward(y, weights, order, pos)
        ctx.k = k
        return native.moe_combine(y.contiguous(), pos, weights, weights.shape[0], k)

    @staticmethod
    def backward(ctx, d_out):
        y, weights, order, pos = ctx.saved_tensors
        d_out = d_out.contiguous()
        d_y = native.moe_gather(d_out, order, ctx.k, scale=weights)
        dw = native.moe_pair_dot(d_out, y.contiguous(), pos, ctx.k).view_as(weights)
        return d_y, dw, None, None, None


def _moe_forward_device(x, logits, w_gate, w_up, w_down, k, num_experts, ep_group, ep_size, aux_coef, layer_key,
                        w_pair=None):
    """bf16 CUDA path without token dropping. Nothing here reads a device value on the host: the expert
    row ranges go to the grouped GEMMs as a device array, and with expert parallelism the rows travel
    through peer memory (`parallel.expert_parallel.peer`)."""
    weights, experts, counts, base, pos, order = _RouteDevice.apply(logits.contiguous(), k)
    aux = aux_loss(logits, experts.long(), num_experts) * aux_coef if aux_coef > 0.0 else None
    P = order.numel()
    if ep_size == 1:
        per_expert = native.DeviceCounts(base, P)
        local_x = _GatherDevice.apply(x, order, pos, k)
    else:
        from ..parallel.expert_parallel import peer as ep_peer
        pm = ep_peer.PeerMoE.get(ep_group, num_experts)
        plan = pm.plan(counts, experts, order, base)
        per_expert = native.DeviceCounts(plan["row_start"], plan["R"])
        local_x = ep_peer.dispatch_tokens(x, pm, plan, order, pos, k, layer_key)
    valid = None if ep_size == 1 else plan["n_recv"]        # rows of the expert-side buffers that hold real pairs
    if w_pair is not None and native.grouped_swiglu_ok(w_pair.shape[1]) and native.grouped_pair_ok(w_pair.shape[1]):
        # SwiGLU inside the grouped GEMMs' epilogues (forward and backward)
        if ep_size == 1:
            y = _ExpertMLP.apply(local_x, w_pair, w_down, per_expert)
            return _CombineDevice.apply(y, weights, order, pos, k), aux
        return ep_peer.expert_mlp_combine(local_x, w_pair, w_down, weights, pm, plan, per_expert, order, pos, k, layer_key), aux
    if w_pair is not None and native.grouped_pair_ok(w_pair.shape[1]):
        gu = _GroupedGateUp.apply(local_x, w_pair, per_expert)
    else:
        gu = torch.cat([grouped_linear(local_x, w_gate, per_expert), grouped_linear(local_x, w_up, per_expert)], dim=-1)
    act = F_ops.swiglu(gu, valid)
    if ep_size == 1:
        y = grouped_linear(act, w_down, per_expert)
        out = _CombineDevice.apply(y, weights, order, pos, k)
    else:
        out = ep_peer.down_combine(act, w_down, weights, pm, plan, per_expert, order, pos, k, layer_key)
    return out, aux


def moe_forward(x, logits, w_gate, w_up, w_down, k: int, num_experts: int, ep_group, ep_size: int,
                aux_coef: float = 0.0, capacity_factor: float = 0.0, layer_key=None, w_pair=None):
    """x `[M, D]`, logits `[M, E]` -> (out `[M, D]`, aux loss or None).

    On CUDA (bf16) the routing never touches the host: expert row ranges stay in
    a device `row_start` array read by the grouped GEMM's tile scheduler, and with
    expert parallelism the rows travel through `parallel.expert_parallel.peer`."""
    M, D = x.shape
    E_local = num_experts // ep_size
    if (x.is_cuda and x.dtype == torch.bfloat16 and capacity_factor <= 0.0 and num_experts <= 256 and k <= 8
            and D % 8 == 0 and (ep_size == 1 or (_peer_enabled() and ep_size <= 8))):
        return _moe_forward_device(x, logits, w_gate, w_up, w_down, k, num_experts, ep_group, ep_size, aux_coef,
                                   layer_key, w_pair)
    weights, experts = route(logits, k)                                    # [M,k]
    aux = aux_loss(logits, experts, num_experts) * aux_coef if aux_coef > 0.0 else None

    flat_e = experts.reshape(-1)                                           # [M*k], pair p = token p//k, slot p%k
    order = torch.sort(flat_e, stable=True).indices                        # pairs sorted by expert id
    keep = None
    if capacity_factor > 0.0:
        # position of each pair inside its expert's queue; drop what exceeds the capacity
        cap = max(1, int(capacity_factor * M * k / num_experts))
        sorted_e = flat_e[order]
        start = torch.searchsorted(sorted_e, torch.arange(num_experts, device=x.device))
        pos = torch.arange(M * k, device=x.device) - start[sorted_e]
        keep = pos < cap
        order = order[keep]
    token_of = torch.div(order, k, rounding_mode="floor")
    sorted_x = x.index_select(0, token_of)                                 # gather (bwd: index_add)
    counts = _count(flat_e[order], num_experts).view(ep_size, E_local)

    if ep_size > 1:
        recv_counts = exchange_counts(counts, ep_group)                    # [src, E_local]
        both = torch.stack([counts, recv_counts]).tolist()                 # one host sync for both
        send_c, recv_c = both
        send_splits = [sum(r) for r in send_c]
        recv_splits = [sum(r) for r in recv_c]
        recv_x = ep_all_to_all(sorted_x, send_splits, recv_splits, ep_group)
        # rows arrive ordered (src, expert); regroup to (expert, src)
        regroup = _regroup_index(recv_c, x.device)
        local_x = recv_x.index_select(0, regroup)
        per_expert = [sum(recv_c[s][e] for s in range(ep_size)) for e in range(E_local)]
    else:
        local_x = sorted_x
        per_expert = counts.view(-1).tolist()

    gate = grouped_linear(local_x, w_gate, per_expert)
    up = grouped_linear(local_x, w_up, per_expert)
    act = F_ops.swiglu(torch.cat([gate, up], dim=-1))
    y = grouped_linear(act, w_down, per_expert)

    if ep_size > 1:
        inv = torch.empty_like(regroup)
        inv[regroup] = torch.arange(regroup.numel(), device=x.device)
        y = ep_all_to_all(y.index_select(0, inv), recv_splits, send_splits, ep_group)

    w_sorted = weights.reshape(-1)[order]                                  # weight of each sorted pair
    contrib = y.float() * w_sorted[:, None]
    out = torch.zeros(M, D, dtype=torch.float32, device=x.device).index_add(0, token_of, contrib)
    return out.to(x.dtype), aux


def _count(idx: torch.Tensor, n: int) -> torch.Tensor:
    """Histogram without the host sync that `torch.bincount` does on CUDA."""
    return torch.zeros(n, dtype=torch.int64, device=idx.device).scatter_add_(0, idx, torch.ones_like(idx))


def _peer_enabled() -> bool:
    from ..parallel import symm
    return symm.use_symm()


def _regroup_index(recv_counts: list[list[int]], device) -> torch.Tensor:
    """Index that reorders rows received as (src-major, expert-minor) blocks
    into (expert-major, src-minor) order. Pure function of the counts."""
    ep, E_local = len(recv_counts), len(recv_counts[0])
    starts, r = [[0] * E_local for _ in range(ep)], 0
    for s in range(ep):
        for e in range(E_local):
            starts[s][e] = r
            r += recv_counts[s][e]
    idx = []
    for e in range(E_local):
        for s in range(ep):
            idx.extend(range(starts[s][e], starts[s][e] + recv_counts[s][e]))
    return torch.tensor(idx, dtype=torch.long, device=device)
