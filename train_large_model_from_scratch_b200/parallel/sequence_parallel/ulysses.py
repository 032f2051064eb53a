"""Ulysses sequence parallelism: the seq<->head all-to-all and the head plan.

Reference: `distributed/sequence_parallel/ulysses.py:5-41` (equal-split
all-to-all autograd function, SP gradient all-reduce) and the re-layout code
around it in `model/modules/attn.py:143-171`. The reference's re-layout uses
raw `.view`s that are a correct permutation only for micro-batch 1 with one
head per rank; the functions here implement the intended mapping for every
shape:

  * rank r of the SP group attends with query heads [r*Hq/sp, (r+1)*Hq/sp) and
    the KV heads those query heads read, over the FULL sequence assembled from
    all ranks' chunks in rank order;
  * its output rows for chunk s go back to rank s.

KV heads travel un-expanded (the reference expands K and V to Hq heads before
the exchange); a KV head needed by several ranks is sent to each of them and
its gradient contributions are summed on the way back by autograd.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllToAllEqual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()          # empty_like of a permuted grad would keep its strides
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None


def ulysses_all_to_all(x: torch.Tensor, group) -> torch.Tensor:
    """Equal-split all-to-all along dim 0 (`x.shape[0]` = group size chunks);
    its own transpose in backward."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _AllToAllEqual.apply(x, group)


def head_plan(n_q: int, n_kv: int, sp: int) -> tuple[list[list[int]], int, int]:
    """For each destination rank, the indices into the packed head axis
    `[q_0..q_{Hq-1}, k_0..k_{Hkv-1}, v_0..v_{Hkv-1}]` that it needs.
    Returns (per-rank index lists, local q heads, local kv heads)."""
    if n_q % sp:
        raise ValueError(f"num_attention_heads ({n_q}) must be divisible by the SP size ({sp})")
    rep = n_q // n_kv
    q_l = n_q // sp
    plans, kv_l = [], None
    for r in range(sp):
        q_heads = list(range(r * q_l, (r + 1) * q_l))
        kv_heads = sorted({h // rep for h in q_heads})
        if kv_l is None:
            kv_l = len(kv_heads)
        if len(kv_heads) != kv_l or q_l % kv_l:
            raise ValueError(f"unsupported GQA/SP combination: Hq={n_q}, Hkv={n_kv}, sp={sp}")
        for i, h in enumerate(q_heads):                     # local q head i must map to local kv head i // (q_l/kv_l)
            assert kv_heads[i // (q_l // kv_l)] == h // rep
        plans.append(q_heads + [n_q + j for j in kv_heads] + [n_q + n_kv + j for j in kv_heads])
    return plans, q_l, kv_l


def seq_to_head(qkv: torch.Tensor, n_q: int, n_kv: int, group) -> tuple[torch.Tensor, int, int]:
    """`[B, T_local, Hq+2Hkv, hd]` (all heads, my chunk) ->
    `[B, T_full, q_l+2kv_l, hd]` (my heads, whole sequence)."""
    sp = dist.get_world_size(group)
    plans, q_l, kv_l = head_plan(n_q, n_kv, sp)
    B, T_l, _, hd = qkv.shape
    idx = torch.tensor([h for plan in plans for h in plan], device=qkv.device)
    send = qkv.index_select(2, idx)                                       # B, T_l, sp*hpr, hd
    hpr = q_l + 2 * kv_l
    send = send.view(B, T_l, sp, hpr, hd).permute(2, 0, 1, 3, 4).contiguous()   # dest, B, T_l, hpr, hd
    recv = ulysses_all_to_all(send, group)                                 # src, B, T_l, hpr, hd
    full = recv.permute(1, 0, 2, 3, 4).reshape(B, sp * T_l, hpr, hd)
    return full, q_l, kv_l


def head_to_seq(o: torch.Tensor, group) -> torch.Tensor:
    """`[B, T_full, q_l, hd]` (my heads, whole sequence) -> `[B, T_local, Hq, hd]`."""
    sp = dist.get_world_size(group)
    B, T_full, q_l, hd = o.shape
    T_l = T_full // sp
    send = o.view(B, sp, T_l, q_l, hd).permute(1, 0, 2, 3, 4).contiguous()      # dest(seq owner), B, T_l, q_l, hd
    recv = ulysses_all_to_all(send, group)                                 # src(head owner), B, T_l, q_l, hd
    return recv.permute(1, 2, 0, 3, 4).reshape(B, T_l, sp * q_l, hd)


def allreduce_non_expert_grads_across_sp(model, sp_group, sp_world_size: int,
                                         expert_local_param_suffixes=()) -> None:
    """Sum the gradients of replicated (non-expert) parameters over the SP
    group. Kept for API compatibility with the reference (`ulysses.py:27-41`),
    which calls it once per step and issues one all-reduce per tensor. With
    flat storage the trainer does not need it: the dense gradient buffer is
    reduced over the whole DP x SP world in one go. When called, it reduces the
    flat dense buffer if there is one, else falls back to per-tensor calls."""
    if sp_world_size <= 1:
        return
    done = set()
    for name, p in model.named_parameters():
        if name.endswith(tuple(expert_local_param_suffixes)):
            continue
        buf = getattr(p, "flat_buffer", None)
        if buf is not None:
            if id(buf) not in done:
                dist.all_reduce(buf.main_grad, op=dist.ReduceOp.SUM, group=sp_group)
                done.add(id(buf))
        else:
            g = getattr(p, "main_grad", None)
            if g is None:
                g = p.grad
            if g is not None:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=sp_group)
