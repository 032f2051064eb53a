"""Expert-parallel token exchange: variable-split all-to-all on `[rows, D]`
whose backward runs the same exchange with the split lists swapped
(reference: `distributed/expert_parallel/comm.py:5-44`)."""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllToAllVariable(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_splits, recv_splits, group):
        ctx.group, ctx.send, ctx.recv = group, list(send_splits), list(recv_splits)
        out = x.new_empty((sum(recv_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=ctx.recv,
                               input_split_sizes=ctx.send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send,
                               input_split_sizes=ctx.recv, group=ctx.group)
        return out, None, None, None


def ep_all_to_all(x: torch.Tensor, send_splits, recv_splits, group) -> torch.Tensor:
    """Rows `[sum(send_splits), ...]` -> `[sum(recv_splits), ...]`; chunk i of the
    input goes to rank i of `group`."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _AllToAllVariable.apply(x, send_splits, recv_splits, group)


def exchange_counts(counts: torch.Tensor, group) -> torch.Tensor:
    """`counts[dest_rank, local_expert]` -> what each source rank sends me,
    `[src_rank, local_expert]`."""
    if group is None or dist.get_world_size(group) == 1:
        return counts
    out = torch.empty_like(counts)
    dist.all_to_all_single(out, counts.contiguous(), group=group)
    return out
