"""Process-group grid: DP x SEP, where the SEP group carries both Ulysses
sequence parallelism and expert parallelism.

Layout matches the reference (`distributed/parallel_state.py:33-48`): SEP
groups are runs of consecutive ranks `[i*sep, (i+1)*sep)`, DP groups are the
strided sets `{i*sep + j}`, and DP_SP is the whole world. `sp_*` and `ep_*`
getters alias `sep_*`.

Unlike the reference, every getter also works before/without
`initialize_model_parallel` (single-process use: sizes 1, ranks 0, groups
None), so models can be built and run on one device with no process group.
"""
from __future__ import annotations

import torch.distributed as dist

_STATE = {"sep": None, "dp": None, "dp_sp": None, "sep_size": 1, "dp_size": 1,
          "sep_ranks": [0], "dp_ranks": [0], "initialized": False}


def group_layout(world_size: int, sep_size: int) -> tuple[list[list[int]], list[list[int]]]:
    """Pure function: (sep_groups, dp_groups) as lists of global ranks."""
    if world_size % sep_size != 0:
        raise AssertionError("World size must be divisible by sep_size")
    dp_size = world_size // sep_size
    sep_groups = [list(range(i * sep_size, (i + 1) * sep_size)) for i in range(dp_size)]
    dp_groups = [[i * sep_size + j for i in range(dp_size)] for j in range(sep_size)]
    return sep_groups, dp_groups


def initialize_model_parallel(config=None, sep_size: int | None = None) -> None:
    """Create the groups. Call after `dist.init_process_group`. Accepts a
    ParallelConfig (reference signature) or a bare `sep_size`."""
    if sep_size is None:
        sep_size = config.sep_size
    assert dist.is_initialized(), "Must initialize the torch.distributed process group first"
    world, rank = dist.get_world_size(), dist.get_rank()
    sep_groups, dp_groups = group_layout(world, sep_size)
    for ranks in sep_groups:
        g = dist.new_group(ranks)
        if rank in ranks:
            _STATE["sep"], _STATE["sep_ranks"] = g, ranks
    for ranks in dp_groups:
        g = dist.new_group(ranks)
        if rank in ranks:
            _STATE["dp"], _STATE["dp_ranks"] = g, ranks
    _STATE["dp_sp"] = dist.new_group(list(range(world)))
    _STATE["sep_size"], _STATE["dp_size"] = sep_size, world // sep_size
    _STATE["initialized"] = True


def destroy_model_parallel() -> None:
    _STATE.update({"sep": None, "dp": None, "dp_sp": None, "sep_size": 1, "dp_size": 1,
                   "sep_ranks": [0], "dp_ranks": [0], "initialized": False})


def is_initialized() -> bool:
    return _STATE["initialized"]


def _rank_in(group) -> int:
    return dist.get_rank(group=group) if _STATE["initialized"] else 0


def _global(group, rank) -> int:
    return dist.get_global_rank(group, rank) if _STATE["initialized"] else 0


# ---- DP -------------------------------------------------------------------
def get_dp_group():
    return _STATE["dp"]


def get_dp_world_size() -> int:
    return _STATE["dp_size"]


def get_dp_rank() -> int:
    return _rank_in(_STATE["dp"])


def get_dp_global_rank(rank: int | None = None) -> int:
    return _global(_STATE["dp"], get_dp_rank() if rank is None else rank)


def get_dp_ranks() -> list[int]:
    return list(_STATE["dp_ranks"])


# ---- SEP (= SP = EP) --------------------------------------------------------
def get_sep_group():
    return _STATE["sep"]


def get_sep_world_size() -> int:
    return _STATE["sep_size"]


def get_sep_rank() -> int:
    return _rank_in(_STATE["sep"])


def get_sep_global_rank(rank: int | None = None) -> int:
    return _global(_STATE["sep"], get_sep_rank() if rank is None else rank)


def get_sep_ranks() -> list[int]:
    return list(_STATE["sep_ranks"])


get_sp_group, get_sp_world_size, get_sp_rank, get_sp_global_rank = (
    get_sep_group, get_sep_world_size, get_sep_rank, get_sep_global_rank)
get_ep_group, get_ep_world_size, get_ep_rank, get_ep_global_rank = (
    get_sep_group, get_sep_world_size, get_sep_rank, get_sep_global_rank)


# ---- DP x SP (the whole world) --------------------------------------------------
def get_dp_sp_group():
    return _STATE["dp_sp"]


def get_dp_sp_world_size() -> int:
    return _STATE["dp_size"] * _STATE["sep_size"]


def get_dp_sp_rank() -> int:
    return _rank_in(_STATE["dp_sp"])


def get_dp_sp_global_rank(rank: int | None = None) -> int:
    return _global(_STATE["dp_sp"], get_dp_sp_rank() if rank is None else rank)
