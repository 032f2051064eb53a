"""Seeded weight initialisation.

The reference draws every weight matrix right after `manual_seed(seed)` inside
`fork_rng` (`model/modules/attn.py:112-124`, `model/modules/mlp.py:32-41,77-93`,
`model/gpt.py:55-62`): the values depend only on (seed, shape), never on the
rank or the parallel layout, so runs with different `sep_size` start from the
same weights; expert e uses `seed + global_expert_index`. The same rule is
applied here with a private generator (the global RNG is left untouched), and
draws are cached per (seed, shape, device) because same-shaped matrices of
every layer are identical under this rule.
"""
from __future__ import annotations

import torch

_CACHE: dict[tuple, torch.Tensor] = {}


def seeded_normal(shape, std: float, seed: int, device, cache: bool = True) -> torch.Tensor:
    device = torch.device(device)
    key = (tuple(shape), float(std), int(seed), str(device))
    if cache and key in _CACHE:
        return _CACHE[key].clone()
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    t = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    t.normal_(mean=0.0, std=std, generator=gen)
    if cache:
        _CACHE[key] = t
        return t.clone()
    return t


def clear_init_cache() -> None:
    _CACHE.clear()
