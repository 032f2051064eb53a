"""Checkpoint save / resume in the reference's on-disk layout
(`training/trainer.py:266-306,377-408`), with prefix `P = {log_dir}/{step:05d}`:

  P_opt/                DCP directory; key `optimizer/rank{RANK}` = this rank's
                        AdamW state dict (torch layout) for the tensors it owns
                        under the whole-tensor ZeRO-1 assignment
  P_rng_rank{RANK}.pt   {'torch', 'cuda', 'numpy'} RNG states
  P_model.pt            fp32 model state dict (rank 0)
  P_meta.pt             configs, step, results, `opt_part_assignment`,
                        sampler state, RNG state (rank 0) -- written LAST

Behaviour the reference intends but does not deliver, implemented here:
Adam moments ARE restored on resume; with expert parallelism `P_model.pt`
holds all experts (gathered over the EP group) so it can be loaded under any
`sep_size`; every file is written to a temporary name and renamed, `P_meta.pt`
is the commit marker and resume picks the newest step whose file set is
complete; steps are ordered numerically, not lexicographically; `log.txt` is
kept on resume; checkpoints whose keys carry the `_orig_mod.` prefix written
by a compiled reference model load transparently.
"""
from __future__ import annotations

import glob
import os
import re
from collections import OrderedDict

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import parallel_state
from ..parallel.flat import is_expert_param
from ..utils.model import strip_compile_prefix


def _atomic_save(obj, path: str) -> None:
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        torch.save(obj, f)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _locate(model, name: str):
    """(optimizer shard index, offset, numel, shape) of parameter `name`."""
    for i, buf in enumerate(b for b in (model.dense_buf, model.expert_buf) if b is not None):
        if name in buf.layout:
            return (i,) + buf.layout[name]
    raise KeyError(name)


def unique_param_names(model) -> list[str]:
    return [n for n, _ in model.named_parameters()]


# --------------------------------------------------------------------------- model
def full_model_state_dict(model, optimizer) -> "OrderedDict[str, torch.Tensor]":
    """fp32 state dict assembled from the master shards; experts concatenated
    over the EP group to `[E, ...]`. Collective: every rank must call it."""
    opt = getattr(optimizer, "optimizer", optimizer)
    fulls = [opt.gather_full(s, "master") for s in opt.shards]
    ep, ep_group = parallel_state.get_ep_world_size(), parallel_state.get_ep_group()
    out = OrderedDict()
    names = {n: p for n, p in model.named_parameters()}
    for key in model.state_dict().keys():
        src = key if key in names else ("wte.weight" if key == "lm_head.weight" else key)
        i, off, n, shape = _locate(model, src)
        t = fulls[i][off:off + n].view(shape).clone()
        if is_expert_param(key) and ep > 1:
            parts = [torch.empty_like(t) for _ in range(ep)]
            dist.all_gather(parts, t, group=ep_group)
            t = torch.cat(parts, dim=0)
        out[key] = t.cpu()
    return out


def load_model_state_dict(model, optimizer, state: dict) -> None:
    """Inverse of `full_model_state_dict`: fills master shards and the
    compute-dtype parameters; slices this rank's experts out of `[E, ...]`."""
    state = strip_compile_prefix(state)
    opt = getattr(optimizer, "optimizer", optimizer)
    ep, ep_rank = parallel_state.get_ep_world_size(), parallel_state.get_ep_rank()
    for name, p in model.named_parameters():
        t = state[name].to(torch.float32)
        if is_expert_param(name) and t.shape[0] != p.shape[0]:
            el = p.shape[0]
            assert t.shape[0] == el * ep, f"{name}: checkpoint has {t.shape[0]} experts, need {el * ep}"
            t = t[ep_rank * el:(ep_rank + 1) * el]
        i, off, n, shape = _locate(model, name)
        s = opt.shards[i]
        s.copy_range_from(s.master, off, n, t.reshape(-1))
    opt.sync_params_from_master()


# --------------------------------------------------------------------------- optimizer
def optimizer_state_dict(model, optimizer) -> dict:
    """torch.optim.AdamW-style dict for the tensors this rank owns."""
    opt = getattr(optimizer, "optimizer", optimizer)
    m_full = [opt.gather_full(s, "exp_avg") for s in opt.shards]
    v_full = [opt.gather_full(s, "exp_avg_sq") for s in opt.shards]
    owned = optimizer.owned_names() if hasattr(optimizer, "owned_names") else unique_param_names(model)
    state = {}
    for j, name in enumerate(owned):
        i, off, n, shape = _locate(model, name)
        state[j] = {
            "step": torch.tensor(float(opt.step_count)),
            "exp_avg": m_full[i][off:off + n].view(shape).clone().cpu(),
            "exp_avg_sq": v_full[i][off:off + n].view(shape).clone().cpu(),
        }
    group = {k: v for k, v in opt.param_groups[0].items() if k != "params"}
    group["betas"] = list(group["betas"])
    group["params"] = list(range(len(owned)))
    return {"state": state, "param_groups": [group]}


def load_optimizer_state_dict(model, optimizer, sd: dict) -> None:
    opt = getattr(optimizer, "optimizer", optimizer)
    owned = optimizer.owned_names() if hasattr(optimizer, "owned_names") else unique_param_names(model)
    dev = opt.shards[0].master.device
    m_full = [torch.zeros(s.buf.padded, dtype=torch.float32, device=dev) for s in opt.shards]
    v_full = [torch.zeros(s.buf.padded, dtype=torch.float32, device=dev) for s in opt.shards]
    step = 0
    for j, name in enumerate(owned):
        st = sd["state"].get(j, sd["state"].get(str(j)))
        if st is None:
            continue
        i, off, n, _ = _locate(model, name)
        m_full[i][off:off + n].copy_(st["exp_avg"].reshape(-1))
        v_full[i][off:off + n].copy_(st["exp_avg_sq"].reshape(-1))
        step = max(step, int(float(st["step"])))
    group = getattr(optimizer, "process_group", None)
    zero1 = hasattr(optimizer, "owned_names") and group is not None and dist.get_world_size(group) > 1
    for i, s in enumerate(opt.shards):
        if zero1:                       # every tensor is owned by exactly one rank of the DP group
            dist.all_reduce(m_full[i], group=group)
            dist.all_reduce(v_full[i], group=group)
        opt.scatter_full(s, "exp_avg", m_full[i])
        opt.scatter_full(s, "exp_avg_sq", v_full[i])
    if zero1:
        t = torch.tensor([step], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        step = int(t.item())
    opt.step_count = step
    pg = sd["param_groups"][0]
    for k in ("lr", "eps", "weight_decay"):
        if k in pg:
            opt.param_groups[0][k] = pg[k]
    if "betas" in pg:
        opt.param_groups[0]["betas"] = tuple(pg["betas"])


# --------------------------------------------------------------------------- RNG
def rng_state(local_rank: int) -> dict:
    st = {"torch": torch.get_rng_state(), "numpy": np.random.get_state()}
    st["cuda"] = torch.cuda.get_rng_state(local_rank) if torch.cuda.is_available() else torch.empty(0, dtype=torch.uint8)
    return st


def set_rng_state(st: dict, local_rank: int) -> None:
    torch.set_rng_state(st["torch"].to(torch.uint8).cpu())
    if torch.cuda.is_available() and st["cuda"].numel():
        torch.cuda.set_rng_state(st["cuda"].to(torch.uint8).cpu(), local_rank)
    np.random.set_state(st["numpy"])


# --------------------------------------------------------------------------- discovery
_STEP_RE = re.compile(r"(\d+)_meta\.pt$")


def find_latest_complete(ckpt_dir: str, rank: int) -> str | None:
    """Prefix of the newest checkpoint whose meta (commit marker), model file,
    optimizer directory and this rank's RNG file all exist."""
    best, best_step = None, -1
    for meta in glob.glob(os.path.join(ckpt_dir, "*_meta.pt")):
        m = _STEP_RE.search(meta)
        if not m:
            continue
        prefix = meta[:-len("_meta.pt")]
        complete = (os.path.exists(prefix + "_model.pt")
                    and os.path.exists(os.path.join(prefix + "_opt", ".metadata"))
                    and os.path.exists(f"{prefix}_rng_rank{rank}.pt"))
        if complete and int(m.group(1)) > best_step:
            best, best_step = prefix, int(m.group(1))
    return best


# --------------------------------------------------------------------------- DCP wrappers
def dcp_save(state_dict: dict, path: str) -> None:
    from torch.distributed.checkpoint import state_dict_saver
    from torch.distributed.checkpoint.filesystem import FileSystemWriter
    state_dict_saver.save(state_dict=state_dict, storage_writer=FileSystemWriter(path))


def dcp_load(state_dict: dict, path: str) -> None:
    from torch.distributed.checkpoint import state_dict_loader
    from torch.distributed.checkpoint.filesystem import FileSystemReader
    state_dict_loader.load(state_dict=state_dict, storage_reader=FileSystemReader(path))
