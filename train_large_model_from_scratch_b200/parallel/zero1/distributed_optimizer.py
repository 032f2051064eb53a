"""AdamW on flat buffers with ZeRO-1 sharding of optimizer state.

Reference: `distributed/zero1/distributed_optimizer.py:1-185` wraps a
`torch.optim.AdamW`, assigns WHOLE tensors to ranks with a greedy
longest-processing-time heuristic, steps the owned tensors and then broadcasts
every tensor from its owner; gradients reach it through DDP's all-reduce plus a
per-tensor SP all-reduce and a separate `clip_grad_norm_` pass.

Here the step is one pipeline over each flat buffer (see `parallel.flat`):

    reduce-scatter(main_grad) -> |g|^2 partial -> one scalar all-reduce ->
    fused clip + AdamW on this rank's even 1/n slice (fp32 master, exp_avg,
    exp_avg_sq) -> all-gather of the updated compute-dtype parameters

so every rank holds exactly 1/n of the optimizer state regardless of tensor
sizes (the reference's owner of the embedding holds 1.4-2.5x the ideal share),
and gradients cross the wire once as a reduce-scatter instead of twice as an
all-reduce. On CUDA the stages run as kernels of this package over NVLink peer
memory (`parallel.symm`); on CPU/Gloo they are `torch.distributed` calls.

The reference's public names are kept: `DistributedOptimizer(optimizer,
process_group, ranks_map, num_parts, verbose)`, `.part_assignment`,
`partition_tensors`, attribute forwarding to the wrapped optimizer, and a
`state_dict()` in `torch.optim.AdamW` layout restricted to the tensors this
rank owns under the whole-tensor assignment (that is the on-disk format).
"""
from __future__ import annotations

import heapq
import math
from collections import OrderedDict

import torch
import torch.distributed as dist

from ...ops import native, oracle
from ..flat import FlatBuffer


def partition_tensors(tensor_dict: "OrderedDict[tuple[int, int], torch.Tensor]", ranks_map: list | None = None,
                      num_parts: int | None = None, verbose: bool = False, deterministic: bool = True):
    """Greedy balanced assignment of tensors to parts: biggest tensor first,
    always to the currently lightest part; ties resolved by key (and by part
    id) so that every rank computes the same answer.
    Returns `(assignment: key -> owner, tensor_dict)`."""
    if ranks_map is not None:
        num_parts = len(ranks_map)
    assert num_parts and num_parts > 0, "num_parts must be a positive integer"
    items = [(k, t.numel()) for k, t in tensor_dict.items()]
    items.sort(key=(lambda kv: (-kv[1], kv[0])) if deterministic else (lambda kv: -kv[1]))
    heap = [(0, part) for part in range(num_parts)]
    heapq.heapify(heap)
    loads = [0] * num_parts
    assignment = {k: None for k in tensor_dict}
    for key, n in items:
        load, part = heapq.heappop(heap)
        assignment[key] = ranks_map[part] if ranks_map is not None else part
        loads[part] = load + n
        heapq.heappush(heap, (load + n, part))
    if verbose:
        for part, load in enumerate(loads):
            if load == 0:
                print(f"[ZeRO-1] Warning: partition {part} is empty.")
        mean = sum(loads) / num_parts + 1e-6
        print(f"[ZeRO-1] Partition load imbalance: {(max(loads) - min(loads)) / mean:.2%}")
    return assignment, tensor_dict


class _Bucket:
    """One contiguous range `[lo, hi)` of a flat buffer and this rank's 1/parts piece of it."""

    __slots__ = ("lo", "hi", "off", "seg", "seg_lo", "group")

    def __init__(self, lo: int, hi: int, off: int, seg: int, seg_lo: int, group: int):
        self.lo, self.hi = lo, hi            # range of the bucket in the flat buffer (elements)
        self.off, self.seg = off, seg        # this rank's piece: `seg` elements at `off` of its local state arrays
        self.seg_lo = seg_lo                 # ... which are elements [seg_lo, seg_lo + seg) of the flat buffer
        self.group = group                   # layer group whose backward completes the bucket's gradients (0: the last)


class _Shard:
    """Optimizer state of one flat buffer on this rank.

    The buffer is cut into buckets (`cuts`: ascending element offsets) and every rank owns the r-th 1/n piece of
    EVERY bucket, not one contiguous 1/n slice of the whole buffer: a bucket's gradients are final as soon as the
    backward pass has left its layers, so its reduce-scatter can run under the rest of the backward pass, and
    after the update its parameters can be handed to the next forward pass bucket by bucket. The local state
    arrays (`master`, `exp_avg`, `exp_avg_sq`, `grad_shard`) are the concatenation of the rank's pieces."""

    def __init__(self, buf: FlatBuffer, group, sharded: bool, cuts: list[int] | None = None,
                 bucket_groups: list[int] | None = None):
        self.buf, self.group = buf, group
        self.n = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.sharded = sharded and self.n > 1
        parts = self.n if self.sharded else 1
        assert buf.padded % parts == 0, "flat buffer must be padded to a multiple of the shard count"
        if parts == 1:
            cuts, bucket_groups = None, None                 # nothing to overlap: one bucket, one kernel
        pts = sorted(set([0, buf.padded] + [int(c) for c in (cuts or []) if 0 < c < buf.padded]))
        if bucket_groups is None or len(bucket_groups) != len(pts) - 1:
            bucket_groups = [0] * (len(pts) - 1)
        unit = parts * 8
        self.buckets: list[_Bucket] = []
        off = 0
        for (lo, hi), g in zip(zip(pts[:-1], pts[1:]), bucket_groups):
            assert parts == 1 or (lo % unit == 0 and hi % unit == 0), \
                f"bucket boundaries must be multiples of 8 * shard count ({unit}): {lo}, {hi}"
            seg = (hi - lo) // parts
            self.buckets.append(_Bucket(lo, hi, off, seg, lo + (self.rank if self.sharded else 0) * seg, g))
            off += seg
        self.len = off
        self.master = self.take_local(buf.init_fp32)
        buf.init_fp32 = None                                    # full fp32 copy no longer needed
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_shard = None if not self.sharded else torch.zeros_like(self.master)
        self.reduced: set = set()                               # buckets already reduced in the current step
        # slice of the buffer whose |g|^2 this rank contributes to the global norm when nothing is sharded
        vlen = buf.padded // self.n
        self.norm_lo, self.norm_hi = self.rank * vlen, (self.rank + 1) * vlen

    # -- local <-> flat ------------------------------------------------------------------
    def take_local(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's pieces of a full-length tensor, concatenated (a new tensor)."""
        if len(self.buckets) == 1:
            b = self.buckets[0]
            return full[b.seg_lo:b.seg_lo + b.seg].clone()
        return torch.cat([full[b.seg_lo:b.seg_lo + b.seg] for b in self.buckets])

    def put_local(self, full: torch.Tensor, local: torch.Tensor) -> None:
        """Inverse of `take_local`: writes the pieces into their places of `full` (dtype of `full`)."""
        for b in self.buckets:
            full[b.seg_lo:b.seg_lo + b.seg].copy_(local[b.off:b.off + b.seg])

    def copy_range_from(self, local: torch.Tensor, off: int, n: int, src: torch.Tensor) -> None:
        """`local` (one of the state arrays) takes the part of flat elements `[off, off + n)` that this rank
        owns from `src` (`n` values: the whole range)."""
        for b in self.buckets:
            lo, hi = max(off, b.seg_lo), min(off + n, b.seg_lo + b.seg)
            if lo < hi:
                local[b.off + lo - b.seg_lo:b.off + hi - b.seg_lo].copy_(src[lo - off:hi - off])

    def assemble_full(self, stack: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """`stack [n, len]` (row r = rank r's local array) -> the full buffer."""
        full = out if out is not None else torch.empty(self.buf.padded, dtype=stack.dtype, device=stack.device)
        for b in self.buckets:
            full[b.lo:b.hi].view(stack.shape[0], b.seg).copy_(stack[:, b.off:b.off + b.seg])
        return full


class FusedAdamW:
    """AdamW (decoupled weight decay on every tensor, like the reference's
    single param group, `training/trainer.py:137-143`) over flat buffers."""

    def __init__(self, buffers: list[FlatBuffer], lr: float = 1e-3, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, groups: list | None = None, grad_divisor: float = 1.0,
                 sharded: bool = False, norm_group=None, cuts: list | None = None, bucket_groups: list | None = None):
        """`cuts[i]` / `bucket_groups[i]` (optional, per buffer): bucket boundaries in elements and, per bucket,
        the layer group whose backward pass completes its gradients (see `_Shard`, `group_backward_done`)."""
        self.buffers = [b for b in buffers if b is not None]
        groups = groups if groups is not None else [None] * len(self.buffers)
        cuts = cuts if cuts is not None else [None] * len(self.buffers)
        bucket_groups = bucket_groups if bucket_groups is not None else [None] * len(self.buffers)
        self.param_groups = [dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                                  amsgrad=False, maximize=False, params=[])]
        self.grad_divisor = float(grad_divisor)
        self.norm_group = norm_group
        self.shards = [_Shard(b, g, sharded, c, bg) for b, g, c, bg in zip(self.buffers, groups, cuts, bucket_groups)]
        self.step_count = 0
        self.grad_norm = None
        self._comm = None              # optional peer-memory collective engine (CUDA)
        self.last_micro_step = True    # set by the trainer: bucket reductions only start in the step's last backward
        # per-step scalars of the AdamW kernels (lr, bias corrections) in device memory, fed from pinned memory
        dev = self.buffers[0].params.device if self.buffers else torch.device("cpu")
        if dev.type == "cuda":
            self._hyper = torch.zeros(4, dtype=torch.float32, device=dev)
            # a ring of pinned staging slots: the host may run several steps ahead of the device (graph replay
            # does not wait), and a slot is only rewritten once the copy that read it has run
            self._hyper_host = [torch.zeros(4, dtype=torch.float32).pin_memory() for _ in range(4)]
            self._hyper_done = [None] * len(self._hyper_host)
        else:
            self._hyper = self._hyper_host = None

    # -- the reference-style surface ------------------------------------------------
    def zero_grad(self, set_to_none: bool = True) -> None:
        # the peers read this rank's gradient buffer in their reduce-scatter: their "parameters ready" flags
        # (which they send after it) must be here before the buffer is cleared for the next step
        self.wait_params_ready()
        for b in self.buffers:
            b.zero_grad()
        for s in self.shards:
            s.reduced.clear()

    # -- hooks of the model's forward / backward pass (peer-memory path only) ---------
    def wait_params_ready(self) -> None:
        """Queue the wait for the buckets no GEMM waits for itself (group 0: embedding, first norm)."""
        if self._comm is not None:
            self._comm.wait_first_buckets(self.shards)

    def before_forward(self) -> None:
        self.wait_params_ready()

    def before_group(self, g: int) -> None:
        """Forward pass is about to enter layer group `g`: its first GEMM waits for the group's parameters."""
        if self._comm is not None:
            self._comm.arm_group(self.shards, g)

    def group_backward_done(self, g: int) -> None:
        """Backward pass has left layer group `g`: on the step's last micro-step the gradients of the group's
        buckets are final, so their reduce-scatter starts now, on the communication stream, under the rest
        of the backward pass (what DDP's bucketed all-reduce gives the reference, `training/trainer.py:133,247`)."""
        if self._comm is None or not self.last_micro_step or self._comm.overlap_blocks <= 0:
            return
        for s in self.shards:
            if not self._comm.handles(s):
                continue
            for bi, b in enumerate(s.buckets):
                if b.group == g and bi not in s.reduced:
                    self._comm.reduce_bucket(s, bi, overlapped=True)
                    s.reduced.add(bi)

    def prepare_step(self) -> None:
        """Host part of a step: advance the step counter and publish this step's scalars (learning rate, bias
        corrections) to the device buffer the kernels read. Kept apart from `step_device` so that the device
        part is launch-for-launch identical every step (it can be recorded once and replayed)."""
        g = self.param_groups[0]
        self.step_count += 1
        if self._hyper is not None:
            b1, b2 = g["betas"]
            vals = native.adam_hyper(self.step_count, g["lr"], b1, b2)
            slot = self.step_count % len(self._hyper_host)
            if self._hyper_done[slot] is not None:
                self._hyper_done[slot].synchronize()          # the copy that last read this slot has run
            host = self._hyper_host[slot]
            host[0], host[1], host[2] = vals
            self._hyper.copy_(host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._hyper_done[slot] = ev

    @torch.no_grad()
    def step_device(self, grad_clip_value: float | None = None):
        """Reduce gradients, clip by global norm, update, re-assemble parameters.
        Returns the global gradient norm (0-d tensor, before clipping)."""
        g = self.param_groups[0]
        inv = 1.0 / self.grad_divisor
        norm_sq = None
        if self._comm is not None:
            self._comm.join()                    # bucket reductions started during backward
        for s in self.shards:
            grad = self._reduce(s)
            if self._comm is not None and self._comm.handles(s):
                part = self._comm.last_sumsq(s)          # produced by the reduce-scatter kernels
            else:
                part = self._sumsq(grad if s.sharded else s.buf.main_grad[s.norm_lo:s.norm_hi])
            norm_sq = part if norm_sq is None else norm_sq + part
        norm_sq = norm_sq * (inv * inv)
        if self.norm_group is not None and dist.get_world_size(self.norm_group) > 1:
            if norm_sq.is_cuda:
                from ..symm import scalar_all_reduce
                norm_sq = scalar_all_reduce(norm_sq, self.norm_group)
            else:
                dist.all_reduce(norm_sq, op=dist.ReduceOp.SUM, group=self.norm_group)
        norm = norm_sq.sqrt()
        if grad_clip_value is not None and grad_clip_value > 0:
            scale = torch.clamp(grad_clip_value / (norm + 1e-6), max=1.0) * inv
        else:
            scale = torch.full_like(norm, inv)
        for s in self.shards:
            grad = s.grad_shard if s.sharded else s.buf.main_grad
            self._update(s, grad, scale, g)
            self._gather(s)
        self.grad_norm = norm
        return norm

    def step(self, grad_clip_value: float | None = None):
        self.prepare_step()
        return self.step_device(grad_clip_value)

    # -- stages -----------------------------------------------------------------------
    def _reduce(self, s: _Shard) -> torch.Tensor:
        mg = s.buf.main_grad
        if s.n == 1:
            return mg
        if self._comm is not None and self._comm.handles(s):
            for bi in range(len(s.buckets)):
                if bi not in s.reduced:
                    self._comm.reduce_bucket(s, bi, overlapped=False)
                    s.reduced.add(bi)
            return s.grad_shard
        if s.sharded:
            if mg.is_cuda:
                for b in s.buckets:             # rank r receives the r-th 1/n piece of every bucket
                    dist.reduce_scatter_tensor(s.grad_shard[b.off:b.off + b.seg], mg[b.lo:b.hi], op=dist.ReduceOp.SUM,
                                               group=s.group)
            else:                                   # Gloo has no reduce-scatter
                dist.all_reduce(mg, op=dist.ReduceOp.SUM, group=s.group)
                for b in s.buckets:
                    s.grad_shard[b.off:b.off + b.seg].copy_(mg[b.seg_lo:b.seg_lo + b.seg])
            return s.grad_shard
        dist.all_reduce(mg, op=dist.ReduceOp.SUM, group=s.group)
        return mg

    @staticmethod
    def _sumsq(x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            return native.sumsq(x)
        return x.double().pow(2).sum().float()

    def _update(self, s: _Shard, grad: torch.Tensor, scale: torch.Tensor, g: dict) -> None:
        b1, b2 = g["betas"]
        if self._comm is not None and self._comm.handles(s):
            for bi in range(len(s.buckets)):                 # bucket 0 first: the next forward pass needs it first
                self._comm.update_and_gather(s, bi, grad, scale, self.step_count, g, hyper=self._hyper)
            return
        for b in s.buckets:
            sl = slice(b.off, b.off + b.seg)
            out = s.buf.params[b.seg_lo:b.seg_lo + b.seg]
            if grad.is_cuda:
                native.adamw_step(s.master[sl], s.exp_avg[sl], s.exp_avg_sq[sl], grad[sl], out, scale, self.step_count,
                                  g["lr"], b1, b2, g["eps"], g["weight_decay"], hyper=self._hyper)
            else:
                m = s.master[sl]
                oracle.adamw_step(m, grad[sl], s.exp_avg[sl], s.exp_avg_sq[sl], self.step_count, g["lr"], b1, b2,
                                  g["eps"], g["weight_decay"], grad_scale=float(scale))
                out.copy_(m.to(out.dtype))

    def _gather(self, s: _Shard, via_library: bool = False) -> None:
        if not s.sharded:
            return
        if not via_library and self._comm is not None and self._comm.handles(s):
            return self._comm.gather_params(s)
        p = s.buf.params
        for b in s.buckets:
            mine = p[b.seg_lo:b.seg_lo + b.seg].clone()
            if p.is_cuda:
                dist.all_gather_into_tensor(p[b.lo:b.hi], mine, group=s.group)
            else:
                chunks = list(p[b.lo:b.hi].view(s.n, b.seg).unbind(0))
                dist.all_gather(chunks, mine, group=s.group)

    # -- full-buffer views of sharded state (checkpointing) -----------------------------
    def gather_full(self, s: _Shard, which: str) -> torch.Tensor:
        """fp32 tensor of the whole buffer for `which` in {master, exp_avg, exp_avg_sq}."""
        local = getattr(s, which)
        if not s.sharded:
            return local.clone()
        stack = torch.empty(s.n, s.len, dtype=torch.float32, device=local.device)
        dist.all_gather(list(stack.unbind(0)), local.contiguous(), group=s.group)
        return s.assemble_full(stack)

    def scatter_full(self, s: _Shard, which: str, full: torch.Tensor) -> None:
        getattr(s, which).copy_(s.take_local(full))

    def sync_params_from_master(self) -> None:
        """Rewrite the compute-dtype parameters from the fp32 master shards."""
        for s in self.shards:
            s.put_local(s.buf.params, s.master)
            self._gather(s, via_library=True)


class DistributedOptimizer:
    """ZeRO-1 front end with the reference's constructor and attribute
    forwarding. `optimizer` is a `FusedAdamW` built with `sharded=True`."""

    _OWN = {"optimizer", "process_group", "ranks_map", "num_parts", "verbose", "part_assignment",
            "tensor_dict", "rank", "world_size", "named_tensors"}

    def __init__(self, optimizer: FusedAdamW, process_group, ranks_map=None, num_parts=None, verbose=False,
                 named_tensors: "OrderedDict[str, torch.Tensor] | None" = None):
        object.__setattr__(self, "optimizer", optimizer)
        object.__setattr__(self, "process_group", process_group)
        object.__setattr__(self, "ranks_map", ranks_map)
        object.__setattr__(self, "verbose", verbose)
        self.rank = dist.get_rank(process_group) if process_group is not None else 0
        self.world_size = dist.get_world_size(process_group) if process_group is not None else 1
        self.num_parts = num_parts if num_parts is not None else self.world_size
        assert 1 <= self.num_parts <= self.world_size
        self.named_tensors = named_tensors if named_tensors is not None else OrderedDict()
        self.apply_zero1()

    def apply_zero1(self, part_assignment=None) -> None:
        """Whole-tensor ownership table keyed `(group_idx, param_idx)`; it only
        decides which rank WRITES which tensor's state into a checkpoint."""
        self.tensor_dict = OrderedDict(((0, i), t) for i, t in enumerate(self.named_tensors.values()))
        if part_assignment is None:
            if self.ranks_map is None:
                owners = list(range(self.num_parts))
            else:
                owners = [dist.get_group_rank(self.process_group, r) for r in self.ranks_map]
                assert len(set(owners)) == len(owners), f"Duplicate owners in ranks_map: {self.ranks_map}"
                self.num_parts = len(owners)
            part_assignment, _ = partition_tensors(self.tensor_dict, ranks_map=owners, verbose=self.verbose)
        self.part_assignment = part_assignment

    def owned_names(self) -> list[str]:
        names = list(self.named_tensors.keys())
        return [names[i] for (g, i), owner in self.part_assignment.items() if owner == self.rank]

    def __getattr__(self, name):
        return getattr(object.__getattribute__(self, "optimizer"), name)

    def __setattr__(self, name, value):
        if name in self._OWN or name.startswith("_"):
            object.__setattr__(self, name, value)
        else:
            setattr(self.optimizer, name, value)

    def __dir__(self):
        return sorted(set(dir(type(self)) + list(self.__dict__.keys()) + dir(self.optimizer)))

    def step(self, *args, **kwargs):
        return self.optimizer.step(*args, **kwargs)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.optimizer.zero_grad(set_to_none)
