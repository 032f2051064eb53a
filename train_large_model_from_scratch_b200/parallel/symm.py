"""Peer-memory collectives for the optimizer step (CUDA, world > 1).

The flat parameter and gradient buffers are allocated in symmetric memory
(`torch.distributed._symmetric_memory`: same size on every rank, every rank
can address every peer's copy over NVLink, plus an NVSwitch multicast address
when the fabric supports it). The kernels in `csrc/collectives.cu` then do the
communication themselves:

  reduce-scatter   each rank reads its 1/n slice of every peer's fp32 gradient
                   buffer (`multimem.ld_reduce` or P2P loads) -> fp32 shard,
                   with the sum of squares for the global norm; with
                   `--grad_wire_dtype bf16` the peers read a bf16 rounding of the
                   gradients instead (half the NVLink bytes, fp32 accumulation);
  AdamW + gather   the optimizer kernel stores the updated bf16 parameters into
                   every rank's replica (`multimem.st` or P2P stores);
  barriers         symmetric flag arrays with bounded waits.

`torch.distributed` (NCCL) stays for the control plane: rendezvous, the scalar
norm / loss reductions, checkpoint traffic. Set `TLM_COMM=nccl` to run the
optimizer collectives through NCCL instead (the baseline for comparisons), and
`TLM_NVLS=0` / `1` to force plain peer loads / stores or the NVSwitch multicast
mapping (default: multicast from 4 ranks up).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..ops import native


def symm_alloc(numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    import torch.distributed._symmetric_memory as symm_mem
    t = symm_mem.empty(numel, dtype=dtype, device=device)
    t.zero_()
    return t


def use_symm() -> bool:
    return (torch.cuda.is_available() and dist.is_initialized() and dist.get_world_size() > 1
            and os.environ.get("TLM_COMM", "symm") == "symm")


class _Peer:
    """Rendezvous result for one symmetric tensor."""

    def __init__(self, tensor: torch.Tensor, group):
        import torch.distributed._symmetric_memory as symm_mem
        self.handle = symm_mem.rendezvous(tensor, group=group)
        self.n = self.handle.world_size
        self.rank = self.handle.rank
        ptrs = list(self.handle.buffer_ptrs)
        self.ptr_array = (ctypes.c_void_p * self.n)(*ptrs)
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        # TLM_NVLS: 1 = always use the NVSwitch multicast mapping, 0 = never, unset = from 4 ranks up (at 2 ranks
        # plain peer loads are faster than the in-switch reduction: 0.90 ms vs 1.64 ms on a 512 MiB shard)
        mode = os.environ.get("TLM_NVLS", "auto")
        use = mode == "1" or (mode not in ("0", "1") and self.n >= 4)
        self.mc_ptr = mc if use else 0


class PeerCollectives:
    def __init__(self):
        self.state = {}          # id(shard) -> dict
        self.wire_dtype = "fp32"

    @classmethod
    def create(cls, fused, wire_dtype: str = "fp32") -> "PeerCollectives":
        self = cls()
        self.wire_dtype = wire_dtype
        for s in fused.shards:
            if s.n == 1 or not s.sharded:
                continue
            dev = s.buf.params.device
            flags = symm_alloc(64, torch.int32, dev)
            st = {
                "grad": _Peer(s.buf.main_grad, s.group),
                "param": _Peer(s.buf.params, s.group),
                "flags": _Peer(flags, s.group),
                "flags_t": flags,
                "partials": torch.zeros(native.lib().tlm_reduce_scatter_blocks(), dtype=torch.float32, device=dev),
                "sumsq": torch.zeros((), dtype=torch.float32, device=dev),
            }
            if wire_dtype == "bf16":
                wire = symm_alloc(s.buf.padded, torch.bfloat16, dev)
                st["wire_t"], st["wire"] = wire, _Peer(wire, s.group)
            self.state[id(s)] = st
            dist.barrier(group=s.group)
        torch.cuda.synchronize()
        return self

    def handles(self, s) -> bool:
        return id(s) in self.state

    def barrier(self, s) -> None:
        f = self.state[id(s)]["flags"]
        native._check(native.lib().tlm_peer_barrier(f.ptr_array, f.rank, f.n, 0, native._stream()), "peer_barrier")

    def reduce_grads(self, s) -> torch.Tensor:
        """Sum of every rank's gradient slice -> `s.grad_shard`; also leaves the
        slice's sum of squares in `self.last_sumsq(s)`. (Epoch argument 0: the kernels count their own
        flag epochs, so the launch is the same every step.)"""
        st = self.state[id(s)]
        g, f = st["grad"], st["flags"]
        if "wire" in st:
            w = st["wire"]
            native._check(native.lib().tlm_reduce_scatter_bf16(
                s.buf.main_grad.data_ptr(), st["wire_t"].data_ptr(), s.buf.padded, w.ptr_array,
                ctypes.c_void_p(w.mc_ptr) if w.mc_ptr else None, f.ptr_array, s.grad_shard.data_ptr(),
                st["partials"].data_ptr(), st["sumsq"].data_ptr(), s.lo, s.len, g.rank, g.n, 0,
                native._stream()), "reduce_scatter_bf16")
            return s.grad_shard
        native._check(native.lib().tlm_reduce_scatter(
            g.ptr_array, ctypes.c_void_p(g.mc_ptr) if g.mc_ptr else None, f.ptr_array, s.grad_shard.data_ptr(),
            st["partials"].data_ptr(), st["sumsq"].data_ptr(), s.lo, s.len, g.rank, g.n, 0,
            native._stream()), "reduce_scatter")
        return s.grad_shard

    def last_sumsq(self, s) -> torch.Tensor:
        return self.state[id(s)]["sumsq"]

    def update_and_gather(self, s, grad, scale, step: int, g: dict, hyper=None) -> None:
        st = self.state[id(s)]
        b1, b2 = g["betas"]
        pr = st["param"]
        lr, inv_bc1, inv_sqrt_bc2 = native.adam_hyper(max(step, 1), g["lr"], b1, b2)
        native._check(native.lib().tlm_adamw_gather(
            s.master.data_ptr(), s.exp_avg.data_ptr(), s.exp_avg_sq.data_ptr(), grad.data_ptr(), pr.ptr_array,
            ctypes.c_void_p(pr.mc_ptr) if pr.mc_ptr else None, scale.data_ptr(), s.lo, s.len, pr.rank, pr.n,
            lr, b1, b2, g["eps"], g["weight_decay"], inv_bc1, inv_sqrt_bc2, native._ptr(hyper), native._stream()),
            "adamw_gather")
        self.barrier(s)          # every replica complete before anyone's next forward reads it

    def gather_params(self, s) -> None:
        """Parameters were already distributed by `update_and_gather`."""
        return None


class PeerScalar:
    """Sum of one fp32 value over a process group through symmetric memory (one kernel: store to every peer's
    slot, flag exchange, ordered sum). Replaces NCCL for the two per-step scalars (gradient norm², loss), so a
    training step contains no library collective at all."""

    def __init__(self, group, device):
        self.group = group
        self.slots_t = symm_alloc(32, torch.float32, device)
        self.flags_t = symm_alloc(64, torch.int32, device)
        self.slots, self.flags = _Peer(self.slots_t, group), _Peer(self.flags_t, group)
        dist.barrier(group=group)

    def all_reduce(self, x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """`scale * sum_ranks(x)` for a 0-d fp32 CUDA tensor; returns a new 0-d tensor."""
        x = x.reshape(()).float().contiguous()
        out = torch.empty((), dtype=torch.float32, device=x.device)
        f = self.flags
        native._check(native.lib().tlm_peer_allreduce_scalar(self.slots.ptr_array, f.ptr_array, x.data_ptr(), out.data_ptr(),
                                                             float(scale), f.rank, f.n, 0, native._stream()),
                      "peer_allreduce_scalar")
        return out


_SCALARS: dict = {}


def scalar_all_reduce(x: torch.Tensor, group, scale: float = 1.0) -> torch.Tensor:
    """`scale * sum over group of x` for a 0-d tensor. On CUDA with the peer-memory path enabled this is one kernel
    of this package (`PeerScalar`); otherwise `dist.all_reduce`. Returns a new tensor; not differentiable."""
    n = dist.get_world_size(group) if group is not None else 1
    if n == 1:
        return x * scale if scale != 1.0 else x
    if x.is_cuda and use_symm() and n <= 16:
        key = id(group)
        ps = _SCALARS.get(key)
        if ps is None:
            ps = _SCALARS[key] = PeerScalar(group, x.device)
        return ps.all_reduce(x.detach(), scale).to(x.dtype)
    y = x.detach().clone()
    dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y * scale if scale != 1.0 else y
