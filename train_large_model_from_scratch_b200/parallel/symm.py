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
                   every rank's replica (`multimem.st` or P2P stores) and ends by
                   publishing per-bucket "parameters ready" words, which the first
                   GEMM of the next forward pass that reads the bucket waits for
                   in its producer warp (no barrier after the optimizer step);
  buckets          the buffer is cut at layer-group boundaries; every rank owns 1/n
                   of each bucket, and a bucket's reduce-scatter starts on a side
                   stream as soon as the last backward pass has left its layers;
  flags            symmetric flag arrays with bounded waits.

`torch.distributed` (NCCL) stays for the control plane: rendezvous, the scalar
norm / loss reductions, checkpoint traffic. Set `TLM_COMM=nccl` to run the
optimizer collectives through NCCL instead (the baseline for comparisons), and
`TLM_NVLS=0` / `1` to force plain peer loads / stores or the NVSwitch multicast
mapping (default: plain peer loads / stores at every group size).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..ops import native


# Debug aids that stand in for a device-side memory checker (both off by default):
#   TLM_SYMM_CANARY=1  every symmetric buffer gets guard bands in front of and behind its payload, filled with a
#                      pattern that `check_guards()` verifies: a peer store that misses its destination tile shows up
#                      as a damaged band instead of silent corruption of a neighbouring allocation.
#   TLM_EPOCH0=<int>   first value of every flag epoch counter (default 0). An odd value swaps the parity of all
#                      double-buffered slots, a value just below 2^31 makes the counters wrap during a short run; the
#                      results of a run must not depend on it.
_GUARD_ELEMS = 2048
_GUARDED: list = []


def _canary_on() -> bool:
    return os.environ.get("TLM_SYMM_CANARY", "0") == "1"


def epoch0() -> int:
    v = int(os.environ.get("TLM_EPOCH0", "0"))
    return ((v + 2 ** 31) % 2 ** 32) - 2 ** 31          # as int32


def _guard_pattern(dtype: torch.dtype):
    return -12345 if not dtype.is_floating_point else -24672.0       # exactly representable in bf16 and fp32


def symm_alloc(numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    import torch.distributed._symmetric_memory as symm_mem
    if not _canary_on():
        t = symm_mem.empty(numel, dtype=dtype, device=device)
        t.zero_()
        return t
    g = _GUARD_ELEMS
    whole = symm_mem.empty(numel + 2 * g, dtype=dtype, device=device)
    whole.fill_(_guard_pattern(dtype))
    payload = whole[g:g + numel]
    payload.zero_()
    _GUARDED.append((whole, numel))
    return payload


def alloc_flags(device: torch.device, n: int = 64) -> torch.Tensor:
    """Symmetric int32 flag array whose words (flags and the self-counted epoch) all start at `epoch0()`."""
    t = symm_alloc(n, torch.int32, device)
    if epoch0():
        t.fill_(epoch0())
    return t


def check_guards() -> list[str]:
    """Damaged guard bands of this rank's symmetric buffers (empty list = intact). Call after a synchronize."""
    bad = []
    for i, (whole, numel) in enumerate(_GUARDED):
        g = _GUARD_ELEMS
        pat = _guard_pattern(whole.dtype)
        for name, band in (("front", whole[:g]), ("back", whole[g + numel:])):
            n_bad = int((band != pat).sum().item())
            if n_bad:
                bad.append(f"buffer {i} ({whole.dtype}, {numel} elements): {n_bad} damaged words in the {name} guard band")
    return bad


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
        # the handle describes the allocation; `tensor` may be a view into it (payload behind a guard band)
        off = tensor.data_ptr() - int(self.handle.buffer_ptrs[self.rank])
        assert 0 <= off < (1 << 40), "the tensor does not lie in its symmetric allocation"
        ptrs = [int(p) + off for p in self.handle.buffer_ptrs]
        self.ptr_array = (ctypes.c_void_p * self.n)(*ptrs)
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        mc = mc + off if mc else 0
        # TLM_NVLS=1 selects the NVSwitch multicast mapping (`multimem.ld_reduce` / `multimem.st`); the default is plain
        # peer loads / stores. Measured on a 1 GiB fp32 buffer: reduce-scatter 0.85 - 0.90 ms (peer loads) vs 1.63 ms
        # (in-switch reduction) at 2 ranks, 1.25 vs 1.57 ms at 4; AdamW + all-gather 0.64 vs 0.80 ms at 4. The in-switch
        # reduction takes ~1.6 ms at any group size because every GPU sends its WHOLE buffer through its links (its own
        # shard included), 1 GiB at ~670 GB/s, while peer loads send (n-1)/n of it; the multicast form only saves
        # ingress, and the links are full duplex. More loads in flight per thread did not change it.
        mode = os.environ.get("TLM_NVLS", "0")
        use = mode == "1"
        self.mc_ptr = mc if use else 0


class PeerCollectives:
    """Bucket-wise gradient reduce-scatter and AdamW + parameter all-gather over peer memory.

    Per flat buffer: one symmetric flag array for the reduce-scatter's "my gradients of this bucket are final"
    exchange (epochs counted by the kernels, one per launch, same launch order on every rank) and one for the
    "parameters ready" words that the update kernels publish and the consumers of the parameters wait for
    (`csrc/common.cuh`, READY_*). Reductions that start during the backward pass run on `comm_stream`
    with a small grid; `join()` brings the main stream behind them."""

    def __init__(self):
        self.state = {}          # id(shard) -> dict
        self.wire_dtype = "fp32"
        self.comm_stream = None
        self._forked = False
        # grid of a reduce-scatter that runs under the backward pass (blocks of 128 threads); 0: no overlap, every
        # bucket is reduced after the backward pass with the full grid
        self.overlap_blocks = int(os.environ.get("TLM_RS_OVERLAP_BLOCKS", "296"))

    @classmethod
    def create(cls, fused, wire_dtype: str = "fp32") -> "PeerCollectives":
        self = cls()
        self.wire_dtype = wire_dtype
        L = native.lib()
        for s in fused.shards:
            if s.n == 1 or not s.sharded:
                continue
            assert len(s.buckets) <= L.tlm_ready_max_buckets() and s.n <= 16
            dev = s.buf.params.device
            if self.comm_stream is None:
                self.comm_stream = torch.cuda.Stream(device=dev, priority=-1)
            flags = alloc_flags(dev)
            ready = symm_alloc(L.tlm_ready_ints(), torch.int32, dev)
            if epoch0():                       # flag words and update counts start at epoch0; block counters at 0
                ready[:L.tlm_ready_max_buckets() * 17].fill_(epoch0())
            st = {
                "grad": _Peer(s.buf.main_grad, s.group),
                "param": _Peer(s.buf.params, s.group),
                "flags": _Peer(flags, s.group),
                "flags_t": flags,
                "ready": _Peer(ready, s.group),
                "ready_t": ready,
                "partials": torch.zeros(L.tlm_reduce_scatter_blocks(), dtype=torch.float32, device=dev),
                "sumsq": torch.zeros(len(s.buckets), dtype=torch.float32, device=dev),
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

    # -- gradients -----------------------------------------------------------------------
    def reduce_bucket(self, s, bi: int, overlapped: bool) -> None:
        """Sum of every rank's gradients over this rank's piece of bucket `bi` -> `s.grad_shard`, and the piece's
        sum of squares -> entry `bi` of the shard's sumsq vector. The kernel's prologue is the flag exchange
        that tells the peers "my gradients of this bucket are final" and waits for theirs. `overlapped`: the
        backward pass is still running; launch on the communication stream behind everything queued so far,
        with a grid that leaves the SMs to the GEMMs."""
        st = self.state[id(s)]
        b = s.buckets[bi]
        g, f = st["grad"], st["flags"]
        out = s.grad_shard[b.off:b.off + b.seg]
        sumsq = st["sumsq"][bi:bi + 1]
        blocks = self.overlap_blocks if overlapped else 0
        if overlapped:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            self._forked = True
            ctx = torch.cuda.stream(self.comm_stream)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx:
            if "wire" in st:
                w = st["wire"]
                native._check(native.lib().tlm_reduce_scatter_bf16(
                    s.buf.main_grad.data_ptr(), st["wire_t"].data_ptr(), b.lo, b.hi - b.lo, w.ptr_array,
                    ctypes.c_void_p(w.mc_ptr) if w.mc_ptr else None, f.ptr_array, out.data_ptr(),
                    st["partials"].data_ptr(), sumsq.data_ptr(), b.seg_lo, b.seg, g.rank, g.n, 0, blocks,
                    native._stream()), "reduce_scatter_bf16")
            else:
                native._check(native.lib().tlm_reduce_scatter(
                    g.ptr_array, ctypes.c_void_p(g.mc_ptr) if g.mc_ptr else None, f.ptr_array, out.data_ptr(),
                    st["partials"].data_ptr(), sumsq.data_ptr(), b.seg_lo, b.seg, g.rank, g.n, 0, blocks,
                    native._stream()), "reduce_scatter")

    def join(self) -> None:
        """The main stream waits for the reductions queued on the communication stream."""
        if self._forked:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            self._forked = False

    def last_sumsq(self, s) -> torch.Tensor:
        return self.state[id(s)]["sumsq"].sum()

    # -- parameters ----------------------------------------------------------------------
    def update_and_gather(self, s, bi: int, grad, scale, step: int, g: dict, hyper=None) -> None:
        """Clipped AdamW on this rank's piece of bucket `bi`; the bf16 result goes into every rank's replica and
        the kernel ends by publishing the bucket's "parameters ready" word to all ranks."""
        st = self.state[id(s)]
        b = s.buckets[bi]
        b1, b2 = g["betas"]
        pr, rd = st["param"], st["ready"]
        sl = slice(b.off, b.off + b.seg)
        lr, inv_bc1, inv_sqrt_bc2 = native.adam_hyper(max(step, 1), g["lr"], b1, b2)
        native._check(native.lib().tlm_adamw_gather(
            s.master[sl].data_ptr(), s.exp_avg[sl].data_ptr(), s.exp_avg_sq[sl].data_ptr(), grad[sl].data_ptr(),
            pr.ptr_array, ctypes.c_void_p(pr.mc_ptr) if pr.mc_ptr else None, scale.data_ptr(), b.seg_lo, b.seg, pr.rank,
            pr.n, lr, b1, b2, g["eps"], g["weight_decay"], inv_bc1, inv_sqrt_bc2, native._ptr(hyper), rd.ptr_array, bi,
            native._stream()), "adamw_gather")

    def gather_params(self, s) -> None:
        """Parameters were already distributed by `update_and_gather`."""
        return None

    def wait_first_buckets(self, shards) -> None:
        """Stream-ordered bounded wait for the buckets of layer group 0 (embedding, first norm; every bucket of
        a buffer whose buckets are not tied to layer groups): no GEMM is their first reader."""
        # gates armed for a GEMM that never came (a forward pass that was cut short) become plain wait kernels
        native._check(native.lib().tlm_gemm_flush_param_waits(native._stream()), "flush_param_waits")
        for s in shards:
            st = self.state.get(id(s))
            if st is None:
                continue
            for bi, b in enumerate(s.buckets):
                if b.group == 0:
                    native._check(native.lib().tlm_wait_params_ready(st["ready_t"].data_ptr(), bi, s.n, native._stream()),
                                  "wait_params_ready")

    def arm_group(self, shards, g: int) -> None:
        """The next GEMM launched waits, in its producer warp, for every rank's update of group `g`'s buckets."""
        if g == 0:
            return
        # gates of the previous group that no projection GEMM took (a block that does not start with one)
        native._check(native.lib().tlm_gemm_flush_param_waits(native._stream()), "flush_param_waits")
        for s in shards:
            st = self.state.get(id(s))
            if st is None:
                continue
            for bi, b in enumerate(s.buckets):
                if b.group == g:
                    native._check(native.lib().tlm_gemm_arm_param_wait(st["ready_t"].data_ptr(), bi, s.n), "arm_param_wait")


class PeerScalar:
    """Sum of one fp32 value over a process group through symmetric memory (one kernel: store to every peer's
    slot, flag exchange, ordered sum). Replaces NCCL for the two per-step scalars (gradient norm², loss), so a
    training step contains no library collective at all."""

    def __init__(self, group, device):
        self.group = group
        self.slots_t = symm_alloc(32, torch.float32, device)
        self.flags_t = alloc_flags(device)
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
