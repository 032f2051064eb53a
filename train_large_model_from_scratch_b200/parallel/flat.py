"""Flat parameter / gradient storage.

All parameters of one replication class live back to back in ONE buffer of the
compute dtype (bf16 on the GPU), and their gradients in ONE fp32 buffer of the
same length (`main_grad`). Each `nn.Parameter` becomes a view into the first
and gets a `.main_grad` view into the second. That gives:

  * one reduce-scatter / one fused optimizer kernel / one all-gather per class
    instead of the reference's per-tensor loops (146 broadcasts + 146
    all-reduces per step for the 16-layer dense model,
    `distributed/zero1/distributed_optimizer.py:106-119`,
    `distributed/sequence_parallel/ulysses.py:27-41`);
  * adjacent matrices can be used as ONE GEMM operand without copies
    (q|k|v -> one `[Nq+2Nkv, D]` weight, gate|up -> one `[2I, D]` weight);
  * an even split of optimizer state over ranks, independent of tensor sizes.

Two classes exist: "dense" parameters are replicated on every rank of the
world (DP x SEP); "expert" parameters (names ending in one of
`EXPERT_LOCAL_PARAM_SUFFIXES`) differ between EP ranks and are replicated only
across the DP group (reference: `model/gpt.py:13-17`).
"""
from __future__ import annotations

from collections import OrderedDict

import torch

EXPERT_LOCAL_PARAM_SUFFIXES = (
    "mlp.experts_gate_weights",
    "mlp.experts_up_weights",
    "mlp.experts_down_weights",
)

_ALIGN = 8          # elements; keeps every view 16-byte aligned in bf16


def is_expert_param(name: str) -> bool:
    return name.endswith(EXPERT_LOCAL_PARAM_SUFFIXES)


class FlatBuffer:
    """One replication class: `params` (compute dtype), `main_grad` (fp32),
    and the name -> (offset, numel, shape) table."""

    def __init__(self, named_params: list[tuple[str, torch.nn.Parameter]], compute_dtype: torch.dtype,
                 device: torch.device, pad_to: int = 1, alloc=None, align: int = _ALIGN):
        """`align` (elements, a multiple of 8): every parameter starts at a multiple of it. With `align = 8 *
        shard count` any parameter boundary can be a bucket boundary of the sharded optimizer step (each
        rank's 1/n part of a bucket then starts 16-byte aligned). The gaps hold zeros and stay zero."""
        self.layout: "OrderedDict[str, tuple[int, int, torch.Size]]" = OrderedDict()
        assert align % _ALIGN == 0
        self.align = align
        off = 0
        seen: dict[int, str] = {}
        for name, p in named_params:
            if id(p) in seen:                      # tied weights appear once
                continue
            seen[id(p)] = name
            n = p.numel()
            if n % _ALIGN:
                raise ValueError(f"parameter {name} has {n} elements; a multiple of {_ALIGN} is required")
            off = ((off + align - 1) // align) * align
            self.layout[name] = (off, n, p.shape)
            off += n
        self.numel = off
        pad_to = max(1, pad_to)
        self.padded = ((off + pad_to - 1) // pad_to) * pad_to if off else 0
        self.compute_dtype = compute_dtype
        # `alloc(numel, dtype, device)` lets the caller place both buffers in symmetric
        # (peer-addressable) memory; it must return zero-filled storage.
        if alloc is None:
            alloc = lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev)
        self.params = alloc(self.padded, compute_dtype, device)
        self.main_grad = alloc(self.padded, torch.float32, device)
        self.init_fp32: torch.Tensor | None = torch.zeros(self.padded, dtype=torch.float32, device=device)
        for name, p in named_params:
            if name not in self.layout:
                continue
            o, n, shape = self.layout[name]
            self.init_fp32[o:o + n].copy_(p.data.reshape(-1).to(device=device, dtype=torch.float32))
            p.data = self.params[o:o + n].view(shape)
            p.main_grad = self.main_grad[o:o + n].view(shape)
            p.flat_offset = o
            p.flat_buffer = self
        self.params.copy_(self.init_fp32.to(compute_dtype))

    def view(self, offset: int, shape) -> tuple[torch.Tensor, torch.Tensor]:
        """(param view, main_grad view) of `shape` starting at element `offset`."""
        n = 1
        for s in shape:
            n *= s
        return self.params[offset:offset + n].view(shape), self.main_grad[offset:offset + n].view(shape)

    def zero_grad(self) -> None:
        self.main_grad.zero_()


def fuse_adjacent(params: list[torch.nn.Parameter]) -> torch.Tensor:
    """One 2-D weight covering several row-stacked matrices. When the parameters
    sit back to back in the same flat buffer the result is a VIEW (with a
    `main_grad` view); otherwise it is a differentiable `cat`."""
    p0 = params[0]
    buf = getattr(p0, "flat_buffer", None)
    cols = p0.shape[-1]
    rows = sum(p.shape[0] for p in params)
    if buf is not None:
        expect = p0.flat_offset
        ok = True
        for p in params:
            if getattr(p, "flat_buffer", None) is not buf or p.flat_offset != expect or p.shape[-1] != cols:
                ok = False
                break
            expect += p.numel()
        if ok:
            w, g = buf.view(p0.flat_offset, (rows, cols))
            w = w.detach()
            w.requires_grad_(p0.requires_grad)
            w.main_grad = g
            return w
    return None


def flatten_model(model: torch.nn.Module, compute_dtype: torch.dtype, device: torch.device,
                  dense_pad: int = 1, expert_pad: int = 1, alloc=None, align: int = _ALIGN) -> tuple[FlatBuffer, FlatBuffer | None]:
    """Move every parameter of `model` into flat storage. Returns (dense, expert)."""
    dense, expert = [], []
    for name, p in model.named_parameters():
        (expert if is_expert_param(name) else dense).append((name, p))
    dense_buf = FlatBuffer(dense, compute_dtype, device, dense_pad, alloc, align)
    expert_buf = FlatBuffer(expert, compute_dtype, device, expert_pad, alloc, align) if expert else None
    for m in model.modules():
        hook = getattr(m, "_post_flatten", None)
        if hook is not None:
            hook()
    return dense_buf, expert_buf
