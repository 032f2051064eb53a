"""Peer-memory communication kernels against their NVLink roofline.

    torchrun --nproc-per-node N -m benchmarks.comm [--mb 1024]

Times, with CUDA events and the maximum over ranks, the kernels that move data between GPUs:

  reduce_scatter   fp32 and bf16 wire, P2P loads and `multimem.ld_reduce`
  adamw_gather     fused AdamW + parameter all-gather (P2P stores and `multimem.st`)
  nccl             `reduce_scatter_tensor` / `all_gather_into_tensor` on the same buffers, for reference

and prints one JSON line per case with the bytes that must cross NVLink per rank, the achieved rate and its
fraction of the measured peer-copy bandwidth (770 GB/s per direction per GPU on this class of machine).
For the reduce-scatter a rank receives (n-1)/n of its shard from peers ((n-1) shard-sized reads through P2P, one
switch-reduced shard through NVLS); for the all-gather it sends its shard to n-1 peers (once through NVLS).
The byte column counts what a rank RECEIVES. In the other direction a rank's links carry (n-1)/n of its buffer with
peer loads but its whole buffer with the in-switch reduction (the switch pulls every rank's copy of every shard), which
is why the multicast reduce-scatter takes the same time at every group size and never beats peer loads.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def _time(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=1024, help="size of the flat fp32 gradient buffer in MiB")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from train_large_model_from_scratch_b200.ops import native
    from train_large_model_from_scratch_b200.parallel.symm import _Peer, symm_alloc
    dev = torch.device("cuda", torch.cuda.current_device())
    n = (a.mb << 20) // 4
    n -= n % (1024 * world)
    shard = n // world
    grads = symm_alloc(n, torch.float32, dev)
    grads.normal_()
    wire = symm_alloc(n, torch.bfloat16, dev)
    params = symm_alloc(n, torch.bfloat16, dev)
    flags = symm_alloc(64, torch.int32, dev)
    group = dist.group.WORLD
    os.environ["TLM_NVLS"] = "1"
    pg, pw, pp, pf = _Peer(grads, group), _Peer(wire, group), _Peer(params, group), _Peer(flags, group)
    out = torch.zeros(shard, device=dev)
    partials = torch.zeros(native.lib().tlm_reduce_scatter_blocks(), device=dev)
    sumsq = torch.zeros((), device=dev)
    master, m, v = torch.randn(shard, device=dev), torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
    scale = torch.ones((), device=dev)
    lo = rank * shard
    epoch = [0]
    st = lambda: torch.cuda.current_stream().cuda_stream
    vp = lambda x: ctypes.c_void_p(x) if x else None

    def rs(mc, bf16, blocks=0):
        epoch[0] += 1
        if bf16:
            native._check(native.lib().tlm_reduce_scatter_bf16(
                grads.data_ptr(), wire.data_ptr(), 0, n, pw.ptr_array, vp(pw.mc_ptr if mc else 0), pf.ptr_array,
                out.data_ptr(), partials.data_ptr(), sumsq.data_ptr(), lo, shard, rank, world, epoch[0], blocks, st()),
                "rs_bf16")
        else:
            native._check(native.lib().tlm_reduce_scatter(
                pg.ptr_array, vp(pg.mc_ptr if mc else 0), pf.ptr_array, out.data_ptr(), partials.data_ptr(),
                sumsq.data_ptr(), lo, shard, rank, world, epoch[0], blocks, st()), "rs")

    ready = symm_alloc(native.lib().tlm_ready_ints(), torch.int32, dev)
    pr = _Peer(ready, group)

    def ag(mc):
        # the update kernel publishes "parameters ready"; the one-warp wait that follows is what the first reader
        # of the parameters does (in training: the producer warp of the first GEMM of the next forward pass)
        native._check(native.lib().tlm_adamw_gather(
            master.data_ptr(), m.data_ptr(), v.data_ptr(), out.data_ptr(), pp.ptr_array, vp(pp.mc_ptr if mc else 0),
            scale.data_ptr(), lo, shard, rank, world, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1.0, 1.0, None, pr.ptr_array, 0, st()),
            "adamw_gather")
        native._check(native.lib().tlm_wait_params_ready(ready.data_ptr(), 0, world, st()), "wait_params_ready")

    has_mc = bool(pg.mc_ptr)
    cases = []
    for mc in ([False, True] if has_mc else [False]):
        tag = "multimem" if mc else "p2p"
        for bf16 in (False, True):
            el = 2 if bf16 else 4
            wire_bytes = shard * el * (1 if mc else (world - 1))
            cases.append((f"reduce_scatter {'bf16' if bf16 else 'fp32'} wire, {tag}", lambda mc=mc, bf16=bf16: rs(mc, bf16), wire_bytes))
        cases.append((f"reduce_scatter fp32 wire, {tag}, 296 blocks of 128 threads (the grid used under the backward pass)",
                      lambda mc=mc: rs(mc, False, 296), shard * 4 * (1 if mc else (world - 1))))
        cases.append((f"adamw + all-gather (bf16 params), {tag}", lambda mc=mc: ag(mc), shard * 2 * (1 if mc else (world - 1))))
    nccl_out = torch.empty(shard, device=dev)
    cases.append(("nccl reduce_scatter_tensor fp32", lambda: dist.reduce_scatter_tensor(nccl_out, grads), shard * 4 * (world - 1)))
    pbuf = torch.empty(n, dtype=torch.bfloat16, device=dev)
    cases.append(("nccl all_gather_into_tensor bf16", lambda: dist.all_gather_into_tensor(pbuf, pbuf[lo:lo + shard].clone()),
                  shard * 2 * (world - 1)))
    for name, fn, nbytes in cases:
        ms = _time(fn)
        if rank == 0:
            gbs = nbytes / ms / 1e6
            print(json.dumps({"case": name, "n_gpus": world, "buffer_MiB": a.mb, "ms": round(ms, 4),
                              "nvlink_bytes_per_rank_MB": round(nbytes / 1e6, 1), "GBps_per_rank": round(gbs, 1),
                              "frac_of_770GBps": round(gbs / LINK_GBS, 3)}), flush=True)
    native.raise_on_device_status()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
