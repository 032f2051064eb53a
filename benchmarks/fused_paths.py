"""Per-kernel times of the fused compute + exchange kernels inside a real multi-GPU step, against their rooflines.

    torchrun --nproc-per-node N -m benchmarks.fused_paths --config C     # Ulysses: QKV / attention / dO / dQKV exchanges
    torchrun --nproc-per-node N -m benchmarks.fused_paths --config D     # MoE: dispatch and combine

Runs a few un-recorded (eager) training steps of one of bench.py's configurations, records two steps with the
CUDA activity profiler on every rank, and has rank 0 print one JSON line per kernel: calls, mean duration and,
for the kernels that both compute and move data between GPUs, the time the slower of the two rooflines allows:

    t_roof = max(FLOPs / measured bf16 GEMM rate, bytes that must leave this GPU / peer-copy bandwidth)

with the measured rates of this class of machine (TLM_MEASURED_PEAKS json, else 1360 TFLOP/s sustained and
770 GB/s per direction). The durations are taken under the profiler, so they serve the comparison kernel by kernel
(shares and fractions), not as throughput numbers; the step time itself is what bench.py reports.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import re
import tempfile

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LINK_GBS = 770.0


def _load_bench():
    spec = importlib.util.spec_from_file_location("tlm_bench_cli", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _peak_tflops() -> float:
    path = os.environ.get("TLM_MEASURED_PEAKS")
    if path and os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops_sustained") or d.get("bf16_tflops") or 1360.0)
    return 1360.0


def _rooflines(bench, n: int) -> list[tuple[str, str, float, float]]:
    """(kernel-name regex, label, FLOPs per call, bytes leaving this GPU per call) for the fused kernels of the config."""
    m = bench.MODEL
    D, Hq, Hkv = m["hidden_size"], m["num_attention_heads"], m["num_key_value_heads"]
    hd = D // Hq
    B, T = bench.MICRO_BATCH, bench.SEQ_LEN
    sp = bench.SEP_SIZE
    rows = B * T // sp                                 # token rows of this rank
    away = (sp - 1) / sp                               # share of an exchanged tensor that leaves the GPU
    out = []
    if sp > 1 and not bench.EXTRA_FLAGS:
        nqkv = (Hq + 2 * Hkv) * hd
        attn_flops = 4.0 * B * (Hq // sp) * T * T * hd / 2          # causal: half of the score matrix
        out += [
            (r"gemm_heads(_pair)?_kernel<false", "QKV GEMM + RoPE + seq->head scatter", 2.0 * rows * nqkv * D, rows * nqkv * 2 * away),
            (r"attn_fwd_kernel", "attention forward + head->seq scatter of O", attn_flops, B * T * (Hq // sp) * hd * 2 * away),
            (r"gemm_heads(_pair)?_kernel<true", "out-proj dgrad + seq->head scatter of dO", 2.0 * rows * D * D, rows * D * 2 * away),
            (r"attn_bwd_kernel<\d+, true", "attention backward + head->seq return of dK, dV", 2.5 * attn_flops,
             B * T * (2 * Hkv // sp) * hd * 2 * away),
            (r"attn_dq_convert_kernel", "dQ conversion + RoPE^T + head->seq return of dQ", 0.0, B * T * (Hq // sp) * hd * 2 * away),
        ]
    if "--use_moe" in bench.EXTRA_FLAGS:
        f = bench.EXTRA_FLAGS
        k = int(f[f.index("--num_experts_per_tok") + 1])
        inter = int(f[f.index("--moe_intermediate_size") + 1])
        routed = rows * k                              # rows this rank sends (and, on average, receives)
        out += [
            (r"peer_scatter_rows_kernel", "dispatch / gradient routes: rows stored into the expert owners' buffers", 0.0, routed * D * 2 * away),
            (r"gemm(_pair)?_kernel<false, (false|true), 7", "expert down projection (and its backward route) + combine stores into the token owners' buffers",
             2.0 * routed * D * inter, routed * D * 2 * away),
        ]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="C")
    ap.add_argument("--steps", type=int, default=2, help="profiled steps")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    os.environ["TLM_CUDA_GRAPH"] = "0"                 # kernels must appear one by one in the activity record
    bench = _load_bench()
    bench._select_config(a.config, world)
    from train_large_model_from_scratch_b200.training import Trainer, build_config, parse_args
    from torch.profiler import ProfilerActivity, profile
    t = Trainer(build_config(parse_args(bench._flags(world, 8 + a.steps, tempfile.mkdtemp()))))
    step = 0
    for _ in range(4):
        t.train_step(step); step += 1
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            t.train_step(step); step += 1
        torch.cuda.synchronize()
    if rank == 0:
        peak = _peak_tflops()
        roofs = _rooflines(bench, world)
        rows = [(e.key, e.count, e.device_time_total / max(e.count, 1)) for e in prof.key_averages() if e.device_time_total > 0]
        rows.sort(key=lambda r: -r[1] * r[2])
        total = sum(c * us for _, c, us in rows)
        for name, count, us in rows[:40]:
            line = {"config": a.config, "n_gpus": world, "kernel": name[:110], "calls_per_step": count / a.steps,
                    "mean_us": round(us, 2), "share": round(count * us / total, 4)}
            for pat, label, flops, nbytes in roofs:
                if re.search(pat, name):
                    t_flop, t_link = flops / (peak * 1e12) * 1e6, nbytes / (LINK_GBS * 1e9) * 1e6
                    line.update({"fused_path": label, "roof_us": round(max(t_flop, t_link), 2),
                                 "roof_bound": "tensor" if t_flop >= t_link else "nvlink",
                                 "fraction_of_roof": round(max(t_flop, t_link) / us, 3),
                                 "nvlink_bytes_per_call": int(nbytes), "flops_per_call": flops})
                    break
            print(json.dumps(line), flush=True)
    t.close()


if __name__ == "__main__":
    main()
