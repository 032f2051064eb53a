"""Headline benchmark: training throughput (tokens/s, whole job) of the
0.25B-class dense GPT (16 layers, hidden 1024, 16 query / 8 KV heads, SwiGLU
4096, vocab 50304, tied embeddings, RoPE), bf16, sequence length 4096,
micro-batch 8 per GPU, 2 gradient-accumulation micro-steps per optimizer step,
ZeRO-1 over DP = N, grad-clip 1.0, synthetic uniform-random tokens, random-init
weights.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch with torchrun (one rank per GPU). Rank 0 prints ONE JSON line.

`value`  : device-timed (CUDA events, max over ranks) tokens/s with the step's
           batches already resident on the device.
`e2e`    : the same metric through the public `Trainer.train_step` API with the
           trainer's own data loader: every step copies its input ids / labels
           from pinned host memory and reads the loss back to the host.
`--impl reference` runs the unmodified reference from `baseline/_ref` through
its own `Trainer` for the same model and batch shape.

The default run (configuration B, the headline) is followed by the other half
of the benchmark: the 0.3B-class MoE (`--config D`, SEP = EP = N) and the same
dense model under Ulysses sequence parallelism (`--config C`, SEP = N), each
measured in a fresh child job on the same GPUs after the headline job has
released them, with its own warm-up, timing and clock samples; their results
are the `moe` and `ulysses` entries of the JSON line (both arms do this, so the
two lines can be compared entry by entry). `--no-extras` skips them.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

MODEL = dict(num_layer=16, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
             intermediate_size=4096, vocab_size=50304, block_size=4096)
SEQ_LEN, MICRO_BATCH, GRAD_ACCUM = 4096, 8, 2
SEP_SIZE, EXTRA_FLAGS, _CONFIG = 1, [], "B"
MODEL_NAME = "dense GPT 16L/1024/16q-8kv/SwiGLU-4096/vocab 50304 tied (0.30B params)"
BASELINE_TOKENS_PER_S = None          # the reference publishes no number

# Other configurations of the same benchmark (`--config`); "B" above is the headline one.
#   C: the same model under Ulysses sequence parallelism over all GPUs, 4096 tokens per rank, micro-batch 1
#   D: 0.3B-class MoE, 8 experts top-2, expert hidden 2048, SEP = number of GPUs (SP and EP share the group)
#   E: 3B-class dense, head dim 128, DP x SEP = (N/2) x 2
#   S: the reference's shipped debug_gpt_0.25b shape (12 layers, 32 query / 4 KV heads of dim 32)
CONFIGS = {
    "C": dict(model=MODEL, name="dense 0.30B, Ulysses sep=N, seq 4096 x N", seq_per_rank=4096, micro=1, ga=2,
              sep="all"),
    "D": dict(model=dict(num_layer=12, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                         intermediate_size=4096, vocab_size=50304, block_size=4096),
              name="MoE 12L/1024/16q-8kv/8 experts top-2/expert hidden 2048", seq=4096, micro=4, ga=2, sep="all",
              extra=["--use_moe", "--num_experts", "8", "--num_experts_per_tok", "2", "--moe_intermediate_size", "2048"]),
    "E": dict(model=dict(num_layer=36, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
                         intermediate_size=8192, vocab_size=50304, block_size=4096),
              name="dense 36L/3072/24q-8kv hd128/SwiGLU-8192 (3.78B params)", seq=4096, micro=2, ga=2, sep=2),
    "S": dict(model=dict(num_layer=12, hidden_size=1024, num_attention_heads=32, num_key_value_heads=4,
                         intermediate_size=4096, vocab_size=50304, block_size=4096),
              name="dense 12L/1024/32q-4kv hd32/SwiGLU-4096 (shipped debug_gpt_0.25b)", seq=4096, micro=8, ga=2, sep=1),
}


def _select_config(name: str, n_gpus: int) -> None:
    global MODEL, SEQ_LEN, MICRO_BATCH, GRAD_ACCUM, SEP_SIZE, EXTRA_FLAGS, MODEL_NAME, _CONFIG
    if name == "B":
        return
    _CONFIG = name
    c = CONFIGS[name]
    SEP_SIZE = n_gpus if c["sep"] == "all" else min(int(c["sep"]), n_gpus)
    SEQ_LEN = c["seq_per_rank"] * SEP_SIZE if "seq_per_rank" in c else c["seq"]
    MODEL = dict(c["model"], block_size=max(4096, SEQ_LEN))
    MICRO_BATCH, GRAD_ACCUM, EXTRA_FLAGS, MODEL_NAME = c["micro"], c["ga"], list(c.get("extra", [])), c["name"]


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock / throttle reasons of this rank's GPU with nvidia-smi
    (read-only queries) while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(suffix=".csv")
        self.gpu, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1])); mx.append(float(p[2]))
                except ValueError:
                    continue
                for n, v in zip(names, p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.remove(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _visible_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


def _dist_env():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    return int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])


def _timed(torch, dist, world, fn, steps):
    """barrier + sync, K steps between CUDA events, sync + barrier; max over ranks (ms)."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = (time.time() - t0) * 1e3
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()), wall


def _steps_for(torch, dist, world, fn, steps: int, min_timed_s: float) -> int:
    """Number of timed steps: `steps`, raised (to at most 400) so that the timed region lasts `min_timed_s`
    seconds: configurations with short steps otherwise finish between two clock samples. All ranks agree."""
    if min_timed_s <= 0:
        return steps
    ms, _ = _timed(torch, dist, world, fn, 2)
    need = int(min_timed_s * 1e3 / max(ms / 2, 1e-3)) + 1
    return max(steps, min(need, 400))


def _flags(n_gpus: int, steps_total: int, log_dir: str) -> list[str]:
    dp = n_gpus // SEP_SIZE
    tokens = SEQ_LEN * MICRO_BATCH * GRAD_ACCUM * dp
    samples = MICRO_BATCH * GRAD_ACCUM * dp * (steps_total + 4)
    f = ["--use_mock_data", "--mock_data_num_samples", str(samples), "--total_batch_size", str(tokens),
         "--batch_size", str(MICRO_BATCH), "--seq_len", str(SEQ_LEN), "--max_steps", str(steps_total + 4),
         "--warmup_steps", "2", "--max_lr", "6e-4", "--min_lr", "6e-5", "--weight_decay", "0.1",
         "--grad_clip_value", "1.0", "--debug", "--sep_size", str(SEP_SIZE), "--use_distributed_optimizer", "--tied_lm_head",
         "--pin_memory", "--precision", "bf16", "--log_dir", log_dir, "--exp_name", "bench"]
    for k, v in MODEL.items():
        f += [f"--{k}", str(v)]
    return f + EXTRA_FLAGS


def _result(impl, n, steps, warmup, ms_total, tokens_per_step, clocks, extra):
    ms_step = ms_total / steps
    value = tokens_per_step / (ms_step / 1e3)
    out = {
        "metric": ("training throughput, 0.25B-class dense GPT (tokens/s, whole job, max over ranks)" if _CONFIG == "B"
                   else f"training throughput, config {_CONFIG} (tokens/s, whole job, max over ranks)"),
        "value": value, "unit": "tokens/s", "n_gpus": n, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
        "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights", "impl": impl,
        "config": {"model": MODEL_NAME,
                   "global_batch": tokens_per_step, "seq_len": SEQ_LEN, "micro_batch": MICRO_BATCH,
                   "grad_accum": GRAD_ACCUM,
                   "parallelism": f"dp{n // SEP_SIZE} zero1" + (f" x sep{SEP_SIZE}" if SEP_SIZE > 1 else ""),
                   "l2": "per-step working set (~20 GB of activations) far exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks,
    }
    out.update(extra)
    return out


# --------------------------------------------------------------------------- our implementation
def run_ours(args) -> dict:
    rank, local_rank, world = _dist_env()
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from train_large_model_from_scratch_b200.ops import native
    from train_large_model_from_scratch_b200.training import Trainer, build_config, parse_args

    n, K, W = args.gpus, args.steps, args.warmup
    assert world == n, f"--gpus {n} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {n}"
    if not torch.cuda.is_available():                  # the CPU path runs, but it is the oracle, not the benchmark
        raise SystemExit("bench.py measures the sm_100a kernels: no CUDA device is visible")
    log_dir = tempfile.mkdtemp(prefix="tlm_bench_")
    cfg = build_config(parse_args(_flags(n, 2 * (K + W) + 900, log_dir)))
    trainer = Trainer(cfg)
    dev = trainer.device
    tokens_per_step = SEQ_LEN * MICRO_BATCH * GRAD_ACCUM * (n // SEP_SIZE)

    # ---- device-resident batches (kernel-side number) ----
    gen = torch.Generator().manual_seed(1234 + rank // SEP_SIZE)      # ranks of one SEP group share their sequences
    pool = []
    for _ in range(4):
        step_batches = []
        for _ in range(GRAD_ACCUM):
            d = torch.randint(0, MODEL["vocab_size"], (MICRO_BATCH, SEQ_LEN + 1), generator=gen)
            step_batches.append({"input_ids": d[:, :-1].to(dev), "labels": d[:, 1:].to(dev)})
        pool.append(step_batches)
    counter = {"i": 0}

    def step_device(i):
        trainer.train_step(counter["i"], batches=pool[counter["i"] % len(pool)])
        counter["i"] += 1

    for i in range(W):
        step_device(i)
    native.raise_on_device_status()
    K = _steps_for(torch, dist, world, step_device, K, args.min_timed_s)
    sampler = ClockSampler(_visible_gpu_index(local_rank))
    sampler.start()
    native.reset_launch_count()
    ms_dev, _ = _timed(torch, dist, world, step_device, K)
    launches = native.launch_count()
    clocks = sampler.stop()
    native.raise_on_device_status()

    # ---- end to end through the public API: loader -> pinned H2D -> step -> loss D2H ----
    losses = []

    def step_e2e(i):
        r = trainer.train_step(counter["i"])
        counter["i"] += 1
        losses.append(float(r["loss"]))            # device -> host read of the step's result

    for i in range(max(1, W // 2)):
        step_e2e(i)
    ms_e2e, _ = _timed(torch, dist, world, step_e2e, K)
    h2d = 2 * GRAD_ACCUM * MICRO_BATCH * (SEQ_LEN // SEP_SIZE) * 8       # ids + labels, int64, per rank
    extra = {
        "e2e": {"value": tokens_per_step / (ms_e2e / K / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                "h2d_bytes_per_step": h2d * n, "d2h_bytes_per_step": 4 * n},
        "gpu_launches": launches,
        "final_loss": losses[-1] if losses else None,
    }
    out = _result("ours", n, K, W, ms_dev, tokens_per_step, clocks, extra)
    if world > 1:
        dist.barrier()
    trainer.close()
    del trainer, pool, step_device, step_e2e              # release the GPUs for the jobs that follow
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out if rank == 0 else None


# --------------------------------------------------------------------------- the reference, unmodified
def run_reference(args) -> dict:
    rank, local_rank, world = _dist_env()
    if not os.path.isdir(os.path.join(REF_DIR, "training")):
        return {"impl": "reference", "unavailable": "baseline/_ref is missing (reference tree not installed)"} \
            if rank == 0 else None
    sys.path[:] = [REF_DIR] + [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    if world > 1 and "TORCHINDUCTOR_COMPILE_THREADS" not in os.environ:
        # every rank compiles the same model: share the host's cores between the ranks' compiler worker pools
        os.environ["TORCHINDUCTOR_COMPILE_THREADS"] = str(max(1, min(8, (os.cpu_count() or 8) // world)))
    import torch
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "the reference requires CUDA (model/gpt.py:42)"} if rank == 0 else None
    import torch.distributed as dist
    from training import Trainer, build_config, parse_args                    # the reference's own modules

    n, K, W = args.gpus, args.steps, args.warmup
    log_dir = tempfile.mkdtemp(prefix="ref_bench_")
    flags = [f for f in _flags(n, 2 * (K + W) + 500, log_dir)]
    state = {}

    def build(use_compile: bool):
        cfg = build_config(parse_args(flags + (["--use_compile"] if use_compile else [])))
        trainer = Trainer(cfg)
        if cfg.model.use_moe and args.moe_fallback:
            for blk in trainer.raw_model.blocks:
                blk.mlp.grouped_gemm_supported = False
        # what Trainer.train() does before and inside its loop (training/trainer.py:308-351)
        trainer.results = {}
        trainer.train_loader_iter = enumerate(trainer.train_loader)
        trainer.start_step = 0
        trainer._init_profiler(cfg)
        state.update(cfg=cfg, trainer=trainer, compiled=use_compile)

    tokens_per_step = SEQ_LEN * MICRO_BATCH * GRAD_ACCUM * (n // SEP_SIZE)
    counter = {"i": 0}
    losses = []

    def step(i):
        trainer = state["trainer"]
        trainer.one_step_results = {}
        trainer._one_training_step(state["cfg"], counter["i"])
        torch.cuda.synchronize()
        losses.append(trainer.one_step_results["loss"].item())
        counter["i"] += 1

    # The reference's launch scripts run it with its tracing compiler on (USE_COMPILE=1 ->
    # `--use_compile`, scripts/debug_gpt_0.25b/pretrain.sh:43,79-81), which is also its faster mode on this
    # hardware, so that is the mode measured; if the compiler cannot run here, its eager mode is measured
    # and the reason is reported.
    compile_note = None
    build(bool(args.ref_compile))
    try:
        step(0)
    except Exception as e:
        if not args.ref_compile:
            raise
        compile_note = f"{type(e).__name__}: {str(e).splitlines()[0][:160] if str(e) else ''}"
        ok = torch.tensor([0], device="cuda")
    else:
        ok = torch.tensor([1], device="cuda")
    if args.ref_compile:
        if world > 1:
            try:
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            except Exception:
                ok.zero_()
        if int(ok.item()) == 0:                        # every rank falls back together
            dist.destroy_process_group()
            state.clear()
            counter["i"] = 0
            losses.clear()
            build(False)
            step(0)
    cfg, trainer = state["cfg"], state["trainer"]
    for i in range(max(0, W - 1)):
        step(i)
    K = _steps_for(torch, dist, world, step, K, args.min_timed_s)
    sampler = ClockSampler(_visible_gpu_index(local_rank))
    sampler.start()
    ms, _ = _timed(torch, dist, world, step, K)
    clocks = sampler.stop()
    h2d = 2 * GRAD_ACCUM * MICRO_BATCH * (SEQ_LEN // SEP_SIZE) * 8
    extra = {"e2e": {"value": tokens_per_step / (ms / K / 1e3), "unit": "tokens/s", "ms_per_step": ms / K,
                     "h2d_bytes_per_step": h2d * n, "d2h_bytes_per_step": 4 * n},
             "gpu_launches": None, "final_loss": losses[-1], "use_compile": bool(state["compiled"])}
    if compile_note:
        extra["compile_fallback"] = compile_note
    if cfg.model.use_moe:
        extra["moe_expert_path"] = ("padded bmm (grouped_gemm_supported forced off: its grouped_mm call needs "
                                    "moe_intermediate_size == hidden_size)" if args.moe_fallback else "grouped_mm")
    out = _result("reference", n, K, W, ms, tokens_per_step, clocks, extra)
    dist.destroy_process_group()
    del trainer, step
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out if rank == 0 else None


def _free_port() -> int:
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


EXTRAS = (("moe", "D"), ("ulysses", "C"))
_KEEP = ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "impl", "config", "clocks", "e2e", "gpu_launches",
         "final_loss", "use_compile", "compile_fallback", "unavailable", "moe_expert_path")


def run_extras(args) -> dict:
    """Measure the other configurations of the benchmark, one child job each, on the GPUs the finished headline
    job has released. Called by rank 0 only, after its process group is gone. A child that fails or exceeds its
    time limit is reported as `{"unavailable": ...}`; it never takes the headline result with it."""
    out = {}
    env = {k: v for k, v in os.environ.items()
           if not (k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_NAME",
                         "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS")
                   or k.startswith("TORCHELASTIC_") or k.startswith("TORCH_NCCL_ASYNC"))}
    steps = min(args.steps, 20)
    for key, cfg in EXTRAS:
        tail = [os.path.join(ROOT, "bench.py"), "--gpus", str(args.gpus), "--steps", str(steps), "--warmup", str(args.warmup),
                "--config", cfg, "--impl", args.impl, "--no-extras", "--ref-compile", str(args.ref_compile),
                "--moe-fallback", str(args.moe_fallback), "--min-timed-s", "3"]
        if args.gpus > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(_free_port())] + tail
        else:
            cmd = [sys.executable] + tail
            # a single-process child makes its own rendezvous: never on the port this process's (possibly still
            # listening) store used
            env["MASTER_ADDR"], env["MASTER_PORT"] = "127.0.0.1", str(_free_port())
        t0 = time.time()
        try:
            proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                                    start_new_session=True)
            try:
                so, se = proc.communicate(timeout=args.extra_timeout)
            except subprocess.TimeoutExpired:
                import signal
                os.killpg(proc.pid, signal.SIGKILL)          # the process group this call started, nothing else
                proc.communicate()
                out[key] = {"unavailable": f"config {cfg}: no result within {args.extra_timeout} s"}
                continue
            line = next((l for l in reversed(so.splitlines()) if l.startswith("{") and l.rstrip().endswith("}")), None)
            if proc.returncode != 0 or line is None:
                err = (se or so).strip().splitlines()
                out[key] = {"unavailable": f"config {cfg}: exit code {proc.returncode}: " + " | ".join(err[-3:])[:300]}
                continue
            r = json.loads(line)
            out[key] = {k: r[k] for k in _KEEP if k in r}
            out[key]["wall_s"] = round(time.time() - t0, 1)
        except Exception as e:                                       # never lose the headline over an extra
            out[key] = {"unavailable": f"config {cfg}: {type(e).__name__}: {str(e)[:200]}"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-compile", type=int, default=1,
                    help="reference arm: pass --use_compile to the reference, as its launch scripts do (1, default; "
                         "falls back to eager if its compiler cannot run) or run it eagerly (0)")
    ap.add_argument("--min-timed-s", type=float, default=0.0,
                    help="raise --steps so that the timed region lasts at least this long (used for the extra "
                         "configurations, whose steps are short)")
    ap.add_argument("--config", default="B", choices=["B"] + sorted(CONFIGS),
                    help="B (default) is the headline configuration; see CONFIGS for the others")
    ap.add_argument("--moe-fallback", type=int, default=1,
                    help="reference arm, MoE configs: force its padded-bmm expert path (its grouped path only "
                         "type-checks for moe_intermediate_size == hidden_size)")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline configuration only: do not measure the MoE and Ulysses configurations afterwards")
    ap.add_argument("--extra-timeout", type=int, default=420, help="time limit of one extra configuration's job (s)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    _select_config(args.config, args.gpus)
    if args.impl == "reference":
        try:
            out = run_reference(args)
        except Exception as e:                                       # report, never crash the driver
            out = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"} \
                if int(os.environ.get("RANK", 0)) == 0 else None
    else:
        out = run_ours(args)
    if out is not None:
        if args.config == "B" and not args.no_extras and "unavailable" not in out:
            out.update(run_extras(args))
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
