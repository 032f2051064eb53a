"""Per-kernel timing against the measured roofline.

    python -m benchmarks.kernels [--what gemm,mlp,attn,elementwise,moe,lmhead,experts] [--small] [--once]

Times each kernel with CUDA events on the launching stream after warm-up,
flushing L2 (a 256 MB write) between timed launches, and prints one JSON line
per case with achieved TFLOP/s or GB/s and, when a peaks file is named by the
`TLM_MEASURED_PEAKS` environment variable (JSON with `bf16_tflops`, `hbm_gbs`),
the fraction of the measured cuBLAS / copy peak. The
library GEMM (`torch.matmul`, cuBLAS) is timed on the same shapes for context.
`--once` launches every kernel a single time without timing (the workload for a
profiler capture).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from train_large_model_from_scratch_b200.ops import native


def _peaks():
    for p in (os.environ.get("TLM_MEASURED_PEAKS"),):
        if p and os.path.exists(p):
            with open(p) as f:
                return json.load(f)
    return {}


_FLUSH = None


_ONCE = False


def _time(fn, iters=10, warmup=3):
    global _FLUSH
    if _ONCE:
        fn()
        torch.cuda.synchronize()
        return 1.0, 1.0
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _FLUSH.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_gemm(small: bool):
    pk = _peaks().get("bf16_tflops")
    M = 4096 if small else 32768
    shapes = [("qkv_fwd", M, 2048, 1024), ("out_fwd", M, 1024, 1024), ("gate_up_fwd", M, 8192, 1024),
              ("down_fwd", M, 1024, 4096), ("lm_head_chunk", 4096, 50304, 1024)] + ([] if small else [("lm_head", 32768, 50304, 1024)])
    for name, m, n, k in shapes:
        x = torch.randn(m, k, device="cuda").bfloat16()
        w = torch.randn(n, k, device="cuda").bfloat16()
        dy = torch.randn(m, n, device="cuda").bfloat16()
        acc = torch.zeros(n, k, device="cuda")
        flops = 2.0 * m * n * k
        cases = [("nt", lambda: native.gemm_nt(x, w), lambda: x @ w.t()),
                 ("nn", lambda: native.gemm_nn(dy, w), lambda: dy @ w),
                 ("tn_acc", lambda: native.gemm_tn_accum(dy, x, acc), lambda: acc.addmm_(dy.t().float(), x.float()) if False else dy.t() @ x)]
        for kind, ours, lib in cases:
            med, best = _time(ours)
            lmed, _ = (1.0, 1.0) if _ONCE else _time(lib)
            rec = {"kernel": f"gemm_{kind}", "case": name, "M": m, "N": n, "K": k, "ms": round(med, 4),
                   "ms_best": round(best, 4), "tflops": round(flops / med / 1e9, 1), "cublas_ms": round(lmed, 4),
                   "cublas_tflops": round(flops / lmed / 1e9, 1)}
            if pk:
                rec["frac_of_measured_peak"] = round(flops / med / 1e9 / pk, 3)
            print(json.dumps(rec), flush=True)


def bench_mlp(small: bool):
    """The two MLP GEMMs that carry the SwiGLU math in their epilogue."""
    pk = _peaks().get("bf16_tflops")
    M, D, I = (4096 if small else 32768), 1024, 4096
    x = torch.randn(M, D, device="cuda").bfloat16()
    w_gu = (torch.randn(2 * I, D, device="cuda") * 0.02).bfloat16()
    w_down = (torch.randn(D, I, device="cuda") * 0.02).bfloat16()
    dy = torch.randn(M, D, device="cuda").bfloat16()
    gu, _ = native.gemm_swiglu(x, w_gu)
    for name, fn, flops in (("gemm_swiglu (gate|up GEMM + SwiGLU)", lambda: native.gemm_swiglu(x, w_gu), 2.0 * M * 2 * I * D),
                            ("gemm_swiglu_bwd (down dgrad + SwiGLU backward)", lambda: native.gemm_swiglu_bwd(dy, w_down, gu),
                             2.0 * M * I * D)):
        med, best = _time(fn)
        rec = {"kernel": name, "M": M, "D": D, "I": I, "ms": round(med, 4), "ms_best": round(best, 4),
               "tflops": round(flops / med / 1e9, 1)}
        if pk:
            rec["frac_of_measured_peak"] = round(flops / med / 1e9 / pk, 3)
        print(json.dumps(rec), flush=True)


def bench_elementwise(small: bool):
    bw = _peaks().get("hbm_gbs")
    rows, D, I = (4096 if small else 32768), 1024, 4096
    x = torch.randn(rows, D, device="cuda")
    delta = torch.randn(rows, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    gu = torch.randn(rows, 2 * I, device="cuda").bfloat16()
    dact = torch.randn(rows, I, device="cuda").bfloat16()
    mg = torch.zeros(D, device="cuda")
    x_new, h, rstd = native.add_rmsnorm_fwd(x, delta, w, 1e-6)
    cases = [
        ("add_rmsnorm_fwd", lambda: native.add_rmsnorm_fwd(x, delta, w, 1e-6), rows * D * (4 + 2 + 4 + 2)),
        ("add_rmsnorm_bwd", lambda: native.add_rmsnorm_bwd(x, delta, x_new, rstd, w, mg, True), rows * D * (4 + 2 + 4 + 4 + 2)),
        ("swiglu_fwd", lambda: native.swiglu_fwd(gu), rows * I * 6),
        ("swiglu_bwd", lambda: native.swiglu_bwd(dact, gu), rows * I * 10),
    ]
    n = 1 << 26
    p, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    sc = torch.ones((), device="cuda")
    cases.append(("adamw", lambda: native.adamw_step(p, m, v, g, out, sc, 3, 1e-4, 0.9, 0.95, 1e-8, 0.1), n * 30))
    cases.append(("sumsq", lambda: native.sumsq(g), n * 4))
    lg = torch.randn(2048 if small else 4096, 50304, device="cuda").bfloat16()
    tg = torch.randint(0, 50304, (lg.shape[0],), device="cuda")
    ls = torch.zeros((), device="cuda")
    cases.append(("ce_inplace", lambda: native.ce_fwd_bwd_inplace(lg, tg, sc, ls, -100, True), lg.numel() * 4))
    for name, fn, nbytes in cases:
        med, best = _time(fn)
        rec = {"kernel": name, "ms": round(med, 4), "ms_best": round(best, 4), "algorithmic_GB": round(nbytes / 1e9, 3),
               "GBps": round(nbytes / med / 1e6, 1)}
        if bw:
            rec["frac_of_measured_copy_bw"] = round(nbytes / med / 1e6 / bw, 3)
        print(json.dumps(rec), flush=True)


def bench_attn(small: bool):
    pk = _peaks().get("bf16_tflops")
    B, T, Hq, Hkv, hd = (1 if small else 8), 4096, 16, 8, int(os.environ.get("TLM_BENCH_HD", "64"))
    qkv = torch.randn(B, T, Hq + 2 * Hkv, hd, device="cuda").bfloat16()
    o, lse = native.flash_attn_fwd(qkv, Hq, Hkv, True)
    do = torch.randn_like(o)
    f_fwd = 4.0 * B * Hq * T * T * hd / 2
    for name, fn, fl in [("attn_fwd", lambda: native.flash_attn_fwd(qkv, Hq, Hkv, True), f_fwd),
                         ("attn_bwd", lambda: native.flash_attn_bwd(do, qkv, o, lse, Hq, Hkv, True), 2.5 * f_fwd)]:
        med, best = _time(fn)
        rec = {"kernel": name, "B": B, "T": T, "Hq": Hq, "Hkv": Hkv, "hd": hd, "ms": round(med, 4),
               "tflops_causal": round(fl / med / 1e9, 1)}
        if pk:
            rec["frac_of_measured_peak"] = round(fl / med / 1e9 / pk, 3)
        print(json.dumps(rec), flush=True)


def bench_lmhead(small: bool):
    """LM head without logits: statistics pass (GEMM + log-sum-exp epilogue + fold) and gradient-tile pass."""
    pk = _peaks().get("bf16_tflops")
    M, V, K = (2048 if small else 8192), 50304, 1024
    h = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(V, K, device="cuda") * 0.02).bfloat16()
    t = torch.randint(0, V, (M,), device="cuda")
    sc = torch.tensor(1.0 / M, device="cuda")
    _, lse = native.linear_cross_entropy_sum(h, w, t, -100, want_lse=True)
    out = torch.empty(M, V, device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * M * V * K
    for name, fn in (("lm_head loss, no logits (gemm EPI_LSE + lse_finish)", lambda: native.linear_cross_entropy_sum(h, w, t, -100)),
                     ("lm_head gradient tiles (gemm + softmax-minus-onehot epilogue)", lambda: native.gemm_dlogits(h, w, lse, t, sc, -100, out=out)),
                     ("lm_head logits (plain gemm_nt, for comparison)", lambda: native.gemm_nt(h, w, out=out))):
        med, best = _time(fn)
        rec = {"kernel": name, "M": M, "V": V, "K": K, "ms": round(med, 4), "tflops": round(fl / med / 1e9, 1)}
        if pk:
            rec["frac_of_measured_peak"] = round(fl / med / 1e9 / pk, 3)
        print(json.dumps(rec), flush=True)


def bench_experts(small: bool):
    """MoE expert MLP on expert-grouped rows: grouped gate|up GEMM with the SwiGLU epilogue, grouped down dgrad with the
    SwiGLU-backward epilogue (8 experts, uneven groups)."""
    pk = _peaks().get("bf16_tflops")
    E, D, I = 8, 1024, 2048
    R = 4096 if small else 32768
    base = R // E
    counts = [base + (i % 3 - 1) * (base // 4) for i in range(E)]
    counts[-1] += R - sum(counts)
    rs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    dc = native.DeviceCounts(rs, max(counts))
    x = torch.randn(R, D, device="cuda").bfloat16()
    dy = torch.randn(R, D, device="cuda").bfloat16()
    w_pair = (torch.randn(2 * E, I, D, device="cuda") * 0.02).bfloat16()
    w_down = (torch.randn(E, D, I, device="cuda") * 0.02).bfloat16()
    gu, act = native.grouped_gemm_swiglu(x, w_pair, dc)
    for name, fn, fl in (("grouped gate|up GEMM + SwiGLU epilogue", lambda: native.grouped_gemm_swiglu(x, w_pair, dc), 2.0 * R * 2 * I * D),
                         ("grouped gate|up GEMM, separate SwiGLU kernel", lambda: native.swiglu_fwd(native.grouped_gemm_pair_fwd(x, w_pair, dc)), 2.0 * R * 2 * I * D),
                         ("grouped down dgrad + SwiGLU-backward epilogue", lambda: native.grouped_gemm_swiglu_bwd(dy, w_down, gu, dc), 2.0 * R * I * D),
                         ("grouped down dgrad, separate SwiGLU-backward kernel", lambda: native.swiglu_bwd(native.grouped_gemm_nn(dy, w_down, dc), gu), 2.0 * R * I * D)):
        med, best = _time(fn)
        rec = {"kernel": name, "rows": R, "experts": E, "D": D, "I": I, "ms": round(med, 4), "tflops": round(fl / med / 1e9, 1)}
        if pk:
            rec["frac_of_measured_peak"] = round(fl / med / 1e9 / pk, 3)
        print(json.dumps(rec), flush=True)


def bench_moe(small: bool):
    """Routing, gather / combine and the head-scatter (QKV + RoPE) GEMM epilogue."""
    import ctypes
    from train_large_model_from_scratch_b200.ops import oracle
    bw = _peaks().get("hbm_gbs")
    M, E, k, D = (4096 if small else 32768), 8, 2, 1024
    logits = torch.randn(M, E, device="cuda").bfloat16()
    x = torch.randn(M, D, device="cuda").bfloat16()
    w, ex, counts, base, pos, order = native.moe_route(logits, k)
    y = torch.randn(M * k, D, device="cuda").bfloat16()
    cases = [("moe_route (3 kernels)", lambda: native.moe_route(logits, k), M * E * 2 + M * k * 16),
             ("moe_gather", lambda: native.moe_gather(x, order, k), M * k * D * 4),
             ("moe_combine", lambda: native.moe_combine(y, pos, w, M, k), M * k * D * 2 + M * D * 2),
             ("moe_pair_dot", lambda: native.moe_pair_dot(x, y, pos, k), M * k * D * 4)]
    for name, fn, nbytes in cases:
        med, best = _time(fn)
        rec = {"kernel": name, "ms": round(med, 4), "algorithmic_GB": round(nbytes / 1e9, 4), "GBps": round(nbytes / med / 1e6, 1)}
        if bw:
            rec["frac_of_measured_copy_bw"] = round(nbytes / med / 1e6 / bw, 3)
        print(json.dumps(rec), flush=True)
    B, T, Hq, Hkv, hd = (1 if small else 8), 4096, 16, 8, 64
    h = torch.randn(B * T, D, device="cuda").bfloat16()
    wq = (torch.randn((Hq + 2 * Hkv) * hd, D, device="cuda") * 0.02).bfloat16()
    cos, sin = oracle.rope_tables(torch.arange(T, device="cuda"), hd, 10000.0, "reference")
    cos, sin = cos.contiguous(), sin.contiguous()
    out = torch.empty(B, T, Hq + 2 * Hkv, hd, device="cuda", dtype=torch.bfloat16)
    dst = (ctypes.c_void_p * 1)(out.data_ptr())
    cs = native.rope_table_fp16(cos, sin)
    fn = lambda: native.gemm_heads(h, wq, False, dst, 1, B, T, T, Hq + 2 * Hkv, 0, Hq, Hkv, Hq, Hkv, hd, Hq + Hkv, cs)
    med, best = _time(fn)
    fl = 2.0 * B * T * D * (Hq + 2 * Hkv) * hd
    rec = {"kernel": "gemm_heads (QKV + RoPE epilogue)", "M": B * T, "N": (Hq + 2 * Hkv) * hd, "K": D, "ms": round(med, 4),
           "tflops": round(fl / med / 1e9, 1)}
    pk = _peaks().get("bf16_tflops")
    if pk:
        rec["frac_of_measured_peak"] = round(fl / med / 1e9 / pk, 3)
    print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,elementwise,attn")
    ap.add_argument("--small", action="store_true", help="reduced sizes (for profiler captures)")
    ap.add_argument("--once", action="store_true", help="launch each kernel once, no timing (profiler workload)")
    a = ap.parse_args()
    _ONCE = a.once
    torch.cuda.set_device(0)
    for w in a.what.split(","):
        {"gemm": bench_gemm, "mlp": bench_mlp, "elementwise": bench_elementwise, "attn": bench_attn, "moe": bench_moe,
         "lmhead": bench_lmhead, "experts": bench_experts}[w](a.small)
    native.raise_on_device_status()
