"""sm_100a kernels against plain PyTorch fp32 references of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    from train_large_model_from_scratch_b200.ops import native
    native.lib()                      # a missing library is an error on a GPU machine
    yield native
    torch.cuda.synchronize()
    assert native.take_device_status() == 0


@pytest.fixture(params=["pairs", "single"])
def gemm_mode(request, nat):
    """Plain GEMMs run as CTA pairs (cta_group::2, the default) and as single CTAs: both forms must agree with the
    fp32 reference, on every operand layout and epilogue."""
    was = nat.set_gemm_pairs(2 if request.param == "pairs" else 0)     # 2: row-grouped GEMMs with small groups as well
    yield request.param
    nat.set_gemm_pairs(was)


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


GEMM_SHAPES = [(128, 256, 64), (256, 512, 256), (384, 768, 192), (200, 264, 72), (1000, 1096, 520),
               (4096, 2048, 1024), (64, 8, 1024)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nt(nat, gemm_mode, M, N, K):
    x, w = _rand(M, K, seed=1), _rand(N, K, seed=2)
    y = nat.gemm_nt(x, w)
    ref = x.float() @ w.float().t()
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert _rel_err(y, ref) < 6e-3


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nn(nat, gemm_mode, M, N, K):
    dy, w = _rand(M, N, seed=3), _rand(N, K, seed=4)
    dx = nat.gemm_nn(dy, w)
    ref = dy.float() @ w.float()
    assert _rel_err(dx, ref) < 6e-3


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_tn_accum(nat, gemm_mode, M, N, K):
    dy, x = _rand(M, N, seed=5), _rand(M, K, seed=6)
    acc = torch.ones(N, K, device="cuda")
    nat.gemm_tn_accum(dy, x, acc)
    ref = 1.0 + dy.float().t() @ x.float()
    assert _rel_err(acc, ref) < 1e-4
    nat.gemm_tn_accum(dy, x, acc)                       # accumulates
    assert _rel_err(acc, 2 * ref - 1.0) < 1e-4


@pytest.mark.parametrize("M,N,K", [(32768, 1024, 1024), (16384, 4096, 1024), (20000, 520, 264)])
def test_gemm_tn_accum_long_reductions(nat, gemm_mode, M, N, K):
    """Weight-gradient shapes: long reductions with few output tiles (split-K with atomic adds)."""
    dy, x = _rand(M, N, seed=25, scale=0.5), _rand(M, K, seed=26, scale=0.5)
    ref = 1.0 + dy.float().t() @ x.float()
    acc = torch.ones(N, K, device="cuda")
    nat.gemm_tn_accum(dy, x, acc)
    nat.raise_on_device_status()
    assert _rel_err(acc, ref) < 1e-4
    nat.gemm_tn_accum(dy, x, acc)                       # accumulates on top
    assert _rel_err(acc, 2 * ref - 1.0) < 1e-4


def test_gemm_strided_output_and_guard_rows(nat, gemm_mode):
    """Output written into a slice of a larger buffer must not touch its neighbours."""
    M, N, K = (200, 264, 72) if gemm_mode == "single" else (456, 264, 72)     # 456 rows: a pair tile with a ragged second half
    x, w = _rand(M, K, seed=7), _rand(N, K, seed=8)
    big = torch.full((M + 16, N + 24), 7.0, device="cuda", dtype=torch.bfloat16)
    out = big[8:8 + M, 8:8 + N]
    nat.gemm_raw(x, w, out, M, N, K, x.stride(0), w.stride(0), big.stride(0), 0, 0, 0)
    assert _rel_err(out, x.float() @ w.float().t()) < 6e-3
    mask = torch.ones_like(big, dtype=torch.bool)
    mask[8:8 + M, 8:8 + N] = False
    assert (big[mask] == 7.0).all()


def test_embedding(nat):
    w = _rand(1000, 256, seed=9)
    idx = torch.randint(0, 1000, (3, 50), device="cuda")
    out = nat.embedding_fwd(idx, w)
    torch.testing.assert_close(out, w[idx.reshape(-1)].float())
    dx = torch.randn(150, 256, device="cuda")
    g = torch.zeros(1000, 256, device="cuda")
    nat.embedding_bwd(idx, dx, g)
    ref = torch.zeros_like(g).index_add_(0, idx.reshape(-1), dx)
    torch.testing.assert_close(g, ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("rows,D,has_delta", [(37, 256, True), (64, 1024, True), (5, 3072, False), (130, 64, True), (9, 2048, True),
                                                (7, 1280, True), (11, 1536, False)])
def test_add_rmsnorm(nat, rows, D, has_delta):
    x = torch.randn(rows, D, device="cuda")
    delta = _rand(rows, D, seed=10) if has_delta else None
    w = (1.0 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
    x_new, h, rstd = nat.add_rmsnorm_fwd(x, delta, w, 1e-6)
    xr = x + (delta.float() if has_delta else 0.0)
    rr = torch.rsqrt(xr.pow(2).mean(-1) + 1e-6)
    torch.testing.assert_close(x_new, xr)
    torch.testing.assert_close(rstd, rr, rtol=1e-5, atol=1e-6)
    assert _rel_err(h, xr * rr[:, None] * w.float()) < 4e-3
    g_xnew = torch.randn(rows, D, device="cuda")
    g_h = _rand(rows, D, seed=11)
    mg = torch.zeros(D, device="cuda")
    g_x, g_delta = nat.add_rmsnorm_bwd(g_xnew, g_h, x_new, rstd, w, mg, has_delta)
    xhat = xr * rr[:, None]
    gxh = g_h.float() * w.float()
    ref = g_xnew + rr[:, None] * (gxh - xhat * (gxh * xhat).mean(-1, keepdim=True))
    torch.testing.assert_close(g_x, ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(mg, (g_h.float() * xhat).sum(0), rtol=1e-3, atol=1e-3)
    if has_delta:
        assert _rel_err(g_delta, ref) < 4e-3
    g_x2, _ = nat.add_rmsnorm_bwd(None, g_h, x_new, rstd, w, mg, False)
    torch.testing.assert_close(g_x2, ref - g_xnew, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("hd,variant", [(64, "reference"), (128, "standard"), (32, "reference")])
def test_rope(nat, hd, variant):
    from train_large_model_from_scratch_b200.ops import oracle
    B, T, Hq, Hkv = 2, 24, 4, 2
    qkv = _rand(B, T, Hq + 2 * Hkv, hd, seed=12)
    cos, sin = oracle.rope_tables(torch.arange(5, 5 + T, device="cuda"), hd, 10000.0, variant)
    ref = qkv.clone().float()
    ref[:, :, :Hq + Hkv] = oracle.rope(qkv[:, :, :Hq + Hkv], cos, sin)
    got = nat.rope_qk(qkv.clone(), cos.contiguous(), sin.contiguous(), Hq + Hkv, False)
    assert _rel_err(got, ref) < 4e-3
    torch.testing.assert_close(got[:, :, Hq + Hkv:], qkv[:, :, Hq + Hkv:])
    refb = qkv.clone().float()
    refb[:, :, :Hq + Hkv] = oracle.rope_bwd(qkv[:, :, :Hq + Hkv], cos, sin)
    gotb = nat.rope_qk(qkv.clone(), cos.contiguous(), sin.contiguous(), Hq + Hkv, True)
    assert _rel_err(gotb, refb) < 4e-3


@pytest.mark.parametrize("hd,Hq,Hkv,B,T,K", [(64, 4, 2, 2, 96, 192), (128, 2, 1, 1, 160, 256), (64, 16, 8, 1, 256, 1024),
                                              (64, 3, 1, 2, 32, 64), (32, 8, 2, 2, 96, 192), (32, 32, 4, 1, 256, 1024),
                                              (32, 3, 1, 1, 64, 64)])
def test_gemm_heads_rope_epilogue(nat, gemm_mode, hd, Hq, Hkv, B, T, K):
    """QKV projection whose epilogue rotates q/k heads and writes the packed tensor, against GEMM -> RoPE in fp32."""
    import ctypes
    from train_large_model_from_scratch_b200.ops import oracle
    Ht = Hq + 2 * Hkv
    x, w = _rand(B * T, K, seed=30), _rand(Ht * hd, K, scale=0.05, seed=31)
    cos, sin = oracle.rope_tables(torch.arange(7, 7 + T, device="cuda"), hd, 10000.0, "reference")
    cos, sin = cos.contiguous(), sin.contiguous()
    out = torch.full((B, T, Ht, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    dst = (ctypes.c_void_p * 1)(out.data_ptr())
    nat.gemm_heads(x, w, False, dst, 1, B, T, T, Ht, 0, Hq, Hkv, Hq, Hkv, hd, Hq + Hkv, nat.rope_table_fp16(cos, sin))
    ref = (x.float() @ w.float().t()).view(B, T, Ht, hd)
    ref[:, :, :Hq + Hkv] = oracle.rope(ref[:, :, :Hq + Hkv], cos, sin)
    assert torch.isfinite(out.float()).all()
    assert _rel_err(out, ref) < 6e-3
    assert _rel_err(out[:, :, Hq + Hkv:], ref[:, :, Hq + Hkv:]) < 6e-3


def test_gemm_heads_scatter_plan(nat, gemm_mode):
    """Two destinations (both local buffers here) with the Ulysses head plan and a row offset; MN-major weight."""
    import ctypes
    hd, Hq, B, T_l, sp, me = 64, 4, 2, 64, 2, 1
    q_l = Hq // sp
    dy, w = _rand(B * T_l, 192, seed=32), _rand(192, Hq * hd, scale=0.05, seed=33)     # dy @ w, w is [K, N]
    bufs = [torch.zeros(B, sp * T_l, q_l, hd, dtype=torch.bfloat16, device="cuda") for _ in range(sp)]
    dst = (ctypes.c_void_p * sp)(*[b.data_ptr() for b in bufs])
    nat.gemm_heads(dy, w, True, dst, sp, B, T_l, sp * T_l, q_l, me * T_l, Hq, 0, q_l, 1, hd, 0, None)
    ref = (dy.float() @ w.float()).view(B, T_l, Hq, hd)
    for r in range(sp):
        got = bufs[r][:, me * T_l:(me + 1) * T_l]
        assert _rel_err(got, ref[:, :, r * q_l:(r + 1) * q_l]) < 6e-3
        assert float(bufs[r][:, :me * T_l].abs().max()) == 0.0            # rows of the other source stay untouched


@pytest.mark.parametrize("hd", [64, 128])
def test_gemm_heads_replicates_kv_heads_to_their_owners(nat, gemm_mode, hd):
    """Fewer KV heads than destinations (8 query heads, 2 KV heads, 4 destinations, all local buffers here): q heads go to
    their owner, KV head j is stored to destinations 2 j and 2 j + 1 in the slots behind their q heads; no RoPE."""
    import ctypes
    Hq, Hkv, B, T_l, sp, me = 8, 2, 2, 128, 4, 2
    q_l, rep = Hq // sp, sp // Hkv
    x, w = _rand(B * T_l, 192, seed=35), _rand((Hq + 2 * Hkv) * hd, 192, scale=0.05, seed=36)
    bufs = [torch.zeros(B, sp * T_l, q_l + 2, hd, dtype=torch.bfloat16, device="cuda") for _ in range(sp)]
    dst = (ctypes.c_void_p * sp)(*[b.data_ptr() for b in bufs])
    nat.gemm_heads(x, w, False, dst, sp, B, T_l, sp * T_l, q_l + 2, me * T_l, Hq, Hkv, q_l, 1, hd, 0, None, rep)
    nat.raise_on_device_status()
    ref = (x.float() @ w.float().t()).view(B, T_l, Hq + 2 * Hkv, hd)
    for r in range(sp):
        got = bufs[r][:, me * T_l:(me + 1) * T_l]
        want = torch.cat([ref[:, :, r * q_l:(r + 1) * q_l], ref[:, :, Hq + r // rep:Hq + r // rep + 1],
                          ref[:, :, Hq + Hkv + r // rep:Hq + Hkv + r // rep + 1]], dim=2)
        assert _rel_err(got, want) < 6e-3, r
        assert float(bufs[r][:, :me * T_l].abs().max()) == 0.0


@pytest.mark.parametrize("M,I,K", [(200, 128, 64), (512, 384, 256), (4096, 1024, 512)])
def test_gemm_swiglu_epilogues(nat, gemm_mode, M, I, K):
    """gate|up GEMM that also emits act, and the down-projection dgrad that emits d(gate|up), against the
    separate GEMM and SwiGLU kernels' math in fp32."""
    x, w = _rand(M, K, seed=50), _rand(2 * I, K, scale=0.1, seed=51)
    gu, act = nat.gemm_swiglu(x, w)
    ref_gu = x.float() @ w.float().t()
    assert _rel_err(gu, ref_gu) < 6e-3
    g, u = gu.float().chunk(2, -1)                        # act is defined on the bf16-rounded gate / up
    assert _rel_err(act, torch.nn.functional.silu(g) * u) < 5e-3
    D = K
    dy, wd = _rand(M, D, seed=52), _rand(D, I, scale=0.1, seed=53)
    dgu = nat.gemm_swiglu_bwd(dy, wd, gu)
    dact = (dy.float() @ wd.float()).to(torch.bfloat16).float()
    sig = torch.sigmoid(g)
    ref = torch.cat([dact * u * sig * (1 + g * (1 - sig)), dact * g * sig], -1)
    assert _rel_err(dgu, ref) < 6e-3


def test_swiglu(nat):
    gu = _rand(77, 2 * 384, seed=13)
    act = nat.swiglu_fwd(gu)
    g, u = gu.float().chunk(2, -1)
    assert _rel_err(act, torch.nn.functional.silu(g) * u) < 4e-3
    dact = _rand(77, 384, seed=14)
    dgu = nat.swiglu_bwd(dact, gu)
    sig = torch.sigmoid(g)
    ref = torch.cat([dact.float() * u * sig * (1 + g * (1 - sig)), dact.float() * g * sig], -1)
    assert _rel_err(dgu, ref) < 4e-3


@pytest.mark.parametrize("V", [50304, 2048, 131072])      # the last one exceeds the row-resident kernel's shared memory
def test_ce_inplace(nat, V):
    rows = 33
    logits = _rand(rows, V, scale=2.0, seed=15)
    t = torch.randint(0, V, (rows,), device="cuda")
    t[3] = -100
    scale = torch.tensor(0.37, device="cuda")
    loss = torch.zeros((), device="cuda")
    work = logits.clone()
    nat.ce_fwd_bwd_inplace(work, t, scale, loss, -100, True)
    lf = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lf, t, ignore_index=-100, reduction="sum")
    (ref * 0.37).backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=1e-4, atol=1e-3)
    assert _rel_err(work, lf.grad) < 6e-3
    assert (work[3] == 0).all()
    loss2 = torch.zeros((), device="cuda")
    keep = logits.clone()
    nat.ce_fwd_bwd_inplace(keep, t, scale, loss2, -100, False)
    torch.testing.assert_close(keep, logits)
    torch.testing.assert_close(loss2, loss)


def test_sumsq(nat):
    for n in (1024, 1 << 20, (1 << 22) + 4):
        x = torch.randn(n, device="cuda")
        torch.testing.assert_close(nat.sumsq(x), x.double().pow(2).sum().float(), rtol=1e-5, atol=1e-3)


def test_adamw_matches_torch(nat):
    n = 1 << 16
    p = torch.randn(n, device="cuda")
    ref = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    scale = torch.tensor(0.5, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref.grad = g * 0.5
        opt.step()
        nat.adamw_step(p, m, v, g, out, scale, step, 1e-2, 0.9, 0.95, 1e-8, 0.1)
    torch.testing.assert_close(p, ref.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(out, p.to(torch.bfloat16))


@pytest.mark.parametrize("counts,N,K", [([130, 0, 64, 257], 512, 256), ([5, 300, 1, 90], 264, 72), ([0, 0, 128], 256, 64),
                                        ([700, 0, 1300, 257], 512, 256)])
def test_grouped_gemms(nat, gemm_mode, counts, N, K):
    R, E = sum(counts), len(counts)
    x, w = _rand(R, K, seed=20), _rand(E, N, K, seed=21)
    dy = _rand(R, N, seed=22)
    y = nat.grouped_gemm_nt(x, w, counts)
    dx = nat.grouped_gemm_nn(dy, w, counts)
    acc = torch.ones(E, N, K, device="cuda")
    nat.grouped_gemm_tn_accum(dy, x, acc, counts)
    r = 0
    for e, c in enumerate(counts):
        if c:
            assert _rel_err(y[r:r + c], x[r:r + c].float() @ w[e].float().t()) < 6e-3, ("nt", e)
            assert _rel_err(dx[r:r + c], dy[r:r + c].float() @ w[e].float()) < 6e-3, ("nn", e)
        ref = 1.0 + dy[r:r + c].float().t() @ x[r:r + c].float()
        assert _rel_err(acc[e], ref) < 1e-4, ("tn", e)
        r += c


@pytest.mark.parametrize("M,E,k", [(300, 8, 2), (129, 128, 8), (64, 4, 1), (1000, 40, 3)])
def test_moe_route_and_row_movement(nat, M, E, k):
    """Device routing (top-k, softmax of the winners, stable expert-major order) and the gather / combine /
    pair-dot kernels against torch."""
    D = 64
    g = torch.Generator(device="cuda").manual_seed(40)
    # distinct logits per row so that the top-k set is unambiguous
    logits = (torch.rand(M, E, device="cuda", generator=g).argsort(dim=1).float() * 0.125 - 2.0).to(torch.bfloat16)
    w, ex, counts, base, pos, order = nat.moe_route(logits, k)
    vals, ref_e = torch.topk(logits.float(), k, dim=-1)
    assert torch.equal(ex.long(), ref_e)
    torch.testing.assert_close(w, torch.softmax(vals, -1), rtol=1e-5, atol=1e-6)
    flat = ref_e.reshape(-1)
    ref_order = torch.sort(flat, stable=True).indices
    assert torch.equal(order.long(), ref_order)
    assert torch.equal(pos.long()[ref_order], torch.arange(M * k, device="cuda"))
    ref_counts = torch.bincount(flat, minlength=E)
    assert torch.equal(counts.long(), ref_counts)
    assert torch.equal(base.long(), torch.cat([ref_counts.new_zeros(1), ref_counts.cumsum(0)]))
    x = _rand(M, D, seed=41)
    rows = nat.moe_gather(x, order, k)
    assert torch.equal(rows, x[ref_order // k])
    y = _rand(M * k, D, seed=42)
    out = nat.moe_combine(y, pos, w, M, k)
    ref = (y.float()[pos.long()].view(M, k, D) * w[:, :, None]).sum(1)
    assert _rel_err(out, ref) < 4e-3
    d_out = _rand(M, D, seed=43)
    dw = nat.moe_pair_dot(d_out, y, pos, k)
    ref_dw = (d_out.float()[:, None, :] * y.float()[pos.long()].view(M, k, D)).sum(-1).reshape(-1)
    torch.testing.assert_close(dw, ref_dw, rtol=1e-4, atol=1e-3)
    scaled = nat.moe_gather(d_out, order, k, scale=w)
    assert _rel_err(scaled, d_out.float()[ref_order // k] * w.reshape(-1)[ref_order][:, None]) < 4e-3
    # gradient of softmax-over-top-k
    dwt = torch.randn(M, k, device="cuda", generator=g)
    dl = nat.moe_route_bwd(dwt, w, ex, M, E)
    lf = logits.float().requires_grad_()
    v2, e2 = torch.topk(lf, k, dim=-1)
    (torch.softmax(v2, -1) * dwt).sum().backward()
    assert _rel_err(dl, lf.grad) < 1e-2


def test_grouped_gemm_row_scatter_epilogue(nat, gemm_mode):
    """Grouped GEMM whose epilogue stores each output row at a looked-up (buffer, row): two local buffers
    stand in for two ranks; rows flagged -1 are dropped."""
    import ctypes
    E, N, K = 3, 256, 128
    counts = [70, 0, 130]
    R = sum(counts)
    x, w = _rand(R + 16, K, seed=44), _rand(E, N, K, scale=0.1, seed=45)      # 16 trailing rows belong to no expert
    rs = torch.tensor([0, 70, 70, 200], dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(46)
    perm = torch.randperm(R, device="cuda", generator=g)
    dest_rank = (perm % 2).to(torch.int32)
    dest_row = (perm // 2).to(torch.int64)
    dest_rank[5] = -1
    dest_rank = torch.cat([dest_rank, dest_rank.new_full((16,), -1)])
    dest_row = torch.cat([dest_row, dest_row.new_zeros(16)])
    bufs = [torch.zeros(R // 2, N, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    ptrs = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in bufs])
    nat.grouped_gemm_nt_scatter(x, w, nat.DeviceCounts(rs, R), dest_rank, dest_row, ptrs, 2, R // 2)
    ref = torch.zeros(2, R // 2, N, device="cuda")
    r = 0
    for e, c in enumerate(counts):
        for i in range(r, r + c):
            if int(dest_rank[i]) >= 0:
                ref[int(dest_rank[i]), int(dest_row[i])] = x[i].float() @ w[e].float().t()
        r += c
    for b in range(2):
        assert _rel_err(bufs[b], ref[b]) < 6e-3


def test_grouped_pair_gemms(nat, gemm_mode):
    """gate | up of all experts in one grouped GEMM, and the data gradient of both in one GEMM with K = 2 I."""
    E, I, D = 3, 256, 192
    counts = [70, 0, 130]
    R = sum(counts)
    x = _rand(R + 8, D, seed=60)
    w = _rand(2 * E, I, D, scale=0.1, seed=61)
    rs = torch.tensor([0, 70, 70, 200], dtype=torch.int32, device="cuda")
    dc = nat.DeviceCounts(rs, R)
    gu = nat.grouped_gemm_pair_fwd(x, w, dc)
    dgu = _rand(R + 8, 2 * I, seed=62)
    dx = nat.grouped_gemm_pair_dgrad(dgu, w, dc)
    r = 0
    for e, c in enumerate(counts):
        if c:
            xs = x[r:r + c].float()
            ref = torch.cat([xs @ w[e].float().t(), xs @ w[E + e].float().t()], -1)
            assert _rel_err(gu[r:r + c], ref) < 6e-3
            dref = dgu[r:r + c, :I].float() @ w[e].float() + dgu[r:r + c, I:].float() @ w[E + e].float()
            assert _rel_err(dx[r:r + c], dref) < 6e-3
        r += c
    # row-limited SwiGLU: rows past the device-side count stay untouched
    n = torch.tensor([150], dtype=torch.int64, device="cuda")
    act = nat.swiglu_fwd(gu[:R].contiguous(), n)
    g, u = gu[:150].float().chunk(2, -1)
    assert _rel_err(act[:150], torch.nn.functional.silu(g) * u) < 5e-3


def test_moe_plan_kernel_matches_table_arithmetic(nat):
    """The expert-parallel plan kernel against the same routes derived with torch ops from the count table,
    for every rank of an emulated group of 4 (the ranks are just four independent routings on this GPU)."""
    ep, E, k, M = 4, 8, 2, 96
    E_l = E // ep
    g = torch.Generator(device="cuda").manual_seed(70)
    routes = []
    for r in range(ep):
        logits = (torch.rand(M, E, device="cuda", generator=g).argsort(dim=1).float() * 0.25).to(torch.bfloat16)
        routes.append(nat.moe_route(logits, k))
    table = torch.stack([rt[2] for rt in routes]).to(torch.int32).contiguous()          # [ep, E]
    C = table.long()
    tot = C.sum(0)
    base = (torch.cumsum(tot.view(ep, E_l), 1) - tot.view(ep, E_l)).view(E)
    src_prefix = torch.cumsum(C, 0) - C
    start_on_src = torch.cumsum(C, 1) - C
    for me in range(ep):
        w, ex, counts, my_start, pos, order = routes[me]
        plan = nat.moe_plan(table, ep, me, ex, order, my_start)
        P = order.numel()
        sorted_e = ex.view(-1)[order.long()].long()
        i = torch.arange(P, device="cuda")
        assert torch.equal(plan["send_rank"].long(), sorted_e // E_l)
        assert torch.equal(plan["send_row"], base[sorted_e] + src_prefix[me][sorted_e] + (i - my_start.long()[sorted_e]))
        mine = slice(me * E_l, (me + 1) * E_l)
        n_recv = int(tot[mine].sum())
        assert int(plan["n_recv"]) == n_recv
        assert torch.equal(plan["row_start"].long(), torch.cat([base[mine], base[mine][-1:] + tot[mine][-1:]]))
        # every received row points back at the pair that was sent to it
        back_rank, back_row = plan["back_rank"].long(), plan["back_row"]
        assert bool((back_rank[n_recv:] == -1).all())
        for s in range(ep):
            ws, exs, cs, starts, poss, orders = routes[s]
            ps = nat.moe_plan(table, ep, s, exs, orders, starts)
            to_me = ps["send_rank"].long() == me
            rows = ps["send_row"][to_me]
            assert bool((back_rank[rows] == s).all())
            assert torch.equal(back_row[rows], torch.arange(orders.numel(), device="cuda")[to_me])


@pytest.mark.parametrize("counts,I,D", [([300, 0, 129, 511], 256, 256), ([128, 128], 512, 192), ([1, 700, 3, 64, 0, 0, 257, 33], 256, 512)])
def test_grouped_swiglu_epilogues(nat, gemm_mode, counts, I, D):
    """MoE expert gate|up GEMM with the SwiGLU epilogue and the down projection's data-gradient GEMM with the
    SwiGLU-backward epilogue, per expert group (groups that end inside a 128-row tile, empty groups), against fp32."""
    E, R = len(counts), sum(counts)
    pad = 40                                                     # rows behind the last group: never read, never written
    x = _rand(R + pad, D, seed=31)
    w_pair = _rand(2 * E, I, D, seed=32, scale=0.05)
    w_down = _rand(E, D, I, seed=33, scale=0.05)
    dy = _rand(R + pad, D, seed=34)
    rs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    dc = nat.DeviceCounts(rs, max(counts))
    gu, act = nat.grouped_gemm_swiglu(x, w_pair, dc)
    nat.raise_on_device_status()
    r = 0
    for e, c in enumerate(counts):
        xe = x[r:r + c].float()
        g, u = xe @ w_pair[e].float().t(), xe @ w_pair[E + e].float().t()
        if c:
            assert _rel_err(gu[r:r + c, :I], g) < 6e-3 and _rel_err(gu[r:r + c, I:], u) < 6e-3
            gb, ub = gu[r:r + c, :I].float(), gu[r:r + c, I:].float()
            assert _rel_err(act[r:r + c], torch.nn.functional.silu(gb) * ub) < 6e-3
        r += c
    # backward: d(gate_up) from dy, w_down and the saved gate_up
    dgu = nat.grouped_gemm_swiglu_bwd(dy, w_down, gu, dc)
    nat.raise_on_device_status()
    r = 0
    for e, c in enumerate(counts):
        if c:
            dact = (dy[r:r + c].float() @ w_down[e].float()).to(torch.bfloat16).float()
            g, u = gu[r:r + c, :I].float(), gu[r:r + c, I:].float()
            sig = torch.sigmoid(g)
            ref = torch.cat([dact * u * sig * (1 + g * (1 - sig)), dact * g * sig], -1)
            assert _rel_err(dgu[r:r + c], ref) < 8e-3
        r += c


@pytest.mark.parametrize("M,V,K", [(300, 50304, 256), (128, 2048, 128), (1000, 33000, 512)])
def test_lm_head_loss_without_logits(nat, gemm_mode, M, V, K):
    """Loss of the LM head from (max, sum-of-exp) statistics kept in the logits GEMM's epilogue, no logits in memory:
    against fp32 `log_softmax` of the bf16-rounded logits, with ignored rows, at the 50304 vocabulary (its last
    256-column tile is half empty)."""
    h, w = _rand(M, K, seed=41), _rand(V, K, seed=42, scale=0.3)
    t = torch.randint(0, V, (M,), device="cuda")
    t[::7] = -100
    t[5] = V - 1
    loss, lse = nat.linear_cross_entropy_sum(h, w, t, -100, want_lse=True)
    nat.raise_on_device_status()
    # the statistics are taken of the bf16-rounded logits; the GEMM that stores logits rounds the same accumulators
    # (a float reference GEMM sums in another order and lands on the other side of a bf16 rounding now and then)
    logits = nat.gemm_nt(h, w).float()
    assert _rel_err(logits, h.float() @ w.float().t()) < 6e-3
    ref = torch.nn.functional.cross_entropy(logits, t, ignore_index=-100, reduction="sum")
    torch.testing.assert_close(loss, ref, rtol=2e-4, atol=1e-2)
    torch.testing.assert_close(lse, torch.logsumexp(logits, -1), rtol=1e-4, atol=2e-3)
    # and through the differentiable op in no-grad mode (the evaluation path)
    from train_large_model_from_scratch_b200.ops import functional as F_ops
    with torch.no_grad():
        got = F_ops.linear_cross_entropy(h, w, t, torch.tensor(1.0, device="cuda"), -100)
    torch.testing.assert_close(got, ref, rtol=2e-4, atol=1e-2)


@pytest.mark.parametrize("M,V,K", [(300, 50304, 256), (520, 2048, 128)])
def test_lm_head_gradient_tiles_from_recomputed_logits(nat, gemm_mode, M, V, K):
    """Second pass of the LM head without logits: `scale * (softmax - onehot)` written by the logits GEMM's epilogue
    from the rows' log-sum-exp, against autograd of fp32 cross-entropy on the same bf16 logits."""
    h, w = _rand(M, K, seed=43), _rand(V, K, seed=44, scale=0.3)
    t = torch.randint(0, V, (M,), device="cuda")
    t[::5] = -100
    scale = torch.tensor(0.37, device="cuda")
    loss, lse = nat.linear_cross_entropy_sum(h, w, t, -100, want_lse=True)
    dl = nat.gemm_dlogits(h, w, lse, t, scale, -100)
    nat.raise_on_device_status()
    lf = nat.gemm_nt(h, w).float().requires_grad_()
    (torch.nn.functional.cross_entropy(lf, t, ignore_index=-100, reduction="sum") * 0.37).backward()
    assert _rel_err(dl, lf.grad) < 8e-3
    assert (dl[::5] == 0).all()


def test_lm_head_recompute_mode_matches_in_place_mode(nat, monkeypatch):
    from train_large_model_from_scratch_b200.ops import functional as F_ops
    M, V, K = 4096 + 512, 8192, 256
    h0, w0 = _rand(M, K, seed=45), _rand(V, K, seed=46, scale=0.2)
    t = torch.randint(0, V, (M,), device="cuda")
    t[::9] = -100
    out = {}
    for mode in ("inplace", "recompute"):
        monkeypatch.setenv("TLM_LM_HEAD", mode)
        h = h0.clone().requires_grad_()
        w = w0.clone().requires_grad_()
        w.main_grad = torch.zeros(V, K, device="cuda")
        gs = torch.tensor(1.0 / M, device="cuda")
        loss = F_ops.linear_cross_entropy(h, w, t, gs, -100) * gs
        loss.backward()
        nat.raise_on_device_status()
        out[mode] = (loss.detach().clone(), h.grad.clone(), w.main_grad.clone())
    torch.testing.assert_close(out["inplace"][0], out["recompute"][0], rtol=1e-4, atol=1e-4)
    assert _rel_err(out["recompute"][1], out["inplace"][1]) < 1e-2
    assert _rel_err(out["recompute"][2], out["inplace"][2]) < 1e-2
