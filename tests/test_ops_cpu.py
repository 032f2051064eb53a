"""Each hand-written backward against torch autograd of the oracle math (CPU, fp32/fp64)."""
import math

import pytest
import torch

from train_large_model_from_scratch_b200.ops import functional as Fo
from train_large_model_from_scratch_b200.ops import oracle, moe_ops


def _param(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    p = torch.randn(*shape, generator=g, dtype=torch.float64).requires_grad_()
    p.main_grad = torch.zeros(shape, dtype=torch.float32)
    return p


def test_embedding_grad():
    w = _param(50, 8)
    idx = torch.tensor([[1, 3, 3], [7, 1, 0]])
    x = Fo.embedding(idx, w)
    assert x.dtype == torch.float32 and x.shape == (6, 8)
    g = torch.randn(6, 8)
    x.backward(g)
    ref = torch.zeros(50, 8).index_add_(0, idx.reshape(-1), g)
    torch.testing.assert_close(w.main_grad, ref)


def test_add_rmsnorm_matches_autograd():
    torch.manual_seed(0)
    x = torch.randn(5, 16, requires_grad=True)
    d = torch.randn(5, 16, requires_grad=True)
    w = _param(16).float().detach().requires_grad_()
    w.main_grad = torch.zeros(16)
    xn, h = Fo.add_rmsnorm(x, d, w, 1e-6)
    gx, gh = torch.randn(5, 16), torch.randn(5, 16)
    (xn * gx).sum().add((h * gh).sum()).backward()
    x2, d2, w2 = (t.detach().clone().requires_grad_() for t in (x, d, w))
    xn2 = x2 + d2
    h2 = oracle.rmsnorm(xn2, w2)
    (xn2 * gx).sum().add((h2 * gh).sum()).backward()
    torch.testing.assert_close(xn, xn2)
    torch.testing.assert_close(h, h2)
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(d.grad, d2.grad, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(w.main_grad, w2.grad, rtol=1e-5, atol=1e-5)


def test_linear_accumulates_main_grad():
    x = torch.randn(7, 12, requires_grad=True)
    w = _param(5, 12).float().detach().requires_grad_()
    w.main_grad = torch.ones(5, 12)
    y = Fo.linear(x, w)
    g = torch.randn(7, 5)
    y.backward(g)
    torch.testing.assert_close(y, x @ w.t())
    torch.testing.assert_close(x.grad, g @ w.detach())
    torch.testing.assert_close(w.main_grad, 1.0 + g.t() @ x.detach())
    assert w.grad is None


@pytest.mark.parametrize("variant", ["reference", "standard"])
def test_rope_matches_reference_formula_and_grad(variant):
    B, T, H, hd = 2, 6, 3, 8
    qkv = torch.randn(B, T, H + 2, hd, dtype=torch.float64, requires_grad=True)
    pos = torch.arange(3, 3 + T)
    cos, sin = oracle.rope_tables(pos, hd, 10000.0, variant)
    out = Fo.rope_qk(qkv, cos.double(), sin.double(), H + 1)
    # restate the reference's construction directly (model/modules/attn.py:20,47-66)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    fr = torch.outer(pos.float(), inv)
    if variant == "reference":
        c = torch.stack([fr.cos(), fr.cos()], -1).flatten(-2)
        s = torch.stack([fr.sin(), fr.sin()], -1).flatten(-2)
    else:
        c, s = torch.cat([fr.cos()] * 2, -1), torch.cat([fr.sin()] * 2, -1)
    x = qkv[:, :, :H + 1].detach()
    rot = torch.cat((-x[..., hd // 2:], x[..., :hd // 2]), -1)
    expect = x * c[None, :, None].double() + rot * s[None, :, None].double()
    torch.testing.assert_close(out[:, :, :H + 1], expect)
    torch.testing.assert_close(out[:, :, H + 1:], qkv[:, :, H + 1:])
    g = torch.randn_like(out)
    out.backward(g)
    q2 = qkv.detach().clone().requires_grad_()
    o2 = torch.cat([q2[:, :, :H + 1] * cos[None, :, None].double()
                    + oracle.rotate_half(q2[:, :, :H + 1]) * sin[None, :, None].double(),
                    q2[:, :, H + 1:]], 2)
    o2.backward(g)
    torch.testing.assert_close(qkv.grad, q2.grad, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("hq,hkv", [(4, 4), (4, 2), (4, 1)])
def test_attention_fwd_bwd(hq, hkv):
    B, T, hd = 2, 9, 8
    qkv = torch.randn(B, T, hq + 2 * hkv, hd, dtype=torch.float64, requires_grad=True)
    o = Fo.attention_packed(qkv, hq, hkv, True)
    g = torch.randn_like(o)
    o.backward(g)
    q2 = qkv.detach().clone().requires_grad_()
    q, k, v = q2[:, :, :hq], q2[:, :, hq:hq + hkv], q2[:, :, hq + hkv:]
    rep = hq // hkv
    sd = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(rep, 1), v.transpose(1, 2).repeat_interleave(rep, 1),
        is_causal=True).transpose(1, 2)
    sd.backward(g)
    torch.testing.assert_close(o, sd.to(o.dtype), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(qkv.grad, q2.grad, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(o.float(), oracle.attention(q.detach(), k.detach(), v.detach()).float(), rtol=1e-5, atol=1e-5)


def test_swiglu_grad():
    gu = torch.randn(6, 10, dtype=torch.float64, requires_grad=True)
    a = Fo.swiglu(gu)
    g = torch.randn_like(a)
    a.backward(g)
    g2 = gu.detach().clone().requires_grad_()
    gate, up = g2.chunk(2, -1)
    (torch.nn.functional.silu(gate) * up).backward(g)
    torch.testing.assert_close(gu.grad, g2.grad)


@pytest.mark.parametrize("chunk", [4096, 3])
def test_linear_cross_entropy(chunk, monkeypatch):
    monkeypatch.setattr(Fo._LinearCrossEntropy, "CHUNK_ROWS", chunk)
    monkeypatch.setattr(Fo._LinearCrossEntropy, "CHUNK_ROWS_CPU", chunk)
    M, D, V = 10, 16, 37
    h = torch.randn(M, D, requires_grad=True)
    w = _param(V, D).float().detach().requires_grad_()
    w.main_grad = torch.zeros(V, D)
    t = torch.randint(0, V, (M,))
    t[2] = -100
    scale = torch.tensor(0.25 / 9)
    s = Fo.linear_cross_entropy(h, w, t, scale)
    (s * scale).backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    s2 = torch.nn.functional.cross_entropy(h2 @ w2.t(), t, ignore_index=-100, reduction="sum")
    (s2 * scale).backward()
    torch.testing.assert_close(s, s2, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(h.grad, h2.grad, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(w.main_grad, w2.grad, rtol=1e-5, atol=1e-6)


def test_moe_local_matches_oracle_and_grads():
    torch.manual_seed(1)
    M, D, I, E, k = 24, 16, 12, 4, 2
    x = torch.randn(M, D, requires_grad=True)
    wr = torch.randn(E, D) * 0.5
    wg, wu, wd = (torch.randn(E, I, D) * 0.2).requires_grad_(), (torch.randn(E, I, D) * 0.2).requires_grad_(), \
        (torch.randn(E, D, I) * 0.2).requires_grad_()
    for w in (wg, wu, wd):
        w.main_grad = torch.zeros_like(w)
    logits = (x @ wr.t())
    out, aux = moe_ops.moe_forward(x, logits, wg, wu, wd, k, E, None, 1)
    g = torch.randn_like(out)
    out.backward(g)
    x2 = x.detach().clone().requires_grad_()
    w2 = [w.detach().clone().requires_grad_() for w in (wg, wu, wd)]
    ref = oracle.moe(x2, wr, *w2, k)
    ref.backward(g)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-4, atol=1e-5)
    for a, b in zip((wg, wu, wd), w2):
        torch.testing.assert_close(a.main_grad, b.grad, rtol=1e-4, atol=1e-5)
    assert aux is None


def test_moe_capacity_drops_and_aux():
    torch.manual_seed(2)
    M, D, I, E, k = 32, 8, 8, 4, 2
    x = torch.randn(M, D)
    logits = torch.randn(M, E)
    ws = [torch.randn(E, I, D), torch.randn(E, I, D), torch.randn(E, D, I)]
    for w in ws:
        w.main_grad = torch.zeros_like(w)
    full, aux = moe_ops.moe_forward(x, logits, *ws, k, E, None, 1, aux_coef=0.01)
    capped, _ = moe_ops.moe_forward(x, logits, *ws, k, E, None, 1, capacity_factor=0.5)
    assert aux is not None and aux.item() > 0
    assert not torch.allclose(full, capped)
    big, _ = moe_ops.moe_forward(x, logits, *ws, k, E, None, 1, capacity_factor=100.0)
    torch.testing.assert_close(full, big)


def test_regroup_index():
    idx = moe_ops._regroup_index([[2, 1], [0, 3]], "cpu")        # rows: s0e0,s0e0,s0e1,s1e1,s1e1,s1e1
    assert idx.tolist() == [0, 1, 2, 3, 4, 5]
    idx = moe_ops._regroup_index([[1, 2], [2, 1]], "cpu")        # s0: e0,e1,e1 ; s1: e0,e0,e1
    assert idx.tolist() == [0, 3, 4, 1, 2, 5]


def test_adamw_matches_torch():
    p = torch.randn(100)
    ref = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(100), torch.zeros(100)
    for step in range(1, 4):
        g = torch.randn(100)
        ref.grad = g.clone()
        opt.step()
        oracle.adamw_step(p, g, m, v, step, 1e-2, 0.9, 0.95, 1e-8, 0.1)
    torch.testing.assert_close(p, ref.detach(), rtol=1e-5, atol=1e-6)


def test_attention_dropout_trains_and_is_off_in_eval():
    """`--dropout > 0` (reference: attn.py:159): active in training mode only, and the step still back-propagates."""
    import warnings

    from train_large_model_from_scratch_b200.models import GPT
    from train_large_model_from_scratch_b200.training.config import ModelConfig

    def build(p):
        cfg = ModelConfig(block_size=32, vocab_size=128, num_layer=2, num_attention_heads=4, num_key_value_heads=2,
                          hidden_size=64, intermediate_size=128, dropout=p)
        return GPT(cfg, device="cpu")

    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, 128, (2, 32), generator=g)
    tgt = torch.randint(0, 128, (2, 32), generator=g)
    plain, drop = build(0.0), build(0.5)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        drop.train()
        torch.manual_seed(0)
        _, loss_d, _ = drop(idx, tgt)
        _, loss_p, _ = plain(idx, tgt)
        assert torch.isfinite(loss_d) and abs(float(loss_d) - float(loss_p)) > 1e-6
        loss_d.backward()
        grads = [p.main_grad if hasattr(p, "main_grad") else p.grad for p in drop.parameters()]
        assert any(gr is not None and float(gr.abs().sum()) > 0 for gr in grads)
        drop.eval()
        with torch.no_grad():
            _, loss_e, _ = drop(idx, tgt)
            plain.eval()
            _, loss_pe, _ = plain(idx, tgt)
        assert abs(float(loss_e) - float(loss_pe)) < 1e-6
