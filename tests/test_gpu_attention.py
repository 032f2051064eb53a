"""tcgen05 flash attention (forward / backward) against an fp32 PyTorch reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [(2, 256, 4, 2, 64), (1, 384, 2, 1, 128), (1, 1024, 2, 2, 64), (2, 128, 2, 2, 64), (1, 512, 4, 1, 128),
         (2, 320, 8, 2, 32), (1, 200, 4, 4, 32)]


def _ref(qkv, n_q, n_kv):
    from train_large_model_from_scratch_b200.ops import oracle
    q, k, v = qkv[:, :, :n_q], qkv[:, :, n_q:n_q + n_kv], qkv[:, :, n_q + n_kv:]
    return oracle.attention(q, k, v, causal=True)


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", CASES)
def test_flash_fwd(B, T, Hq, Hkv, hd):
    from train_large_model_from_scratch_b200.ops import native
    torch.manual_seed(0)
    qkv = torch.randn(B, T, Hq + 2 * Hkv, hd, device="cuda").to(torch.bfloat16)
    o, lse = native.flash_attn_fwd(qkv, Hq, Hkv, True)
    native.raise_on_device_status()
    ref = _ref(qkv, Hq, Hkv)
    err = (o.float() - ref).abs().max().item()
    assert err < 2e-2, err
    # logsumexp of the scaled scores
    q = qkv[:, :, :Hq].float().permute(0, 2, 1, 3)
    k = qkv[:, :, Hq:Hq + Hkv].float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    s = q @ k.transpose(-1, -2) / math.sqrt(hd)
    s = s.masked_fill(torch.ones(T, T, dtype=torch.bool, device="cuda").triu(1), float("-inf"))
    torch.testing.assert_close(lse, torch.logsumexp(s, -1), rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", CASES)
def test_flash_bwd(B, T, Hq, Hkv, hd):
    from train_large_model_from_scratch_b200.ops import native
    torch.manual_seed(1)
    qkv = torch.randn(B, T, Hq + 2 * Hkv, hd, device="cuda").to(torch.bfloat16)
    do = torch.randn(B, T, Hq, hd, device="cuda").to(torch.bfloat16)
    o, lse = native.flash_attn_fwd(qkv, Hq, Hkv, True)
    dqkv = native.flash_attn_bwd(do, qkv, o, lse, Hq, Hkv, True)
    native.raise_on_device_status()
    x = qkv.float().requires_grad_()
    _ref(x, Hq, Hkv).backward(do.float())
    for name, sl in (("dq", slice(0, Hq)), ("dk", slice(Hq, Hq + Hkv)), ("dv", slice(Hq + Hkv, None))):
        a, b = dqkv[:, :, sl].float(), x.grad[:, :, sl]
        rel = ((a - b).norm() / b.norm()).item()
        assert rel < 2e-2, (name, rel)


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", [(2, 256, 4, 2, 64), (1, 384, 2, 1, 128), (2, 320, 8, 2, 32), (1, 200, 4, 4, 64)])
@pytest.mark.parametrize("variant", ["reference", "standard"])
def test_flash_bwd_with_transposed_rope_on_the_way_out(B, T, Hq, Hkv, hd, variant):
    """`rope=(cos, sin)`: dQ and dK come back as gradients of the UN-rotated heads. Oracle: the fp32 autograd
    gradient of the rotated heads pushed through the transposed rotation in fp32."""
    from train_large_model_from_scratch_b200.ops import native, oracle
    torch.manual_seed(3)
    qkv = torch.randn(B, T, Hq + 2 * Hkv, hd, device="cuda").to(torch.bfloat16)
    do = torch.randn(B, T, Hq, hd, device="cuda").to(torch.bfloat16)
    cos, sin = oracle.rope_tables(torch.arange(T, device="cuda"), hd, 10000.0, variant)
    o, lse = native.flash_attn_fwd(qkv, Hq, Hkv, True)
    dqkv = native.flash_attn_bwd(do, qkv, o, lse, Hq, Hkv, True, rope=(cos.contiguous(), sin.contiguous()))
    native.raise_on_device_status()
    x = qkv.float().requires_grad_()
    _ref(x, Hq, Hkv).backward(do.float())
    ref = x.grad.clone()
    ref[:, :, :Hq + Hkv] = oracle.rope_bwd(x.grad[:, :, :Hq + Hkv], cos, sin)
    for name, sl in (("dq", slice(0, Hq)), ("dk", slice(Hq, Hq + Hkv)), ("dv", slice(Hq + Hkv, None))):
        a, b = dqkv[:, :, sl].float(), ref[:, :, sl]
        rel = ((a - b).norm() / b.norm()).item()
        assert rel < 2e-2, (name, rel)


def test_flash_fwd_bwd_at_the_headline_shape():
    """B = 8, T = 4096, 16 query / 8 KV heads of 64 (the benchmark's attention shape: 128 (batch, head) pairs,
    32 KV tiles): the kernels run on the whole batch, the fp32 oracle one batch entry at a time."""
    from train_large_model_from_scratch_b200.ops import native
    B, T, Hq, Hkv, hd = 8, 4096, 16, 8, 64
    torch.manual_seed(4)
    qkv = (torch.randn(B, T, Hq + 2 * Hkv, hd, device="cuda") * 0.7).to(torch.bfloat16)
    do = torch.randn(B, T, Hq, hd, device="cuda").to(torch.bfloat16)
    o, lse = native.flash_attn_fwd(qkv, Hq, Hkv, True)
    dqkv = native.flash_attn_bwd(do, qkv, o, lse, Hq, Hkv, True)
    native.raise_on_device_status()
    for b in (0, 3, 7):
        x = qkv[b:b + 1].float().requires_grad_()
        ref = _ref(x, Hq, Hkv)
        assert (o[b:b + 1].float() - ref).abs().max().item() < 2e-2
        ref.backward(do[b:b + 1].float())
        for name, sl in (("dq", slice(0, Hq)), ("dk", slice(Hq, Hq + Hkv)), ("dv", slice(Hq + Hkv, None))):
            a, g = dqkv[b:b + 1, :, sl].float(), x.grad[:, :, sl]
            rel = ((a - g).norm() / g.norm()).item()
            assert rel < 2e-2, (b, name, rel)
        del x, ref
        torch.cuda.empty_cache()


@pytest.mark.parametrize("group", ["1", "2", "5", "64"])
def test_results_do_not_depend_on_the_block_order(group, monkeypatch):
    """The grids are decoded heavy-first over groups of heads (`csrc/tile_order.h`); any group size, including one that
    leaves a smaller last group (3 x 2 query heads and 3 x 1 KV heads in groups of 2 and 5), must give the same tensors."""
    from train_large_model_from_scratch_b200.ops import native
    torch.manual_seed(5)
    B, T, Hq, Hkv, hd = 3, 640, 2, 1, 64
    qkv = torch.randn(B, T, Hq + 2 * Hkv, hd, device="cuda").to(torch.bfloat16)
    do = torch.randn(B, T, Hq, hd, device="cuda").to(torch.bfloat16)
    o0, lse0 = native.flash_attn_fwd(qkv, Hq, Hkv, True)
    d0 = native.flash_attn_bwd(do, qkv, o0, lse0, Hq, Hkv, True)
    monkeypatch.setenv("TLM_ATTN_FWD_GROUP", group)
    monkeypatch.setenv("TLM_ATTN_BWD_GROUP", group)
    o1, lse1 = native.flash_attn_fwd(qkv, Hq, Hkv, True)
    d1 = native.flash_attn_bwd(do, qkv, o1, lse1, Hq, Hkv, True)
    native.raise_on_device_status()
    assert torch.equal(o0, o1) and torch.equal(lse0, lse1)
    assert torch.equal(d0[:, :, Hq:], d1[:, :, Hq:])                       # dK, dV: one block each, fixed order
    rel = ((d0[:, :, :Hq].float() - d1[:, :, :Hq].float()).norm() / d0[:, :, :Hq].float().norm()).item()
    assert rel < 5e-3, rel                                                 # dQ: fp32 adds from several blocks, any order
    ref = _ref(qkv, Hq, Hkv)
    assert (o1.float() - ref).abs().max().item() < 2e-2
