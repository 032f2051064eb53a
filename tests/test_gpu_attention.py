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
