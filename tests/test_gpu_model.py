"""The GPT on the GPU (bf16 kernels) against the same model on CPU (fp32 oracle path)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(device, dtype, **over):
    from train_large_model_from_scratch_b200.models import GPT
    from train_large_model_from_scratch_b200.models.modules.init import clear_init_cache
    from train_large_model_from_scratch_b200.training.config import ModelConfig
    clear_init_cache()
    kw = dict(num_layer=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=512, vocab_size=4096, block_size=512)
    kw.update(over)
    return GPT(ModelConfig(**kw), device=device, compute_dtype=dtype)


@pytest.mark.parametrize("heads", [(4, 2), (8, 2)])          # head dim 64, and 32 (the shipped 0.25B model's)
def test_dense_model_matches_cpu_oracle(heads):
    from train_large_model_from_scratch_b200.ops import native
    over = dict(num_attention_heads=heads[0], num_key_value_heads=heads[1])
    gpu = _build("cuda", torch.bfloat16, **over)
    cpu = _build("cpu", torch.float32, **over)
    cpu.dense_buf.params.copy_(gpu.dense_buf.params.float().cpu())       # same (bf16-rounded) weights
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, 4096, (2, 257), generator=g)
    x, y = data[:, :-1].contiguous(), data[:, 1:].contiguous()
    _, lg, _ = gpu(x.cuda(), y.cuda())
    lg.backward()
    _, lc, _ = cpu(x, y)
    lc.backward()
    native.raise_on_device_status()
    assert abs(lg.item() - lc.item()) < 2e-2, (lg.item(), lc.item())
    gg, gc = gpu.dense_buf.main_grad.cpu(), cpu.dense_buf.main_grad
    cos = torch.nn.functional.cosine_similarity(gg, gc, dim=0).item()
    assert cos > 0.995, cos
    for name, (off, n, _) in cpu.dense_buf.layout.items():
        a, b = gg[off:off + n], gc[off:off + n]
        c = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
        assert c > 0.98, (name, c)


def test_training_reduces_loss_on_fixed_batch():
    from train_large_model_from_scratch_b200.parallel.zero1.distributed_optimizer import FusedAdamW
    model = _build("cuda", torch.bfloat16)
    opt = FusedAdamW([model.dense_buf], lr=2e-3, weight_decay=0.0)
    data = torch.randint(0, 4096, (4, 129), generator=torch.Generator().manual_seed(1)).cuda()
    losses = []
    for _ in range(8):
        opt.zero_grad()
        _, loss, _ = model(data[:, :-1].contiguous(), data[:, 1:].contiguous())
        loss.backward()
        opt.step(grad_clip_value=1.0)
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.5, losses


def test_smoke_entry():
    import __graft_entry__
    __graft_entry__.smoke()


def test_moe_model_matches_cpu_oracle():
    from train_large_model_from_scratch_b200.ops import native
    kw = dict(use_moe=True, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=256)
    gpu = _build("cuda", torch.bfloat16, **kw)
    cpu = _build("cpu", torch.float32, **kw)
    cpu.dense_buf.params.copy_(gpu.dense_buf.params.float().cpu())
    cpu.expert_buf.params.copy_(gpu.expert_buf.params.float().cpu())
    data = torch.randint(0, 4096, (2, 257), generator=torch.Generator().manual_seed(3))
    x, y = data[:, :-1].contiguous(), data[:, 1:].contiguous()
    _, lg, _ = gpu(x.cuda(), y.cuda())
    lg.backward()
    _, lc, _ = cpu(x, y)
    lc.backward()
    native.raise_on_device_status()
    assert abs(lg.item() - lc.item()) < 3e-2, (lg.item(), lc.item())
    for a, b in ((gpu.dense_buf, cpu.dense_buf), (gpu.expert_buf, cpu.expert_buf)):
        cos = torch.nn.functional.cosine_similarity(a.main_grad.cpu(), b.main_grad, dim=0).item()
        assert cos > 0.98, cos


def test_lm_head_cross_entropy_is_chunk_invariant(monkeypatch):
    """The fused LM-head + cross-entropy gives the same loss and gradients in one chunk and in several."""
    from train_large_model_from_scratch_b200.ops import functional as Fo
    from train_large_model_from_scratch_b200.ops import native
    data = torch.randint(0, 4096, (2, 257), generator=torch.Generator().manual_seed(3))
    x, y = data[:, :-1].contiguous().cuda(), data[:, 1:].contiguous().cuda()
    out = []
    for chunk in (32768, 192):                       # 512 rows: one chunk, then three (the last one ragged)
        monkeypatch.setattr(Fo._LinearCrossEntropy, "CHUNK_ROWS", chunk)
        m = _build("cuda", torch.bfloat16)
        _, loss, _ = m(x, y)
        loss.backward()
        native.raise_on_device_status()
        out.append((loss.item(), m.dense_buf.main_grad.clone()))
    assert abs(out[0][0] - out[1][0]) < 1e-4, (out[0][0], out[1][0])
    cos = torch.nn.functional.cosine_similarity(out[0][1], out[1][1], dim=0).item()
    assert cos > 0.9999, cos
