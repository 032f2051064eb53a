"""Child process: build the reference's GPT (unmodified sources, made to run on CPU by pointing
`torch.cuda.current_device` at the CPU) and this package's GPT with the same configuration, load the
reference's state dict into ours, and compare loss and gradients on one batch. Prints a JSON line."""
import json
import os
import sys

REF, ROOT, MODE = sys.argv[1], sys.argv[2], sys.argv[3]
sys.path[:] = [REF] + [p for p in sys.path if os.path.abspath(p or ".") not in (ROOT, REF)] + [ROOT]

import torch
import torch.distributed as dist

cpu = torch.device("cpu")
torch.cuda.current_device = lambda: cpu
_fork = torch.random.fork_rng
torch.random.fork_rng = lambda devices=None, **kw: _fork(devices=[], **kw)

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("MASTER_PORT", sys.argv[4])
dist.init_process_group("gloo", rank=0, world_size=1)

# ---- the reference (its own top-level packages: training / model / distributed)
from training.config import ModelConfig as RefModelConfig, ParallelConfig as RefParallelConfig
from distributed import parallel_state as ref_ps
ref_ps.initialize_model_parallel(RefParallelConfig(sep_size=1))
from model import GPT as RefGPT

moe = MODE == "moe"
kw = dict(block_size=64, vocab_size=512, num_layer=2, num_attention_heads=4, num_key_value_heads=2, hidden_size=64,
          intermediate_size=128, tied_lm_head=True, use_moe=moe, num_experts=4, num_experts_per_tok=2,
          moe_intermediate_size=64)          # the reference's grouped path needs moe_intermediate_size == hidden_size
ref = RefGPT(RefModelConfig(**kw))
if moe:
    for blk in ref.blocks:                   # x @ W^T semantics for every shape (its padded-bmm path)
        blk.mlp.grouped_gemm_supported = False

# ---- this package
from train_large_model_from_scratch_b200.models import GPT
from train_large_model_from_scratch_b200.parallel import parallel_state
from train_large_model_from_scratch_b200.parallel.zero1.distributed_optimizer import FusedAdamW
from train_large_model_from_scratch_b200.training import checkpoint as ckpt
from train_large_model_from_scratch_b200.training.config import ModelConfig, ParallelConfig
parallel_state.initialize_model_parallel(config=ParallelConfig(sep_size=1))
ours = GPT(ModelConfig(**kw), device="cpu", compute_dtype=torch.float32)
bufs = [ours.dense_buf] + ([ours.expert_buf] if ours.expert_buf is not None else [])
opt = FusedAdamW(bufs, lr=1e-3)

ref_state = ref.state_dict()
same_keys = list(ref_state.keys()) == list(ours.state_dict().keys())
init_equal = all(torch.equal(ref_state[k], ours.state_dict()[k].float()) for k in ref_state) if same_keys else False
# move the reference off its all-matrices-equal initial point so that the comparison is not degenerate
g = torch.Generator().manual_seed(5)
with torch.no_grad():
    for p in ref.parameters():
        p.add_(torch.randn(p.shape, generator=g) * 0.02)
ckpt.load_model_state_dict(ours, opt, ref.state_dict())

data = torch.randint(0, 512, (2, 65), generator=g)
x, y = data[:, :-1].contiguous(), data[:, 1:].contiguous()
_, loss_ref, log_ref = ref(x, y)
loss_ref.backward()
_, loss_ours, log_ours = ours(x, y)
loss_ours.backward()

worst = 0.0
for name, p in ref.named_parameters():
    q = dict(ours.named_parameters())[name]
    gr, go = p.grad, q.main_grad
    worst = max(worst, float((gr - go).abs().max() / gr.abs().max().clamp_min(1e-12)))
print(json.dumps({"same_keys": same_keys, "init_equal": init_equal, "loss_ref": float(loss_ref),
                  "loss_ours": float(loss_ours), "log_ref": float(log_ref), "log_ours": float(log_ours),
                  "worst_grad_rel": worst}))
dist.destroy_process_group()
