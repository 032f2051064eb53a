"""Mock data determinism and the packed-token pipeline (CPU)."""
import os
import subprocess
import sys
import tempfile

import torch

from train_large_model_from_scratch_b200.training.data import MockDataset, PackedTokenDataset, build_loader

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_mock_dataset_depends_only_on_index():
    a, b = MockDataset(10, 32, base_seed=7), MockDataset(10, 32, base_seed=7)
    assert torch.equal(a[3]["input_ids"], b[3]["input_ids"])
    assert torch.equal(a[3]["input_ids"][1:], a[3]["labels"][:-1])
    g = torch.Generator().manual_seed(7 + 3)
    assert torch.equal(a[3]["input_ids"], torch.randint(0, 50304, (33,), generator=g)[:32])
    assert not torch.equal(a[3]["input_ids"], a[4]["input_ids"])
    v = MockDataset(10, 32, base_seed=7, seed_offset=1_000_000_000)
    assert not torch.equal(a[3]["input_ids"], v[3]["input_ids"])
    assert int(MockDataset(4, 64, vocab_size=100)[0]["input_ids"].max()) < 100


def test_sampler_is_keyed_by_dp_rank():
    ds = MockDataset(16, 8)
    _, l0 = build_loader(ds, 2, 2, 0, True)
    _, l1 = build_loader(ds, 2, 2, 1, True)
    _, full = build_loader(ds, 4, 1, 0, True)
    b0, b1, bf = next(iter(l0)), next(iter(l1)), next(iter(full))
    got = torch.cat([b0["input_ids"], b1["input_ids"]])
    assert sorted(map(tuple, got.tolist())) == sorted(map(tuple, bf["input_ids"].tolist()))


def test_packed_token_dataset():
    texts = ["abcd", "x", "efghij"]
    ds = PackedTokenDataset(texts, lambda s: [ord(c) for c in s], eos_token_id=0, seq_len=4, min_chars=2)
    # stream: a b c d 0 e f g h i j 0 -> windows of 5
    assert len(ds) == 2
    assert ds[0]["input_ids"].tolist() == [97, 98, 99, 100] and ds[0]["labels"].tolist() == [98, 99, 100, 0]
    assert ds[1]["input_ids"].tolist() == [101, 102, 103, 104]
    assert len(PackedTokenDataset(texts * 10, lambda s: [1] * len(s), 0, 4, max_samples=3)) == 3


def test_example_entry_trains_on_local_text():
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "a.txt"), "w") as f:
        f.write("the quick brown fox jumps over the lazy dog. " * 400)
    log = tempfile.mkdtemp()
    cmd = [sys.executable, os.path.join(ROOT, "pretrain_example.py"), "--dataset_path", d, "--seq_len", "64",
           "--batch_size", "2", "--total_batch_size", "256", "--max_steps", "3", "--max_epochs", "1", "--warmup_steps", "1",
           "--num_layer", "1", "--hidden_size", "64", "--num_attention_heads", "2", "--num_key_value_heads", "1",
           "--intermediate_size", "128", "--vocab_size", "50304", "--tied_lm_head", "--sep_size", "1", "--backend", "gloo",
           "--precision", "fp32", "--debug", "--log_dir", log, "--max_lr", "1e-3"]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", HF_HUB_OFFLINE="1")
    cmd[cmd.index("--max_epochs") + 1] = "1"
    # max_steps and max_epochs must agree with the dataset size, so only give epochs
    i = cmd.index("--max_steps"); del cmd[i:i + 2]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    logs = [l for l in open(os.path.join(log, os.listdir(log)[0], "log.txt")).read().splitlines() if " train " in l]
    assert len(logs) >= 2 and float(logs[-1].split()[-1]) < float(logs[0].split()[-1])
