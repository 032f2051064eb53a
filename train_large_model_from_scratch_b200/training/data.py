"""Datasets and loaders.

`MockDataset` reproduces the reference's mock data (`training/trainer.py:83-106`):
item `idx` is `seq_len + 1` int64 tokens uniform in `[0, vocab)`, inputs are
the first `seq_len`, labels the last `seq_len`. The reference seeds by index
only in `--deterministic` mode and otherwise draws from the per-rank global
RNG, which hands different sequences to the ranks of one SEP group; here the
index-seeded draw (`Generator().manual_seed(base_seed + offset + idx)`) is
always used, so every parallel layout sees identical tokens for the same
index.

`PackedTokenDataset` is the real-text pipeline of the reference's
`pretrain_example.py:30-74`: tokenise documents, append EOS, concatenate, cut
into `seq_len + 1` windows.
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch
from torch.utils.data import DataLoader, Dataset
from torch.utils.data.distributed import DistributedSampler

MOCK_VOCAB = 50304


class MockDataset(Dataset):
    def __init__(self, length: int, seq_len: int, vocab_size: int = MOCK_VOCAB, deterministic: bool = True,
                 base_seed: int = 0, seed_offset: int = 0):
        self.length, self.seq_len, self.vocab_size = length, seq_len, vocab_size
        self.deterministic = deterministic
        self.base_seed, self.seed_offset = int(base_seed), int(seed_offset)

    def __len__(self) -> int:
        return self.length

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        g = torch.Generator(device="cpu")
        g.manual_seed(self.base_seed + self.seed_offset + int(idx))
        data = torch.randint(0, self.vocab_size, (self.seq_len + 1,), dtype=torch.long, generator=g)
        return {"input_ids": data[:self.seq_len], "labels": data[1:self.seq_len + 1]}


class PackedTokenDataset(Dataset):
    """Documents -> one token stream (EOS after each document) -> fixed windows."""

    def __init__(self, texts: Iterable[str], tokenize: Callable[[str], list[int]], eos_token_id: int,
                 seq_len: int, max_samples: int | None = None, min_chars: int = 0):
        stream: list[int] = []
        window = seq_len + 1
        self.samples: list[torch.Tensor] = []
        for text in texts:
            if text is None or len(text) < min_chars:
                continue
            stream.extend(tokenize(text))
            stream.append(eos_token_id)
            while len(stream) >= window:
                self.samples.append(torch.tensor(stream[:window], dtype=torch.long))
                del stream[:window]
                if max_samples is not None and len(self.samples) >= max_samples:
                    break
            if max_samples is not None and len(self.samples) >= max_samples:
                break
        self.seq_len = seq_len

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        d = self.samples[idx]
        return {"input_ids": d[:-1], "labels": d[1:]}


def build_loader(dataset: Dataset, batch_size: int, dp_world_size: int, dp_rank: int, shuffle: bool,
                 num_workers: int = 0, pin_memory: bool = False, seed: int = 0):
    """DistributedSampler keyed by the DP rank (not the world rank), so all
    ranks of one SEP group read the same sequences (`trainer.py:114`)."""
    sampler = DistributedSampler(dataset, num_replicas=dp_world_size, rank=dp_rank, shuffle=shuffle, seed=seed)
    loader = DataLoader(dataset, batch_size=batch_size, sampler=sampler, num_workers=num_workers,
                        pin_memory=pin_memory and torch.cuda.is_available())
    return sampler, loader
