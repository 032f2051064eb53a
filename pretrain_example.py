"""Pre-training on real text: a `Trainer` subclass that overrides the dataset hook.

Same role as the reference's `pretrain_example.py:77-153`: stream documents,
tokenise, append EOS, pack into `seq_len + 1` token windows, train with the
unchanged step loop. Two sources are supported:

  * a Hugging Face dataset (streaming), when the `datasets` package and network
    access are available -- `DatasetConfig.hf_dataset`;
  * local text: every `*.txt` / `*.jsonl` (field `text`) file under
    `--dataset_path`.

The tokenizer is a Hugging Face tokenizer when it can be loaded, else a
byte-level tokenizer (256 byte ids + EOS) so that the pipeline runs offline.
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass

from training import Trainer, build_config, parse_args
from train_large_model_from_scratch_b200.training.data import PackedTokenDataset


@dataclass(frozen=True)
class DatasetConfig:
    hf_dataset: str = "HuggingFaceFW/fineweb-edu"
    hf_subset: str = "sample-10BT"
    tokenizer: str = "gpt2"
    text_field: str = "text"
    max_samples: int = 200_000
    min_chars: int = 50


class ByteTokenizer:
    """Offline stand-in: UTF-8 bytes as token ids, 256 = end of text."""
    eos_token_id = 256

    def __len__(self) -> int:
        return 257

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))


def load_tokenizer(name: str):
    try:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(name, local_files_only=not bool(os.environ.get("HF_HUB_ONLINE")))
        return tok
    except Exception:
        return ByteTokenizer()


def local_texts(path: str, field: str):
    for f in sorted(glob.glob(os.path.join(path, "**", "*"), recursive=True)):
        if f.endswith(".txt"):
            with open(f, encoding="utf-8", errors="ignore") as fh:
                yield fh.read()
        elif f.endswith(".jsonl"):
            with open(f, encoding="utf-8", errors="ignore") as fh:
                for line in fh:
                    line = line.strip()
                    if line:
                        yield json.loads(line).get(field, "")


def hf_texts(cfg: DatasetConfig):
    from datasets import load_dataset
    ds = load_dataset(cfg.hf_dataset, name=cfg.hf_subset, split="train", streaming=True)
    for row in ds:
        yield row[cfg.text_field]


class OurTrainer(Trainer):
    dataset_config = DatasetConfig()

    def _init_dataset(self, config):
        dc = self.dataset_config
        tok = load_tokenizer(dc.tokenizer)
        assert config.model.vocab_size >= len(tok), \
            f"vocab_size {config.model.vocab_size} is smaller than the tokenizer's {len(tok)}"
        path = config.data.dataset_path
        texts = local_texts(path, dc.text_field) if path and os.path.isdir(path) else hf_texts(dc)
        encode = (lambda s: tok.encode(s)) if isinstance(tok, ByteTokenizer) else \
            (lambda s: tok(s, add_special_tokens=False)["input_ids"])
        self.train_dataset = PackedTokenDataset(texts, encode, tok.eos_token_id, config.train.seq_len,
                                                max_samples=dc.max_samples, min_chars=dc.min_chars)
        if len(self.train_dataset) == 0:
            raise RuntimeError(f"no training windows could be built from {path or dc.hf_dataset}")
        self.val_dataset = None
        self._build_loaders(config)


def main():
    args = parse_args()
    config = build_config(args)
    assert not config.train.do_val, "this example has no validation split"
    OurTrainer(config).train()


if __name__ == "__main__":
    main()
