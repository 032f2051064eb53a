"""Command-line surface. Same flags, defaults and groups as the reference's
`training/arguments.py:29-130`; a table drives the parser instead of one
function per group. Abbreviations are disabled like in the reference (`:18`).

Flags marked "(added)" do not exist in the reference; their defaults keep the
reference's behaviour.
"""
from __future__ import annotations

import argparse

# (group, [(flag, kwargs), ...])
_S = "store_true"
_FLAG_TABLE: list[tuple[str, list[tuple[str, dict]]]] = [
    ("logging", [
        ("--exp_name", dict(type=str, default="gpt")),
        ("--log_dir", dict(type=str, default="./log/")),
        ("--log_every", dict(type=int, default=10)),
        ("--print_config", dict(action=_S)),
    ]),
    ("reproducibility", [
        ("--seed", dict(type=int, default=1337)),
        ("--deterministic", dict(action=_S)),
    ]),
    ("data", [
        ("--dataset_path", dict(type=str, default="../data/fineweb-edu-sample-10BT/")),
        ("--use_mock_data", dict(action=_S)),
        ("--mock_data_num_samples", dict(type=int, default=1280)),
        ("--num_workers", dict(type=int, default=0)),
        ("--pin_memory", dict(action=_S)),
    ]),
    ("training", [
        ("--total_batch_size", dict(type=int, default=524288, help="global batch size in tokens")),
        ("--batch_size", dict(type=int, default=8, help="micro batch size per DP rank")),
        ("--seq_len", dict(type=int, default=4096, help="full sequence length")),
        ("--max_steps", dict(type=int, default=None)),
        ("--max_epochs", dict(type=int, default=1)),
        ("--do_val", dict(action=_S)),
        ("--val_every_steps", dict(type=int, default=250)),
        ("--split_rate", dict(type=float, default=None)),
        ("--grad_clip_value", dict(type=float, default=1.0)),
        ("--debug", dict(action=_S)),
        ("--precision", dict(type=str, default="bf16", choices=["bf16", "fp16", "fp32"])),
        ("--use_compile", dict(action=_S, help="capture the micro-step in a CUDA graph where possible; never routes ops to a tracing compiler")),
        ("--use_profiler", dict(action=_S)),
        ("--steps_to_profile", dict(type=int, nargs="+", default=[15, 20])),
    ]),
    ("optimizer", [
        ("--max_lr", dict(type=float, default=4e-3)),
        ("--min_lr", dict(type=float, default=3e-5)),
        ("--warmup_steps", dict(type=int, default=1000)),
        ("--weight_decay", dict(type=float, default=0.1)),
        ("--adam_beta1", dict(type=float, default=0.9)),
        ("--adam_beta2", dict(type=float, default=0.95)),
        ("--adam_eps", dict(type=float, default=1e-8)),
    ]),
    ("checkpoint", [
        ("--do_save", dict(action=_S)),
        ("--save_every_steps", dict(type=int, default=5000)),
        ("--resume_path", dict(type=str, default=None, help="checkpoint directory")),
    ]),
    ("distributed", [
        ("--backend", dict(type=str, default="nccl")),
        ("--init_method", dict(type=str, default="env://")),
        ("--sep_size", dict(type=int, default=8, help="size of the joint SP/EP group")),
        ("--ddp_find_unused_parameters", dict(action=_S)),
        ("--ddp_gradient_as_bucket_view", dict(action=_S)),
        ("--use_distributed_optimizer", dict(action=_S, help="ZeRO-1 optimizer-state sharding")),
        ("--grad_wire_dtype", dict(type=str, default="fp32", choices=["bf16", "fp32"], help="(added) dtype of gradients on the wire")),
        ("--heartbeat_timeout_s", dict(type=float, default=0.0, help="(added) > 0: ranks exchange heartbeats between steps; a rank silent for this long fails the job")),
        ("--dist_timeout_s", dict(type=float, default=1800.0, help="(added) process-group timeout for collectives")),
    ]),
    ("model", [
        ("--block_size", dict(type=int, default=4096)),
        ("--vocab_size", dict(type=int, default=50304)),
        ("--num_layer", dict(type=int, default=32)),
        ("--num_attention_heads", dict(type=int, default=128)),
        ("--num_key_value_heads", dict(type=int, default=8)),
        ("--hidden_size", dict(type=int, default=1024)),
        ("--intermediate_size", dict(type=int, default=4096)),
        ("--dropout", dict(type=float, default=0.0)),
        ("--init_std", dict(type=float, default=0.013)),
        ("--tied_lm_head", dict(action=_S)),
        ("--use_moe", dict(action=_S)),
        ("--num_experts", dict(type=int, default=128)),
        ("--num_experts_per_tok", dict(type=int, default=8)),
        ("--moe_intermediate_size", dict(type=int, default=256)),
        ("--moe_aux_loss_coef", dict(type=float, default=0.0, help="(added) load-balance loss weight")),
        ("--moe_capacity_factor", dict(type=float, default=0.0, help="(added) 0 = dropless")),
        ("--rope_variant", dict(type=str, default="reference", choices=["reference", "standard"], help="(added)")),
    ]),
]


def add_all_arguments(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    for group_name, flags in _FLAG_TABLE:
        group = parser.add_argument_group(group_name)
        for flag, kwargs in flags:
            group.add_argument(flag, **kwargs)
    return parser


def build_parser() -> argparse.ArgumentParser:
    return add_all_arguments(argparse.ArgumentParser("pretrain", allow_abbrev=False))


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    return build_parser().parse_args(argv)
