"""Analytic parameter counts and checkpoint-key helpers.

`get_dense_model_params` restates the reference's `utils/model.py:24-60`
(`V*H + L*(4H^2 + 3HI)`, i.e. it ignores GQA and norm weights). For MoE the
reference's estimate adds a dense FFN that MoE blocks do not have
(`utils/model.py:101`); `get_moe_model_params` here counts what the model
builds and reports total and activated parameters. `count_exact_params` gives
the exact number for any ModelConfig.
"""
from __future__ import annotations

from ..training.config import ModelConfig


def get_dense_model_params(num_layer: int, hidden_size: int, intermediate_size: int, vocab_size: int) -> dict:
    total = vocab_size * hidden_size + num_layer * (4 * hidden_size ** 2 + 3 * hidden_size * intermediate_size)
    return {"total_params_B": total / 1e9, "dense_params_B": total / 1e9}


def get_moe_model_params(num_layer: int, hidden_size: int, intermediate_size: int, vocab_size: int,
                         num_expert: int, top_k: int, moe_intermediate_size: int) -> dict:
    H, L = hidden_size, num_layer
    attn = 4 * H * H
    router = H * num_expert
    expert = 3 * H * moe_intermediate_size
    total = vocab_size * H + L * (attn + router + num_expert * expert)
    active = vocab_size * H + L * (attn + router + top_k * expert)
    return {
        "total_params_B": total / 1e9,
        "activated_params_B": active / 1e9,
        "expert_params_B": L * num_expert * expert / 1e9,
    }


def get_model_params(model_config: ModelConfig) -> dict:
    c = model_config
    if c.use_moe:
        return get_moe_model_params(c.num_layer, c.hidden_size, c.intermediate_size, c.vocab_size,
                                    c.num_experts, c.num_experts_per_tok, c.moe_intermediate_size)
    return get_dense_model_params(c.num_layer, c.hidden_size, c.intermediate_size, c.vocab_size)


def count_exact_params(c: ModelConfig, ep_size: int = 1) -> int:
    """Exact number of parameters held by one rank (experts divided by `ep_size`)."""
    H, hd = c.hidden_size, c.hidden_size // c.num_attention_heads
    attn = H * c.num_attention_heads * hd + 2 * H * c.num_key_value_heads * hd + H * H
    if c.use_moe:
        ffn = H * c.num_experts + (c.num_experts // ep_size) * 3 * H * c.moe_intermediate_size
    else:
        ffn = 3 * H * c.intermediate_size
    total = c.vocab_size * H + c.num_layer * (attn + ffn + 2 * H) + H
    if not c.tied_lm_head:
        total += c.vocab_size * H
    return total


_COMPILE_PREFIX = "_orig_mod."


def get_compiled_to_uncompiled_mapping(state_dict_keys) -> dict[str, str]:
    """Map checkpoint keys written from a `torch.compile`d module (every key
    carries `_orig_mod.` somewhere in its path) to plain module keys
    (reference helper: `utils/model.py:132-178`)."""
    return {k: k.replace(_COMPILE_PREFIX, "") for k in state_dict_keys}


def strip_compile_prefix(state_dict: dict) -> dict:
    return {k.replace(_COMPILE_PREFIX, ""): v for k, v in state_dict.items()}
