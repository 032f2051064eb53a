from train_large_model_from_scratch_b200.models.modules.attn import Attention, rope_impl, gqa_impl  # noqa: F401
