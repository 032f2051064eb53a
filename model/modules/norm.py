from train_large_model_from_scratch_b200.models.modules.norm import LayerNorm  # noqa: F401
