from train_large_model_from_scratch_b200.models.modules.mlp import MLP, MoE  # noqa: F401
