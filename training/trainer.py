from train_large_model_from_scratch_b200.training.trainer import Trainer  # noqa: F401
