from train_large_model_from_scratch_b200.models.modules.loss import CrossEntropyLoss  # noqa: F401
