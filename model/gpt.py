from train_large_model_from_scratch_b200.models.gpt import GPT, Block, EXPERT_LOCAL_PARAM_SUFFIXES  # noqa: F401
