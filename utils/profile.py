from train_large_model_from_scratch_b200.utils.profile import *  # noqa: F401,F403
