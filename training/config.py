from train_large_model_from_scratch_b200.training.config import *  # noqa: F401,F403
from train_large_model_from_scratch_b200.training.config import build_config, validate_static
