from train_large_model_from_scratch_b200.training.arguments import *  # noqa: F401,F403
from train_large_model_from_scratch_b200.training.arguments import build_parser, parse_args, add_all_arguments
