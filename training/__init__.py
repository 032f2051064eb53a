"""Import surface of the reference (`from training import parse_args, build_config, Trainer`);
the implementation lives in `train_large_model_from_scratch_b200.training`."""
from train_large_model_from_scratch_b200.training import build_parser, parse_args, build_config
from train_large_model_from_scratch_b200.training import config, arguments
from train_large_model_from_scratch_b200.training.trainer import Trainer

__all__ = ["build_parser", "parse_args", "build_config", "Trainer"]
