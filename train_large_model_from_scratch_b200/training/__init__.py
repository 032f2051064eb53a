from .arguments import build_parser, parse_args
from .config import (build_config, Config, TrainingConfig, LoggingConfig, SeedConfig, DataConfig,
                     OptimConfig, CheckpointConfig, ParallelConfig, ModelConfig)


def __getattr__(name):
    if name == "Trainer":                      # imported lazily: trainer pulls in models/parallel
        from .trainer import Trainer
        return Trainer
    raise AttributeError(name)


__all__ = ["build_parser", "parse_args", "build_config", "Trainer"]
