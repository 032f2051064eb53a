from train_large_model_from_scratch_b200.parallel.zero1.distributed_optimizer import DistributedOptimizer, FusedAdamW, partition_tensors  # noqa: F401
