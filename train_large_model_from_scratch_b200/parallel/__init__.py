from . import parallel_state
from .sequence_parallel.ulysses import ulysses_all_to_all, allreduce_non_expert_grads_across_sp
from .expert_parallel.comm import ep_all_to_all
from .zero1.distributed_optimizer import DistributedOptimizer, FusedAdamW, partition_tensors
