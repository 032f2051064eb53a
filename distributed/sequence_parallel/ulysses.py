from train_large_model_from_scratch_b200.parallel.sequence_parallel.ulysses import *  # noqa: F401,F403
from train_large_model_from_scratch_b200.parallel.sequence_parallel.ulysses import ulysses_all_to_all, allreduce_non_expert_grads_across_sp, head_plan, seq_to_head, head_to_seq
