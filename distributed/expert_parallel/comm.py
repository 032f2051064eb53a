from train_large_model_from_scratch_b200.parallel.expert_parallel.comm import ep_all_to_all, exchange_counts  # noqa: F401
