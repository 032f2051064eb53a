from train_large_model_from_scratch_b200.parallel.parallel_state import *  # noqa: F401,F403
from train_large_model_from_scratch_b200.parallel import parallel_state as _ps
globals().update({k: getattr(_ps, k) for k in dir(_ps) if k.startswith(('get_', 'initialize_', 'destroy_', 'is_', 'group_'))})
