"""Import surface of the reference's `utils` package; see `train_large_model_from_scratch_b200.utils`."""
from train_large_model_from_scratch_b200.utils import (get_training_info, set_seed, torch_version_ge, sm_ge, get_model_params,
                      get_compiled_to_uncompiled_mapping, get_gpu_peak_flops, compute_mfu)
