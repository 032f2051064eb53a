from .training import get_training_info, set_seed, torch_version_ge, sm_ge, lr_schedule
from .model import (get_model_params, get_dense_model_params, get_moe_model_params,
                    get_compiled_to_uncompiled_mapping, count_exact_params, strip_compile_prefix)
from .profile import get_gpu_peak_flops, compute_mfu, get_measured_peak_flops, GPU_PEAK_FLOPS
from .health import Heartbeat, PeerFailure
