"""B200-native GPT pre-training stack (sm_100a kernels + NVLink peer-memory
collectives under a PyTorch front end)."""
__version__ = "0.1.0"
