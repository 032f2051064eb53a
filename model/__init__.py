"""Import surface of the reference's `model` package; see `train_large_model_from_scratch_b200.models`."""
from train_large_model_from_scratch_b200.models import (GPT, Block, TextEmbedding, ImgEmbedding, Attention, MLP, MoE, LayerNorm,
                       CrossEntropyLoss, EXPERT_LOCAL_PARAM_SUFFIXES)
