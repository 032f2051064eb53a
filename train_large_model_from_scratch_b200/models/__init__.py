from .gpt import GPT, Block, EXPERT_LOCAL_PARAM_SUFFIXES
from .modules.emb import TextEmbedding, ImgEmbedding
from .modules.attn import Attention, rope_impl, gqa_impl
from .modules.mlp import MLP, MoE
from .modules.norm import LayerNorm
from .modules.loss import CrossEntropyLoss
