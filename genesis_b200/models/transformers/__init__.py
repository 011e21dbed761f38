from .config import (TransformerConfig, MoEConfig, get_transformer_config, get_moe_config,
                     TRANSFORMER_PRETRAINED_CONFIG_ARCHIVE_MAP, MOE_PRETRAINED_CONFIG_ARCHIVE_MAP)
from .components import RotaryEmbedding, apply_rotary_pos_emb, apply_rope, rotate_half, find_multiple
from .dense import QwenModel, QwenForCausalLM, TransformerBlock, Attention, FeedForward, ModelArgs
from .moe import (MoEGate, MoEExpert, MoELayer, MoEAttention, MoEDecoderLayer, DenseFFN, MoEPreTrainedModel,
                  MoEModel, MoEForCausalLM, MoETransformerBlock, AddAuxiliaryLoss, GroupedExperts)
