"""`genesis.nn.attention` import path of the reference (`nn/attention.py:409-532`): flash attention on tcgen05."""
from .functional import FusedAttention, fused_attention, scaled_dot_product_attention, flash_attention  # noqa: F401
