"""Model configurations. Parity: reference `genesis/models/transformers/config.py:12-372`
(field names, defaults, validation messages, presets), plus the Qwen2.5 / Qwen3-MoE shapes
the benchmarks use."""
from dataclasses import dataclass, fields
from typing import Any, Dict, Optional


@dataclass
class TransformerConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    max_position_embeddings: int = 4096
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    norm_eps: float = 1e-6
    use_cache: bool = True
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    initializer_range: float = 0.02

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        self._validate_config()

    def _validate_config(self):
        if self.hidden_size % self.num_attention_heads != 0:
            raise ValueError(f"hidden_size ({self.hidden_size}) must be divisible by "
                             f"num_attention_heads ({self.num_attention_heads})")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ValueError(f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                             f"num_key_value_heads ({self.num_key_value_heads})")

    @property
    def n_layer(self):
        return self.num_hidden_layers

    @property
    def rope_base(self):
        return self.rope_theta

    @classmethod
    def from_dict(cls, config_dict):
        return cls(**config_dict)

    @classmethod
    def from_name(cls, name):
        return get_transformer_config(name)

    def to_dict(self):
        return {f.name: getattr(self, f.name) for f in fields(self)}


@dataclass
class MoEConfig(TransformerConfig):
    num_experts_per_tok: int = 2
    num_local_experts: int = 8
    num_shared_experts: Optional[int] = None
    moe_intermediate_size: Optional[int] = None
    shared_expert_intermediate_size: Optional[int] = None
    router_aux_loss_coef: float = 0.01
    router_z_loss_coef: float = 0.001
    scoring_func: str = "softmax"
    seq_aux: bool = True
    norm_topk_prob: bool = True
    expert_bias: bool = False
    use_moe_in_all_layers: bool = True
    moe_layer_interval: int = 1
    first_moe_layer: int = 0

    def __post_init__(self):
        super().__post_init__()
        if self.moe_intermediate_size is None:
            self.moe_intermediate_size = self.intermediate_size
        self._validate_moe_config()

    def _validate_moe_config(self):
        if self.num_experts_per_tok > self.num_local_experts:
            raise ValueError(f"num_experts_per_tok ({self.num_experts_per_tok}) cannot be greater than "
                             f"num_local_experts ({self.num_local_experts})")
        if self.scoring_func not in ("softmax", "sigmoid"):
            raise ValueError(f"scoring_func must be 'softmax' or 'sigmoid', got '{self.scoring_func}'")

    @classmethod
    def from_name(cls, name):
        return get_moe_config(name)


TRANSFORMER_PRETRAINED_CONFIG_ARCHIVE_MAP = {
    "llama-7b": dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                     num_attention_heads=32, num_key_value_heads=32, max_position_embeddings=4096,
                     rope_theta=10000.0),
    "llama-13b": dict(vocab_size=32000, hidden_size=5120, intermediate_size=13824, num_hidden_layers=40,
                      num_attention_heads=40, num_key_value_heads=40, max_position_embeddings=4096,
                      rope_theta=10000.0),
    "qwen-0.5b": dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                      num_attention_heads=14, num_key_value_heads=2, max_position_embeddings=32768,
                      rope_theta=1000000.0),
    # Qwen2.5 shapes used by the training benchmarks (tied embeddings, q/k/v bias)
    "qwen2.5-0.5b": dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                         num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                         max_position_embeddings=32768, rope_theta=1000000.0, norm_eps=1e-6,
                         tie_word_embeddings=True, attention_bias=True),
    "qwen2.5-1.5b": dict(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                         num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                         max_position_embeddings=32768, rope_theta=1000000.0, norm_eps=1e-6,
                         tie_word_embeddings=True, attention_bias=True),
}

MOE_PRETRAINED_CONFIG_ARCHIVE_MAP = {
    "deepseek-moe-16b": dict(hidden_size=2048, intermediate_size=10944, num_hidden_layers=28,
                             num_attention_heads=16, num_key_value_heads=16, num_experts_per_tok=6,
                             num_local_experts=64, num_shared_experts=2, moe_intermediate_size=1408,
                             shared_expert_intermediate_size=2816, vocab_size=102400,
                             max_position_embeddings=4096),
    "mixtral-8x7b": dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                         num_attention_heads=32, num_key_value_heads=8, num_experts_per_tok=2,
                         num_local_experts=8, num_shared_experts=None, vocab_size=32000,
                         max_position_embeddings=32768, rope_theta=1000000.0),
    "moe-small": dict(hidden_size=768, intermediate_size=2048, num_hidden_layers=12, num_attention_heads=12,
                      num_key_value_heads=12, num_experts_per_tok=2, num_local_experts=4,
                      num_shared_experts=None, vocab_size=32000, max_position_embeddings=2048),
    # Qwen3-MoE-shaped benchmark model: every layer MoE, 128 experts of SwiGLU width 768, top-8
    "qwen3-moe-bench": dict(vocab_size=151936, hidden_size=2048, intermediate_size=768, num_hidden_layers=24,
                            num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                            max_position_embeddings=32768, rope_theta=1000000.0, num_experts_per_tok=8,
                            num_local_experts=128, moe_intermediate_size=768, router_aux_loss_coef=0.001,
                            norm_topk_prob=True, scoring_func="softmax"),
}


def get_transformer_config(name):
    if name not in TRANSFORMER_PRETRAINED_CONFIG_ARCHIVE_MAP:
        raise ValueError(f"Unknown model name: {name}. Available: "
                         f"{list(TRANSFORMER_PRETRAINED_CONFIG_ARCHIVE_MAP)}")
    return TransformerConfig(**TRANSFORMER_PRETRAINED_CONFIG_ARCHIVE_MAP[name])


def get_moe_config(name):
    if name not in MOE_PRETRAINED_CONFIG_ARCHIVE_MAP:
        raise ValueError(f"Unknown model name: {name}. Available: {list(MOE_PRETRAINED_CONFIG_ARCHIVE_MAP)}")
    return MoEConfig(**MOE_PRETRAINED_CONFIG_ARCHIVE_MAP[name])
