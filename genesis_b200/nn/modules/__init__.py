from .module import Module, Parameter
from .container import Sequential, ModuleList, ModuleDict
from .linear import Linear, Flatten
from .activation import ReLU, Softmax, SiLU, GELU, Sigmoid, Tanh, Residual
from .dropout import Dropout
from .normalization import BatchNorm1d, LayerNorm, FusedLayerNorm, RMSNorm
from .sparse import Embedding, RotaryEmbedding
from .loss import SoftmaxLoss, CrossEntropyLoss, MSELoss, L1Loss, BCELoss, BCEWithLogitsLoss
from .transformer import FeedFowardSwiGLU, FeedForwardSwiGLU, MultiheadAttention, FusedMultiheadAttention
