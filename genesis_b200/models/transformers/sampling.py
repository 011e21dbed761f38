"""Next-token sampling shared by the dense and MoE language models: temperature, top-k, nucleus (top-p), drawn with
the Gumbel-max trick so the whole step stays on the device (top-k / sort / arg-max are the framework's own kernels,
the noise comes from its Philox generator).  Reference counterpart: the sampling loop of
genesis/models/transformers/moe.py:546-590 (softmax + multinomial on the host library)."""
import torch

from ... import random as _random
from ...ops import dispatch as K


def sample_next(logits, temperature=1.0, top_k=None, top_p=None):
    """logits: raw float tensor [B, V] -> int64 token ids [B, 1].  temperature 0 means greedy."""
    x = logits.float()
    if temperature is None or temperature <= 0.0:
        return K.argmax(x, -1, True)
    if temperature != 1.0:
        x = x / temperature
    V = x.shape[-1]
    if top_k is not None and 0 < top_k < V:
        kth = K.topk(x, int(top_k), -1, True)[0][:, -1:]
        x = torch.where(x < kth, torch.full_like(x, float("-inf")), x)
    if top_p is not None and 0.0 < top_p < 1.0:
        sv, si = K.sort(x, -1, True)
        sp = torch.softmax(sv, -1)
        before = torch.cumsum(sp, -1) - sp                     # probability mass ranked above each token
        sv = torch.where(before >= top_p, torch.full_like(sv, float("-inf")), sv)
        x = torch.full_like(x, float("-inf")).scatter_(-1, si, sv)
    seed, offset = _random.default_generator().next_philox()
    u = K.random_fill("uniform", tuple(x.shape), torch.float32, x.device, seed, offset, 0.0, 1.0)
    u = u.clamp_(1e-20, 1.0 - 1e-7)
    gumbel = -torch.log(-torch.log(u))
    return K.argmax(x + gumbel, -1, True)
