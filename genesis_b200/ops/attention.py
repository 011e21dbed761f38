"""Flash-attention bindings (kernels in `csrc/attention_sm100.cu`)."""


def forward(q, k, v, causal, scale):
    return NotImplemented


def backward(do, q, k, v, o, lse, causal, scale):
    return NotImplemented
