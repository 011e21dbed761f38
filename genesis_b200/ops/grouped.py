"""Grouped (ragged) GEMM bindings for mixture-of-experts (GROUP_M / GROUP_K modes of `csrc/gemm_sm100.cu`)."""


def moe_sort(experts, num_experts, align):
    return NotImplemented


def grouped_linear(x, w, offsets):
    return NotImplemented


def grouped_dgrad(gy, w, offsets):
    return NotImplemented


def grouped_wgrad(gy, x, offsets, num_groups, out_dtype):
    return NotImplemented
