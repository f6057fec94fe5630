"""``int8conv_cuda`` (pytorch/int8conv-extension/int8conv.cpp:35-45) on niti_b200.

``group_conv(input, weight, stride, padding, dilation, groups)`` as conv2d_weight_int8 (ti_torch.py:194-233) calls
it for the first layer's weight gradient: input [1,H,W,G] int8 with one channel per group, weight [G*Kg,R,S,1]
int8, float32 result [1,P,Q,G*Kg] (the reference's cuDNN call accumulates in float, int8conv_kernel.cu:298-334;
here the sums are exact integers converted to float32, which is the same value whenever float32 holds it).
The reference passes (dilation, padding, stride) in that order for parameters named (stride, padding, dilation);
both orders mean 1, pad, 1 and anything else is refused.
"""
import torch

from niti_b200 import ops
from niti_b200.compat import check_input


def group_conv(input, weight, stride, padding, dilation, groups):
    check_input(input, weight)
    if stride != 1 or dilation != 1:
        raise RuntimeError("group_conv: only stride 1 and dilation 1 are implemented")
    if input.dim() != 4 or weight.dim() != 4 or input.shape[0] != 1 or input.shape[3] != groups or weight.shape[3] != 1 \
            or weight.shape[0] % groups != 0:
        raise RuntimeError("group_conv: expected input [1,H,W,groups] and weight [groups*k,R,S,1] (one channel per group)")
    return ops.group_conv1(input, weight, padding).float()
