"""``int8pool_cuda`` (pytorch/int8pool-extension/int8pool.cpp) on niti_b200.

``int8_pool(x, k, stride, pad)``: int8 NHWC max pooling (int8pool_kernel.cu:28-80).
``int8_pool_backward(y, dy, x, k, stride, pad)``: the reference passes fp16 copies because cuDNN has no int8
pooling backward (ti_torch.py:309-316, int8pool_kernel.cu:82-138) and converts the fp16 result back; the same
tensors are accepted here, narrowed to int8 (exact: every value is an int8), pooled backward in int8 and
returned in the dtype they came in.  Ties inside a window go to its first maximum (rows, then columns).
"""
import torch

from niti_b200 import ops
from niti_b200.compat import check_input


def int8_pool(input, kernel_size, stride, padding):
    check_input(input)
    if padding != 0:
        raise RuntimeError("int8_pool: padding is not implemented (the reference's models use 0)")
    return ops.maxpool_fwd(input, kernel_size, stride)


def int8_pool_backward(y, dy, x, kernel_size, stride, padding):
    check_input(y, dy, x)
    if padding != 0:
        raise RuntimeError("int8_pool_backward: padding is not implemented (the reference's models use 0)")
    dx = ops.maxpool_bwd(x.to(torch.int8), dy.to(torch.int8), kernel_size, stride)
    return dx.to(dy.dtype)
