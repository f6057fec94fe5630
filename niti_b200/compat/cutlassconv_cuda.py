"""``cutlassconv_cuda`` (pytorch/cutlass-extension/cutlassconv.cpp:57-73) on the tcgen05 kernels of niti_b200.

``sp_conv`` / ``sp_conv_optimized(input, weight, stride, padding)``: int8 NHWC input [N,H,W,C] and int8 filters
[K,R,S,C] -> int32 [N,P,Q,K], P = H + 2*padding - R + 1 (cutlassconv_kernel.cu:133-138).  The reference calls it
in three ways (ti_torch.py:178-192, 403-405, 429-432): the forward convolution, the error convolution over
flipped / transposed filters, and the weight gradient written as a convolution of the transposed activations with
the transposed errors as image-sized filters.  The last form is recognised by its shape and handed to the
weight-gradient kernel; everything else goes to the forward kernel, which takes any filter size.
"""
import torch

from niti_b200 import ops
from niti_b200.compat import check_input


def _conv(input, weight, stride, padding):
    check_input(input, weight)
    if input.dtype != torch.int8 or weight.dtype != torch.int8 or input.dim() != 4 or weight.dim() != 4:
        raise RuntimeError("sp_conv: int8 NHWC input and int8 [K,R,S,C] filters expected")
    if stride != 1:
        raise RuntimeError("sp_conv: only stride 1 is implemented (the reference's models use no other)")
    C, H, W, N = input.shape
    K, R, S, _ = weight.shape
    P, Q = H + 2 * padding - R + 1, W + 2 * padding - S + 1
    if R > 2 * padding + 1 and S > 2 * padding + 1 and P * Q <= 49 and C % 16 == 0 and K % 16 == 0 and N % 16 == 0:
        # weight gradient in disguise: input = activations [C,H,W,N], filters = errors [K,P',Q',N] of the layer's
        # output size; out[c,p,q,k] = sum_{n,h,w} x[n,h+p-pad,w+q-pad,c] * err[n,h,w,k] = dW[k,p,q,c]
        x = input.permute(3, 1, 2, 0).contiguous()
        err = weight.permute(3, 1, 2, 0).contiguous()
        if err.shape[1] + 2 * padding - P + 1 == H and P == Q:
            g32, _ = ops.conv_wgrad_acc(x, err, P, Q, padding)
            return g32.permute(3, 1, 2, 0).contiguous()
    return ops.conv_fprop_acc(input, weight, padding, stride)[0]


def sp_conv(input, weight, stride, padding):
    return _conv(input, weight, stride, padding)


def sp_conv_optimized(input, weight, stride, padding):
    return _conv(input, weight, stride, padding)


def _conv4(input, weight):
    check_input(input, weight)
    if input.dim() != 4 or weight.dim() != 4 or input.shape[3] != weight.shape[3]:
        raise RuntimeError("int4_conv: [N,H,W,C/2] input and [K,R,S,C/2] filters expected (two int4 per byte)")
    return ops.conv_fprop_i4(input.view(torch.uint8), weight.view(torch.uint8), 1)[0]


def int4_conv(input, weight):
    """cutlassconv.cpp:83-89: 3x3, pad 1, stride 1; int4 pairs packed in the bytes of int8 / uint8 tensors."""
    return _conv4(input, weight)


def int4_conv_optimized(input, weight):
    return _conv4(input, weight)
