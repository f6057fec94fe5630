"""``int8mm_cuda`` (pytorch/int8mm-extension/int8mm.cpp:9-18) on niti_b200: ``int8_mm(lhs [m,k], rhs [k,n])`` ->
int32 [m,n], exact (the reference runs cublasGemmEx with int32 accumulation, int8mm_kernel.cu:8-34, and needs
k and n to be multiples of 4; any size is taken here)."""
import torch

from niti_b200 import ops
from niti_b200.compat import check_input


def int8_mm(lhs, rhs):
    check_input(lhs, rhs)
    if lhs.dtype != torch.int8 or rhs.dtype != torch.int8 or lhs.dim() != 2 or rhs.dim() != 2 or lhs.shape[1] != rhs.shape[0]:
        raise RuntimeError("int8_mm: int8 [m,k] and [k,n] matrices expected")
    return ops.gemm_acc(lhs, rhs)[0]
