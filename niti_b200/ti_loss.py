"""Drop-in for the reference's ``ti_loss`` module: the integer cross-entropy error of NITI."""
import torch
from torch.nn.modules import Module

from . import ops
from . import ti_torch


class TiLoss(Module):
    """TiLoss.forward of the reference (ti_loss.py:6-36) as one kernel: base-2 softmax error in
    the reference's float32 order of operations (the branch on ``out_exp > -7`` is taken on the
    device), then StoShift by 4 bits.  Returns ``(int8 error [B, classes], exponent 0)``."""

    def forward(self, out_val, out_exp, target):
        dev = out_val.device
        self.out_grad = ops.loss_err(out_val.contiguous(), ti_torch.exp_tensor(out_exp, dev),
                                     target.to(device=dev, dtype=torch.int64).contiguous(),
                                     ti_torch.RNG_SEED(dev), 0xFFFF, ti_torch.SAMPLE_OFFSET)
        return self.out_grad, torch.zeros((), dtype=torch.int32, device=dev)
