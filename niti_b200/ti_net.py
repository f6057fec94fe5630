"""Drop-in for the reference's ``ti_net`` module: forward / hand-written backward walk of an
integer network (ti_net.py:8-48)."""
import collections

import torch
from torch.nn.modules import Module

from .ti_loss import TiLoss
from .ti_torch import RangeEstimate, TiFloatToInt8, exp_tensor


class TiNet(Module):
    """Integer network: quantise the float input, run the layers on (int8, exponent) tuples, and
    back-propagate the integer error layer by layer -- no autograd (ti_net.py:17-32)."""

    def __init__(self):
        super(TiNet, self).__init__()
        self.loss = TiLoss()

    def assign_layer_ids(self):
        """Number the weighted layers in forward order; the ids select their random-bit streams."""
        i = 0
        for l in self.forward_layers:
            if hasattr(l, 'weight'):
                l.layer_id = i
                i += 1

    def weighted_layers(self):
        return [l for l in self.forward_layers if hasattr(l, 'weight')]

    def forward(self, x):
        x = TiFloatToInt8(x)  # NCHW float -> NHWC int8 + exponent
        self.out, self.out_exp = self.forward_layers(x)
        return self.out, self.out_exp

    @property
    def out_bits(self):
        """Bit-width of the logits (ti_net.py:22); computed on demand because it synchronises."""
        return RangeEstimate(self.out)

    def backward(self, target):
        x = self.loss(self.out, self.out_exp, target)
        for layer in reversed(self.forward_layers):
            if isinstance(layer, torch.nn.Sequential):
                for block in reversed(layer):
                    x = block.backward(x)
            else:
                x = layer.backward(x)

    def state_dict(self):
        """Same keys as the reference (ti_net.py:34-41): layers.<idx>.weight / .weight_exp."""
        state_dict = collections.OrderedDict()
        for idx, l in enumerate(self.forward_layers):
            if hasattr(l, 'weight'):
                layer_prefix = 'layers.' + str(idx) + '.'
                state_dict[layer_prefix + 'weight'] = l.weight
                state_dict[layer_prefix + 'weight_exp'] = l.weight_exp
        return state_dict

    def load_state_dict(self, state_dict):
        """Accepts a reference checkpoint (float 0-dim ``weight_exp`` on the host) or one of ours."""
        for idx, l in enumerate(self.forward_layers):
            if hasattr(l, 'weight'):
                layer_prefix = 'layers.' + str(idx) + '.'
                dev = l.weight.device
                l.weight = state_dict[layer_prefix + 'weight'].to(device=dev, dtype=torch.int8).contiguous()
                l.weight_exp = exp_tensor(state_dict[layer_prefix + 'weight_exp'], dev)
