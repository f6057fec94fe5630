"""Drop-in for the reference's ``ti_net`` module: forward / hand-written backward walk of an
integer network (ti_net.py:8-48)."""
import collections

import torch
from torch.nn.modules import Module

from . import ops, ti_torch
from .ti_loss import TiLoss
from .ti_torch import RangeEstimate, TiDropout, TiFloatToInt8, TiLinear, exp_tensor


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

    def _fusable_head(self, batch):
        """(number of head layers, has dropout) if the network ends in [TiDropout,] TiLinear of a size the
        one-kernel classifier head takes, else None."""
        layers = list(self.forward_layers)
        if not (ti_torch.FUSE_HEAD and ti_torch.TRAINING and ti_torch.GLOBAL_MAX_GROUP is None and layers
                and isinstance(layers[-1], TiLinear)):
            return None
        drop = len(layers) >= 2 and isinstance(layers[-2], TiDropout)
        J, F = layers[-1].weight.shape
        if len(layers) - (2 if drop else 1) < 1 or not ops.fc_head_supported(batch, F, J):
            return None
        return (2 if drop else 1), drop

    def train_step(self, x, target):
        """forward(x) followed by backward(target), with the same results; when the network ends in
        [TiDropout,] TiLinear the whole classifier head (dropout, FC forward, loss, FC backward, update)
        runs as one kernel instead of eleven."""
        head = self._fusable_head(x.shape[0])
        if head is None:
            out = self.forward(x)
            self.backward(target)
            return out
        n_head, drop = head
        layers = list(self.forward_layers)
        body, lin = layers[:-n_head], layers[-1]
        h = TiFloatToInt8(x)
        for l in body:
            h = l(h)
        feat, feat_exp = h
        dev = feat.device
        lin.act_in = h
        out8, out_exp, err8, e8, err_exp, g32, gm = ops.fc_head_train(
            feat.contiguous(), exp_tensor(feat_exp, dev), lin.weight, lin.weight_exp,
            target.to(device=dev, dtype=torch.int64).contiguous(), ti_torch.RNG_SEED(dev), 16 * lin.layer_id,
            dropout=drop, bits=ti_torch.BITWIDTH, act_mode=ti_torch._mode(ti_torch.ACT_ROUND_METHOD),
            err_mode=ti_torch._mode(ti_torch.ERROR_ROUND_METHOD), grad_mode=ti_torch._mode(ti_torch.GRAD_ROUND_METHOD),
            mu=ti_torch.GRAD_BITWIDTH, update=not lin.defer_update, sample_offset=ti_torch.SAMPLE_OFFSET,
            g32=lin.grad_buffer)
        self.out, self.out_exp = out8, out_exp
        self.loss.out_grad = err8
        lin.grad_int32acc, lin.grad_maxabs, lin.err_exp = g32, gm, err_exp
        if lin.grad_ready is not None:
            lin.grad_ready(lin)
        e = (e8, err_exp)
        for l in reversed(body):
            e = l.backward(e)
        return self.out, self.out_exp

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
        """Accepts a reference checkpoint (float 0-dim ``weight_exp`` on the host) or one of ours.  The values are
        copied INTO the existing weight tensors (same shape): captured CUDA graphs and a data-parallel trainer's
        peer-visible arena keep pointing at that memory, so a checkpoint may be loaded at any time between steps."""
        for idx, l in enumerate(self.forward_layers):
            if hasattr(l, 'weight'):
                layer_prefix = 'layers.' + str(idx) + '.'
                dev = l.weight.device
                w = state_dict[layer_prefix + 'weight']
                e = exp_tensor(state_dict[layer_prefix + 'weight_exp'], dev)
                if tuple(w.shape) == tuple(l.weight.shape) and l.weight.dtype == torch.int8:
                    l.weight.copy_(w.to(device=dev, dtype=torch.int8))
                else:
                    l.weight = w.to(device=dev, dtype=torch.int8).contiguous()
                if isinstance(l.weight_exp, torch.Tensor) and l.weight_exp.device == e.device and l.weight_exp.dtype == e.dtype:
                    l.weight_exp.copy_(e)
                else:
                    l.weight_exp = e
