"""Drop-in for the reference's ``ti_vgg`` module, plus the layer lists the benchmark configs name."""
from torch.nn.modules import Sequential

from .ti_net import TiNet
from .ti_torch import TiConv2d, TiDropout, TiFlat, TiLinear, TiMaxpool2d, TiReLU

cifar_cfg = {
    # the reference's three depths (ti_vgg.py:10-14)
    7: [128, 128, 'M', 256, 256, 'M', 512, 512, 'M'],
    8: [128, 128, 128, 'M', 256, 256, 'M', 512, 512, 'M'],
    9: [128, 128, 128, 'M', 256, 256, 256, 'M', 512, 512, 'M'],
    # layer lists of the benchmark configurations that are not in the reference's table
    'vgg9_wide': [128, 128, 'M', 256, 256, 'M', 512, 512, 'M', 512, 512],
    'vgg13': [64, 64, 'M', 128, 128, 'M', 256, 256, 'M', 512, 512, 'M', 512, 512, 'M'],
}


class TiVGG_cifar(TiNet):
    """VGG-style integer CNN for 32x32 inputs (ti_vgg.py:16-42).  ``dropout`` keeps or drops the
    TiDropout the reference puts before the classifier; ``fuse_relu`` folds each ReLU's forward
    into the preceding convolution's requantisation kernel (same values, one pass less)."""

    def __init__(self, depth=None, dropout=True, fuse_relu=True, classes=10):
        super(TiVGG_cifar, self).__init__()
        self.forward_layers = self._make_layers(cifar_cfg[depth] if not isinstance(depth, list) else depth,
                                                dropout, fuse_relu, classes)
        self.assign_layer_ids()
        self.regime = [{'epoch': 0, 'gb': 5},
                       {'epoch': 100, 'gb': 4},
                       {'epoch': 150, 'gb': 3}]

    def _make_layers(self, cfg, dropout=True, fuse_relu=True, classes=10):
        layers = []
        in_channels = 3
        image_size = 32
        for idx, x in enumerate(cfg):
            if x == 'M':
                pool = TiMaxpool2d(2, 2)
                if fuse_relu and layers and isinstance(layers[-1], TiReLU):
                    # conv -> ReLU -> pool: the pool's backward also applies the ReLU's mask, and the convolution's
                    # kernel writes the pooled tensor too where it can
                    layers[-1].backward_in_next_layer = True
                    pool.relu_backward_fused = True
                    if len(layers) >= 2 and isinstance(layers[-2], TiConv2d):
                        layers[-2].pool_layer = pool
                layers += [pool]
                image_size = image_size // 2
            else:
                conv = TiConv2d(in_channels, x, first_layer=(idx == 0), fuse_relu=fuse_relu)
                if fuse_relu and layers and isinstance(layers[-1], TiReLU):
                    # conv -> ReLU -> conv: the second convolution's error-backward kernel applies the ReLU's mask
                    layers[-1].backward_in_next_layer = True
                    conv.relu_backward_fused = True
                layers += [conv, TiReLU(fused=fuse_relu)]
                in_channels = x
        layers += [TiFlat()]
        if dropout:
            layers += [TiDropout()]
        layers += [TiLinear(in_channels * image_size * image_size, classes, last_layer=True)]
        return Sequential(*layers)
