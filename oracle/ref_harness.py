"""Run the reference's own Python (ti_torch / ti_loss / ti_net / ti_vgg) on the CPU, unmodified.

TEST INFRASTRUCTURE.  Used in the build container only, to pin the oracle restatement and
to generate the golden vectors under ``tests/golden``; nothing on a GPU box imports it
(the reference tree does not travel).  ``load(ref_dir)`` returns the imported reference
modules after arranging that:

1. the four CUDA extension modules the reference imports (``cutlassconv_cuda``,
   ``int8mm_cuda``, ``int8pool_cuda``, ``int8conv_cuda``; ti_torch.py:3-6) resolve to
   exact CPU integer stand-ins with the extension signatures;
2. ``options`` (argparse at import, options.py:22) sees a clean ``sys.argv``;
3. every call that names ``device='cuda'`` / ``.to('cuda')`` lands on the CPU;
4. ``tensor // int`` truncates toward zero, as in the torch 1.7 the reference targets;
5. ``torch.randint`` returns injected words, so stochastic rounding and dropout use the
   same counter-based bits as the kernels under test.

Items 3-5 are a ``TorchFunctionMode`` active only inside ``with harness.active(...)``.
"""
import contextlib
import importlib
import os
import sys
import types

import numpy as np
import torch
from torch.overrides import TorchFunctionMode

from . import niti_oracle as O


def _np(t):
    return t.detach().cpu().numpy()


def _stub_modules():
    conv = types.ModuleType("cutlassconv_cuda")

    def sp_conv(inp, weight, stride, padding):
        assert inp.dtype == torch.int8 and weight.dtype == torch.int8
        assert inp.size(3) % 16 == 0, "extension contract: C % 16 == 0"
        acc = O.conv_fprop(_np(inp), _np(weight), pad=padding, stride=stride)
        return torch.from_numpy(acc.astype(np.int32))

    conv.sp_conv = sp_conv
    conv.sp_conv_optimized = sp_conv

    mm = types.ModuleType("int8mm_cuda")

    def int8_mm(a, b):
        assert a.size(1) % 4 == 0 and b.size(1) % 4 == 0, "extension contract: n, k % 4 == 0"
        return torch.from_numpy(O.int8_mm(_np(a), _np(b)).astype(np.int32))

    mm.int8_mm = int8_mm

    pool = types.ModuleType("int8pool_cuda")

    def int8_pool(x, k, stride, pad):
        assert pad == 0
        return torch.from_numpy(O.maxpool_fwd(_np(x), k, stride))

    def int8_pool_backward(y_half, dy_half, x_half, k, stride, pad):
        assert pad == 0
        dx = O.maxpool_bwd(_np(x_half).astype(np.int8), _np(dy_half).astype(np.int8), k, stride)
        return torch.from_numpy(dx.astype(np.float16))

    pool.int8_pool = int8_pool
    pool.int8_pool_backward = int8_pool_backward

    gconv = types.ModuleType("int8conv_cuda")

    def group_conv(inp, weight, a, padding, b, groups):
        # NHWC grouped cross-correlation, float32 result (int8conv_kernel.cu:248-334)
        x = inp.permute(0, 3, 1, 2).double()
        w = weight.permute(0, 3, 1, 2).double()
        y = torch.nn.functional.conv2d(x, w, None, 1, padding, 1, groups)
        return y.permute(0, 2, 3, 1).contiguous().float()

    gconv.group_conv = group_conv
    return {m.__name__: m for m in (conv, mm, pool, gconv)}


class _Mode(TorchFunctionMode):
    def __init__(self, rand_provider):
        super().__init__()
        self.rand_provider = rand_provider
        self.rand_calls = 0

    def __torch_function__(self, func, types_, args=(), kwargs=None):
        kwargs = dict(kwargs or {})
        dev = kwargs.get("device")
        if dev is not None and str(dev).startswith("cuda"):
            kwargs["device"] = "cpu"
        if func is torch.Tensor.to and len(args) >= 2 and isinstance(args[1], (str, torch.device)) \
                and str(args[1]).startswith("cuda"):
            args = (args[0], "cpu") + tuple(args[2:])
        if func in (torch.Tensor.__floordiv__, torch.floor_divide, torch.Tensor.floor_divide):
            return torch.div(args[0], args[1], rounding_mode="trunc")
        if func is torch.randint:
            size = kwargs.get("size")
            high = kwargs.get("high")
            if size is None or high is None:
                raise RuntimeError("unexpected randint call form")
            words = self.rand_provider(self.rand_calls, tuple(size), int(high))
            self.rand_calls += 1
            assert high & (high - 1) == 0
            vals = (np.asarray(words).astype(np.int64) & (high - 1))
            return torch.from_numpy(vals).to(kwargs.get("dtype", torch.int64)).reshape(tuple(size))
        return func(*args, **kwargs)


class Harness:
    def __init__(self, mods):
        self.ti_torch = mods["ti_torch"]
        self.ti_loss = mods["ti_loss"]
        self.ti_net = mods["ti_net"]
        self.ti_vgg = mods["ti_vgg"]

    @contextlib.contextmanager
    def active(self, rand_provider=None, grad_bitwidth=5, training=True):
        def no_rand(i, size, high):
            raise RuntimeError("randint called but no random words were injected")
        self.ti_torch.GPU = "cpu"
        self.ti_torch.GRAD_BITWIDTH = grad_bitwidth
        self.ti_torch.TRAINING = training
        with _Mode(rand_provider or no_rand) as m:
            yield m


def load(ref_dir=None):
    """Import the reference modules from ``ref_dir`` (a checkout of wangmaolin/niti; default: the directory named by
    the NITI_REFERENCE_DIR environment variable) under the stand-ins; returns a Harness."""
    ref_dir = ref_dir or os.environ.get("NITI_REFERENCE_DIR")
    if not ref_dir or not os.path.isdir(ref_dir):
        raise FileNotFoundError("the reference checkout is needed: pass its directory or set NITI_REFERENCE_DIR")
    for name, mod in _stub_modules().items():
        sys.modules[name] = mod
    saved_argv = sys.argv
    sys.argv = [saved_argv[0] if saved_argv else "harness"]
    sys.path.insert(0, ref_dir)
    try:
        mods = {}
        for name in ("options", "ti_torch", "ti_loss", "ti_net", "ti_vgg"):
            sys.modules.pop(name, None)
        for name in ("ti_torch", "ti_loss", "ti_net", "ti_vgg"):
            mods[name] = importlib.import_module(name)
    finally:
        sys.argv = saved_argv
        sys.path.remove(ref_dir)
    return Harness(mods)
