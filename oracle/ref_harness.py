"""Run the reference's own Python (ti_torch / ti_loss / ti_net / ti_vgg) on the CPU, unmodified.

TEST INFRASTRUCTURE.  Used to pin the oracle restatement, to generate the golden vectors under
``tests/golden``, as the timed CPU arm of the benchmark (``bench.py --impl reference``) and, in
its GPU form, to run the reference's layers over this library's kernels.  ``load(ref_dir)``
(default: ``oracle/_ref``, which ``oracle/make_ref.py`` fills from a checkout of the reference)
returns the imported reference modules after arranging that:

1. the four CUDA extension modules the reference imports (``cutlassconv_cuda``,
   ``int8mm_cuda``, ``int8pool_cuda``, ``int8conv_cuda``; ti_torch.py:3-6) resolve to
   exact CPU integer stand-ins with the extension signatures;
2. ``options`` (argparse at import, options.py:22) sees a clean ``sys.argv``;
3. every call that names ``device='cuda'`` / ``.to('cuda')`` lands on the CPU;
4. ``tensor // int`` truncates toward zero, as in the torch 1.7 the reference targets;
5. ``torch.randint`` returns injected words, so stochastic rounding and dropout use the
   same counter-based bits as the kernels under test.

Items 3-5 are a ``TorchFunctionMode`` active only inside ``with harness.active(...)``.

``load(..., device="cuda", extension_dir=...)`` is the GPU form: item 1 is replaced by putting
``extension_dir`` (modules with the four extension names, e.g. ``niti_b200/compat``) on the import path and
item 3 is dropped, so the reference's Python runs on the GPU and calls those modules.
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
        x, w = _np(inp), _np(weight)
        R, S = w.shape[1], w.shape[2]
        P, Q = x.shape[1] + 2 * padding - R + 1, x.shape[2] + 2 * padding - S + 1
        if stride == 1 and R > 2 * padding + 1 and S > 2 * padding + 1 and P * Q <= 49:
            # the weight gradient written as a convolution with image-sized filters (ti_torch.py:429-432):
            # out[c,p,q,k] = sum_{n,h,w} x[c,h+p-pad,w+q-pad,n] * w[k,h,w,n] -- the same exact sums, taken tap by tap
            g = O.conv_wgrad(np.ascontiguousarray(x.transpose(3, 1, 2, 0)), np.ascontiguousarray(w.transpose(3, 1, 2, 0)), P, Q, padding)
            return torch.from_numpy(np.ascontiguousarray(g.transpose(3, 1, 2, 0)).astype(np.int32))
        acc = O.conv_fprop(x, w, pad=padding, stride=stride)
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
    def __init__(self, rand_provider, device="cpu"):
        super().__init__()
        self.rand_provider = rand_provider
        self.rand_calls = 0
        self.device = device

    def __torch_function__(self, func, types_, args=(), kwargs=None):
        kwargs = dict(kwargs or {})
        dev = kwargs.get("device")
        if self.device == "cpu":
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
            return torch.from_numpy(vals).to(kwargs.get("dtype", torch.int64)).reshape(tuple(size)).to(self.device)
        return func(*args, **kwargs)


class Harness:
    def __init__(self, mods, device="cpu"):
        self.device = device
        self.ti_torch = mods["ti_torch"]
        self.ti_loss = mods["ti_loss"]
        self.ti_net = mods["ti_net"]
        self.ti_vgg = mods["ti_vgg"]

    @contextlib.contextmanager
    def active(self, rand_provider=None, grad_bitwidth=5, training=True):
        def no_rand(i, size, high):
            raise RuntimeError("randint called but no random words were injected")
        self.ti_torch.GPU = self.device
        self.ti_torch.GRAD_BITWIDTH = grad_bitwidth
        self.ti_torch.TRAINING = training
        with _Mode(rand_provider or no_rand, self.device) as m:
            yield m


def default_ref_dir():
    """oracle/_ref when oracle/make_ref.py has filled it, else the NITI_REFERENCE_DIR environment variable, else None."""
    from . import make_ref
    if make_ref.available():
        return make_ref.REF_OUT
    return os.environ.get("NITI_REFERENCE_DIR")


def load(ref_dir=None, device="cpu", extension_dir=None):
    """Import the reference modules from ``ref_dir`` (default: see default_ref_dir) and return a Harness.
    device="cpu": the extension modules are the exact CPU stand-ins above.  device="cuda": ``extension_dir`` must
    hold modules named like the reference's extensions; they are imported from there and the reference runs on the GPU."""
    ref_dir = ref_dir or default_ref_dir()
    if not ref_dir or not os.path.isdir(ref_dir):
        raise FileNotFoundError("the reference's Python is needed: run `python -m oracle.make_ref <checkout>`, "
                                "pass its directory or set NITI_REFERENCE_DIR")
    ext_names = ("cutlassconv_cuda", "int8mm_cuda", "int8pool_cuda", "int8conv_cuda")
    if device == "cpu":
        for name, mod in _stub_modules().items():
            sys.modules[name] = mod
    else:
        if not extension_dir:
            raise ValueError("the GPU form needs extension_dir (modules named " + ", ".join(ext_names) + ")")
        for name in ext_names:
            sys.modules.pop(name, None)
        sys.path.insert(0, extension_dir)
        try:
            for name in ext_names:
                importlib.import_module(name)
        finally:
            sys.path.remove(extension_dir)
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
        for name in ("options", "ti_torch", "ti_loss", "ti_net", "ti_vgg") + ext_names:
            sys.modules.pop(name, None)  # the reference's module names must not shadow anything else in the process
    return Harness(mods, device)
