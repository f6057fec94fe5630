"""Generate the golden vectors under tests/golden by executing the REFERENCE's own Python.

Run in a checkout that has the reference tree available::

    python tests/golden/make_golden.py [/path/to/reference]

The reference ships no tests or fixtures, so the vectors are produced by importing its
``ti_torch.py`` / ``ti_loss.py`` / ``ti_net.py`` / ``ti_vgg.py`` unmodified on the CPU under
``oracle/ref_harness.py`` (extension modules replaced by exact integer stand-ins, torch-1.7
truncating ``//``, injected random words).  Inputs are regenerated from the recorded seeds
with ``numpy.random.Generator(PCG64)``; outputs are stored in full when small and as CRC32
otherwise.  ``tests/test_oracle_golden.py`` checks the oracle restatement against them.
"""
import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import niti_oracle as O, philox, ref_harness  # noqa: E402


def crc(a):
    return np.uint32(zlib.crc32(np.ascontiguousarray(a).tobytes()))


def t8(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def xavier_exp(shape):
    """Exponent weight_quant (ti_torch.py:334-339) gives a tensor whose max reaches the xavier bound."""
    if len(shape) == 4:
        K, R, S, C = shape
        fan_in, fan_out = C * R * S, K * R * S
    else:
        fan_out, fan_in = shape
    a = np.sqrt(6.0 / (fan_in + fan_out))
    return int(np.ceil(np.log2(a))) - 7


def synth_images(rng, B):
    """uint8 images -> /255 -> normalise with the CIFAR-10 statistics of data.py:5-6."""
    mean = np.array([0.49139968, 0.48215827, 0.44653124], dtype=np.float32)
    std = np.array([0.24703233, 0.24348505, 0.26158768], dtype=np.float32)
    u8 = rng.integers(0, 256, size=(B, 3, 32, 32), dtype=np.uint8)
    x = (u8.astype(np.float32) / np.float32(255.0) - mean[None, :, None, None]) / std[None, :, None, None]
    return x.astype(np.float32)


def gen_requant(H, out):
    T = H.ti_torch
    rng = np.random.default_rng(101)
    recs = {}
    for shift in (1, 2, 3, 4, 5, 8, 11, 16, 24):
        hi = 1 << min(30, shift + 8)
        x = rng.integers(-hi, hi, size=4096).astype(np.int32)
        x[:8] = [0, 1, -1, (1 << shift) - 1, -(1 << shift) + 1, 1 << (shift - 1), -(1 << (shift - 1)), (1 << (shift - 1)) - 1]
        words = philox.random_u32_tensor(11, shift, x.shape)
        with H.active(rand_provider=lambda i, size, high: words):
            recs[f"round_{shift}"] = T.RoundShift(t8(x), shift).numpy()
            recs[f"psto_{shift}"] = T.PstoShift(t8(x), shift).numpy()
            recs[f"sto_{shift}"] = T.StoShift(t8(x), shift).numpy()
    # act/err/grad_calc around the bit-width edges (max = 2^k, 2^k +- 1), including the wrap at 128
    for mx in (0, 1, 2, 64, 127, 128, 129, 255, 256, 257, 1000, 4096, 4097, 65535, 65536, 65537, 1 << 20):
        x = rng.integers(-mx, mx + 1, size=2048).astype(np.int32)
        x[0] = mx
        x[1] = -mx
        with H.active():
            a, e = T.act_calc(t8(x), 3)
            recs[f"act_{mx}"] = a.numpy()
            recs[f"act_{mx}_exp"] = np.int32(e)
            a, e = T.err_calc(t8(x))
            recs[f"err_{mx}"] = a.numpy()
            recs[f"err_{mx}_shift"] = np.int32(e)
            for mu in (5, 4, 3):
                a, e = T.grad_calc(t8(x), mu)
                recs[f"grad{mu}_{mx}"] = a.numpy()
                recs[f"grad{mu}_{mx}_shift"] = np.int32(e)
    np.savez_compressed(os.path.join(out, "requant.npz"), **recs)


def gen_layers(H, out):
    """TiConv2d / TiLinear / TiMaxpool2d / TiReLU / TiLoss forward+backward on small shapes."""
    T = H.ti_torch
    recs = {}
    rng = np.random.default_rng(202)
    N, Hh, W, C, K = 4, 8, 8, 16, 32
    x = rng.integers(-127, 128, size=(N, Hh, W, C)).astype(np.int8)
    w = rng.integers(-127, 128, size=(K, 3, 3, C)).astype(np.int8)
    err = rng.integers(-127, 128, size=(N, Hh, W, K)).astype(np.int8)
    with H.active(grad_bitwidth=5):
        conv = T.TiConv2d(C, K)
        conv.weight, conv.weight_exp = t8(w), torch.tensor(-9.0)
        y, ye = conv.forward((t8(x), torch.tensor(-5.0)))
        e, ee = conv.backward((t8(err), 0))
        recs["conv_y"], recs["conv_y_exp"] = y.numpy(), np.int32(ye)
        recs["conv_e"], recs["conv_e_exp"] = e.numpy(), np.int32(ee)
        recs["conv_g32"] = conv.grad_int32acc.numpy().astype(np.int32)
        recs["conv_w_new"] = conv.weight.numpy()
        # first layer (C=3): group-conv weight gradient, no error propagation
        x3 = rng.integers(-127, 128, size=(N, Hh, W, 3)).astype(np.int8)
        w3 = rng.integers(-127, 128, size=(K, 3, 3, 3)).astype(np.int8)
        c1 = T.TiConv2d(3, K, first_layer=True)
        c1.weight, c1.weight_exp = t8(w3), torch.tensor(-8.0)
        y, ye = c1.forward((t8(x3), torch.tensor(-6.0)))
        c1.backward((t8(err), 0))
        recs["conv1_y"], recs["conv1_y_exp"] = y.numpy(), np.int32(ye)
        recs["conv1_g32"] = c1.grad_int32acc.numpy().astype(np.int32)
        recs["conv1_w_new"] = c1.weight.numpy()
        # linear
        B, fin, fout = 8, 256, 10
        a = rng.integers(-127, 128, size=(B, fin)).astype(np.int8)
        wl = rng.integers(-127, 128, size=(fout, fin)).astype(np.int8)
        el = rng.integers(-127, 128, size=(B, fout)).astype(np.int8)
        lin = T.TiLinear(fin, fout)
        lin.weight, lin.weight_exp = t8(wl), torch.tensor(-9.0)
        y, ye = lin.forward((t8(a), torch.tensor(-3.0)))
        e, ee = lin.backward((t8(el), 0))
        recs["lin_y"], recs["lin_y_exp"] = y.numpy(), np.int32(ye)
        recs["lin_e"], recs["lin_e_exp"] = e.numpy(), np.int32(ee)
        recs["lin_g32"] = lin.grad_int32acc.numpy().astype(np.int32)
        recs["lin_w_new"] = lin.weight.numpy()
        # relu / pool (pool input chosen without ties inside a window: tie routing is unpinned)
        relu = T.TiReLU()
        y, _ = relu.forward((t8(x), 0))
        e, _ = relu.backward((t8(rng.integers(-127, 128, size=x.shape).astype(np.int8)), 0))
        recs["relu_y"], recs["relu_e"] = y.numpy(), e.numpy()
        perm = np.stack([rng.permutation(256)[:Hh * W].reshape(Hh, W) for _ in range(N * C)])
        xp = (perm.reshape(N, C, Hh, W).transpose(0, 2, 3, 1) - 128).astype(np.int8)
        pool = T.TiMaxpool2d(2, 2)
        y, _ = pool.forward((t8(xp), 0))
        dy = rng.integers(-127, 128, size=y.shape).astype(np.int8)
        e, _ = pool.backward((t8(dy), 0))
        recs["pool_x"], recs["pool_y"], recs["pool_dy"], recs["pool_dx"] = xp, y.numpy(), dy, e.numpy()
    recs.update(x=x, w=w, err=err, x3=x3, w3=w3, lin_a=a, lin_w=wl, lin_err=el)
    # TiLoss over both branches of out_exp and several logit scales
    loss = H.ti_loss.TiLoss()
    for k, out_exp in enumerate((-9, -7, -6, -3, 0, 2)):
        B = 64
        ov = rng.integers(-127, 128, size=(B, 10)).astype(np.int8)
        if k % 2:
            ov = (ov // 8).astype(np.int8)
        tgt = rng.integers(0, 10, size=B)
        words = philox.random_u32_tensor(5, 0xFFFF, (B, 10))
        with H.active(rand_provider=lambda i, size, high: words):
            g, ge = loss.forward(t8(ov), torch.tensor(float(out_exp)), torch.from_numpy(tgt))
        recs[f"loss{k}_out"], recs[f"loss{k}_exp"], recs[f"loss{k}_tgt"] = ov, np.int32(out_exp), tgt
        recs[f"loss{k}_err"] = g.numpy()
    np.savez_compressed(os.path.join(out, "layers.npz"), **recs)


def run_ref_net(H, cfg, B, seed, dropout, steps=1, mu=5):
    """One or more full training steps of the reference's TiNet over ``cfg``; returns a record."""
    T, V = H.ti_torch, H.ti_vgg
    rng = np.random.default_rng(seed)
    shapes, cin = [], 3
    for c in cfg:
        if c != "M":
            shapes.append((c, 3, 3, cin))
            cin = c
    feat = 512 * (32 // 2 ** cfg.count("M")) ** 2
    shapes.append((10, feat))
    weights = [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes]
    wexps = [xavier_exp(s) for s in shapes]
    rec = {"cfg": np.array([0 if c == "M" else c for c in cfg]), "B": B, "seed": seed,
           "dropout": int(dropout), "steps": steps, "mu": mu}
    with H.active(grad_bitwidth=mu, training=True) as mode:
        net = V.TiVGG_cifar.__new__(V.TiVGG_cifar)
        H.ti_net.TiNet.__init__(net)
        layers = list(V.TiVGG_cifar._make_layers(net, cfg))
        if not dropout:
            layers = [l for l in layers if not isinstance(l, T.TiDropout)]
        net.forward_layers = torch.nn.Sequential(*layers)
        wl = [l for l in net.forward_layers if hasattr(l, "weight")]
        for l, w, e in zip(wl, weights, wexps):
            l.weight, l.weight_exp = t8(w), torch.tensor(float(e))
        for step in range(steps):
            x = synth_images(rng, B)
            tgt = rng.integers(0, 10, size=B)
            calls = []
            if dropout:
                calls.append(philox.random_u32_tensor(seed + step, 0xFFFE, (feat,)))
            calls.append(philox.random_u32_tensor(seed + step, 0xFFFF, (B, 10)))
            mode.rand_calls = 0
            mode.rand_provider = lambda i, size, high, calls=calls: calls[i]
            out, out_exp = net.forward(torch.from_numpy(x))
            net.backward(torch.from_numpy(tgt))
            rec[f"s{step}_out"] = out.numpy()
            rec[f"s{step}_out_exp"] = np.int32(out_exp)
            rec[f"s{step}_loss_err"] = net.loss.out_grad.numpy()
            for i, l in enumerate(wl):
                rec[f"s{step}_w{i}_crc"] = crc(l.weight.numpy())
                rec[f"s{step}_g{i}_crc"] = crc(l.grad_int32acc.numpy().astype(np.int32))
                if i:
                    rec[f"s{step}_errexp{i}"] = np.int32(l.err_exp)
    return rec


def gen_nets(H, out):
    small = [16, "M", 32, "M", 512, "M"]
    np.savez_compressed(os.path.join(out, "net_small.npz"), **run_ref_net(H, small, 4, 1235, True, steps=2))
    np.savez_compressed(os.path.join(out, "net_small_nodrop.npz"), **run_ref_net(H, small, 8, 1236, False, steps=2, mu=4))
    vgg7 = [128, 128, "M", 256, 256, "M", 512, 512, "M"]
    np.savez_compressed(os.path.join(out, "net_vgg7_b4.npz"), **run_ref_net(H, vgg7, 4, 1237, True, steps=1))


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NITI_REFERENCE_DIR")  # a checkout of wangmaolin/niti
    H = ref_harness.load(ref)
    gen_requant(H, HERE)
    gen_layers(H, HERE)
    gen_nets(H, HERE)
    print("golden vectors written to", HERE)
