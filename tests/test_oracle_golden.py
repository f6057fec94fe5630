"""The oracle restatement against the vectors the reference's own Python produced
(tests/golden/make_golden.py)."""
import os
import zlib

import numpy as np
import pytest

from oracle import niti_oracle as O, philox
from tests.golden.make_golden import synth_images, xavier_exp


def crc(a):
    return np.uint32(zlib.crc32(np.ascontiguousarray(a).tobytes()))


def test_requant_closed_forms(golden_dir):
    g = np.load(os.path.join(golden_dir, "requant.npz"))
    rng = np.random.default_rng(101)
    for shift in (1, 2, 3, 4, 5, 8, 11, 16, 24):
        hi = 1 << min(30, shift + 8)
        x = rng.integers(-hi, hi, size=4096).astype(np.int32)
        x[:8] = [0, 1, -1, (1 << shift) - 1, -(1 << shift) + 1, 1 << (shift - 1), -(1 << (shift - 1)), (1 << (shift - 1)) - 1]
        words = philox.random_u32_tensor(11, shift, x.shape)
        assert np.array_equal(O.round_shift(x, shift), g[f"round_{shift}"])
        assert np.array_equal(O.psto_shift(x, shift), g[f"psto_{shift}"])
        assert np.array_equal(O.sto_shift(x, shift, words), g[f"sto_{shift}"])
    for mx in (0, 1, 2, 64, 127, 128, 129, 255, 256, 257, 1000, 4096, 4097, 65535, 65536, 65537, 1 << 20):
        x = rng.integers(-mx, mx + 1, size=2048).astype(np.int32)
        x[0] = mx
        x[1] = -mx
        a, e, _ = O.act_calc(x, 3)
        assert np.array_equal(a, g[f"act_{mx}"]) and e == g[f"act_{mx}_exp"]
        a, s = O.err_calc(x)
        assert np.array_equal(a, g[f"err_{mx}"]) and s == g[f"err_{mx}_shift"]
        for mu in (5, 4, 3):
            a, s = O.grad_calc(x, mu)
            assert np.array_equal(a, g[f"grad{mu}_{mx}"]) and s == g[f"grad{mu}_{mx}_shift"]


def test_layers(golden_dir):
    g = np.load(os.path.join(golden_dir, "layers.npz"))
    x, w, err = g["x"], g["w"], g["err"]
    y, ye, _ = O.act_calc(O.conv_fprop(x, w), -5 + -9)
    assert np.array_equal(y, g["conv_y"]) and ye == g["conv_y_exp"]
    e, sh = O.err_calc(O.conv_dgrad(err, w))
    assert np.array_equal(e, g["conv_e"]) and sh + -9 == g["conv_e_exp"]
    g32 = O.conv_wgrad(x, err)
    assert np.array_equal(g32, g["conv_g32"])
    assert np.array_equal(O.weight_update(w, g32, 5)[0], g["conv_w_new"])
    y, ye, _ = O.act_calc(O.conv_fprop(g["x3"], g["w3"]), -6 + -8)
    assert np.array_equal(y, g["conv1_y"]) and ye == g["conv1_y_exp"]
    g32 = O.conv_wgrad(g["x3"], err)
    assert np.array_equal(g32, g["conv1_g32"])
    assert np.array_equal(O.weight_update(g["w3"], g32, 5)[0], g["conv1_w_new"])
    a, wl, el = g["lin_a"], g["lin_w"], g["lin_err"]
    y, ye, _ = O.act_calc(O.int8_mm(a, wl.T), -3 + -9)
    assert np.array_equal(y, g["lin_y"]) and ye == g["lin_y_exp"]
    e, sh = O.err_calc(O.int8_mm(el, wl))
    assert np.array_equal(e, g["lin_e"]) and sh + -9 == g["lin_e_exp"]
    g32 = O.int8_mm(np.ascontiguousarray(el.T), a)
    assert np.array_equal(g32, g["lin_g32"])
    assert np.array_equal(O.weight_update(wl, g32, 5)[0], g["lin_w_new"])
    assert np.array_equal(O.relu_fwd(x), g["relu_y"])
    assert np.array_equal(O.maxpool_fwd(g["pool_x"]), g["pool_y"])
    assert np.array_equal(O.maxpool_bwd(g["pool_x"], g["pool_dy"]), g["pool_dx"])


def test_loss_matches_reference_float_path(golden_dir):
    """TiLoss: the oracle fixes 2**s with exp2_det; the reference used torch's float32 pow.
    The int8 errors must agree everywhere on these vectors."""
    g = np.load(os.path.join(golden_dir, "layers.npz"))
    for k in range(6):
        words = philox.random_u32_tensor(5, 0xFFFF, (64, 10))
        e, ee = O.ti_loss(g[f"loss{k}_out"], int(g[f"loss{k}_exp"]), g[f"loss{k}_tgt"], words)
        assert ee == 0
        assert np.array_equal(e, g[f"loss{k}_err"]), k


def oracle_net_record(rec):
    cfg = ["M" if c == 0 else int(c) for c in rec["cfg"]]
    B, seed, dropout, steps, mu = int(rec["B"]), int(rec["seed"]), bool(rec["dropout"]), int(rec["steps"]), int(rec["mu"])
    rng = np.random.default_rng(seed)
    shapes, cin = [], 3
    for c in cfg:
        if c != "M":
            shapes.append((c, 3, 3, cin))
            cin = c
    shapes.append((10, 512 * (32 // 2 ** cfg.count("M")) ** 2))
    weights = [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes]
    net = O.Net(cfg, weights, [xavier_exp(s) for s in shapes], dropout=dropout, mu=mu, seed=seed)
    out = {}
    for step in range(steps):
        x = synth_images(rng, B)
        tgt = rng.integers(0, 10, size=B)
        x8, xe = O.float_to_int8(x)
        y, ye = net.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=step)
        grads = net.backward(tgt, step=step)
        out[f"s{step}_out"], out[f"s{step}_out_exp"] = y, ye
        out[f"s{step}_loss_err"] = net.trace["loss_err"]
        for i in range(len(shapes)):
            out[f"s{step}_w{i}_crc"] = crc(net.w[i])
            out[f"s{step}_g{i}_crc"] = crc(grads[i].astype(np.int32))
    return out


@pytest.mark.parametrize("name", ["net_small", "net_small_nodrop", "net_vgg7_b4"])
def test_full_training_steps(golden_dir, name):
    rec = np.load(os.path.join(golden_dir, name + ".npz"))
    got = oracle_net_record(rec)
    for k, v in got.items():
        assert np.array_equal(np.asarray(v), rec[k]), k


def test_philox_known_answers():
    """Philox4x32-10 known-answer vectors of the Random123 distribution (zero, all-ones, pi digits)."""
    def run(c, k):
        return [int(v[0]) for v in philox.philox4x32_10([c[0]], [c[1]], [c[2]], [c[3]], k[0], k[1])]
    assert run((0, 0, 0, 0), (0, 0)) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    f = 0xFFFFFFFF
    assert run((f, f, f, f), (f, f)) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert run((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0)) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    # element -> word mapping: element idx uses counter (idx >> 2) and lane idx & 3
    w = philox.random_u32_tensor(5, 9, (8,), offset=2)
    blk = philox.philox4x32_10([0, 1, 2], [0, 0, 0], [9, 9, 9], [0, 0, 0], 5, 0)
    flat = [int(blk[l][b]) for b in range(3) for l in range(4)]
    assert [int(v) for v in w] == flat[2:10]
