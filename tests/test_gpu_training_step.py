"""Whole training steps through the drop-in modules (TiVGG_cifar / TiNet / Trainer) against the
oracle's layer-by-layer restatement and the reference-generated golden records."""
import os
import zlib

import numpy as np
import pytest
import torch

from oracle import niti_oracle as O
from tests.golden.make_golden import synth_images, xavier_exp

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from niti_b200 import ti_torch, ti_vgg  # noqa: E402
from niti_b200.trainer import Trainer  # noqa: E402

DEV = "cuda:0"


def crc(a):
    return np.uint32(zlib.crc32(np.ascontiguousarray(a).tobytes()))


def build(cfg, seed, dropout, fuse_relu, mu):
    rng = np.random.default_rng(seed)
    shapes, cin = [], 3
    for c in cfg:
        if c != "M":
            shapes.append((c, 3, 3, cin))
            cin = c
    shapes.append((10, cin * (32 // 2 ** cfg.count("M")) ** 2))
    weights = [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes]
    wexps = [xavier_exp(s) for s in shapes]
    ti_torch.GRAD_BITWIDTH = mu
    ti_torch.TRAINING = True
    model = ti_vgg.TiVGG_cifar(list(cfg), dropout=dropout, fuse_relu=fuse_relu)
    for l, w, e in zip(model.weighted_layers(), weights, wexps):
        l.weight = torch.from_numpy(w).to(DEV)
        l.weight_exp = ti_torch.exp_tensor(e, DEV)
    oracle = O.Net(cfg, weights, wexps, dropout=dropout, mu=mu, seed=seed)
    return model, oracle, rng


def run_steps(cfg, B, seed, dropout, steps, mu, fuse_relu, use_graph, rec=None, keep_gradients=True, prefetch=False):
    """keep_gradients: compare every layer's int32 gradient too (the default trainer zeroes them in its update launch).
    prefetch: hand every step the next batch, whose host-to-device copy then overlaps the step."""
    model, oracle, rng = build(cfg, seed, dropout, fuse_relu, mu)
    tr = Trainer(model, B, DEV, use_graph=use_graph, seed=seed, warmup_steps=1, keep_gradients=keep_gradients)
    data = []
    for step in range(steps):
        x = synth_images(rng, B)
        tgt = rng.integers(0, 10, size=B)
        data.append((x, tgt, torch.from_numpy(x).pin_memory(), torch.from_numpy(tgt).pin_memory()))
    if prefetch:
        tr.prefetch(data[0][2], data[0][3])
    for step in range(steps):
        x, tgt, xh, th = data[step]
        nxt = (data[step + 1][2], data[step + 1][3]) if prefetch and step + 1 < steps else None
        out_h, exp_h = tr.step(xh, th, prefetch_next=nxt)
        tr.sync()
        x8, xe = O.float_to_int8(x)
        want, want_e = oracle.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=step)
        grads = oracle.backward(tgt, step=step)
        assert np.array_equal(out_h.numpy(), want), f"logits differ at step {step}"
        assert int(exp_h) == want_e
        assert np.array_equal(model.loss.out_grad.cpu().numpy(), oracle.trace["loss_err"]), f"loss error differs at step {step}"
        for i, l in enumerate(model.weighted_layers()):
            if keep_gradients:
                assert np.array_equal(l.grad_int32acc.cpu().numpy(), grads[i].astype(np.int32)), f"grad {i} step {step}"
            else:
                assert int(l.grad_int32acc.abs().max()) == 0, "the update launch leaves the accumulators cleared"
            assert np.array_equal(l.weight.cpu().numpy(), oracle.w[i]), f"weights {i} step {step}"
            if rec is not None:
                assert crc(l.weight.cpu().numpy()) == rec[f"s{step}_w{i}_crc"]
                if keep_gradients:
                    assert crc(l.grad_int32acc.cpu().numpy()) == rec[f"s{step}_g{i}_crc"]
        if rec is not None:
            assert np.array_equal(out_h.numpy(), rec[f"s{step}_out"]) and int(exp_h) == rec[f"s{step}_out_exp"]
            assert np.array_equal(model.loss.out_grad.cpu().numpy(), rec[f"s{step}_loss_err"])


@pytest.mark.parametrize("name,fuse_relu,use_graph", [
    ("net_small", False, False), ("net_small", True, True), ("net_small_nodrop", True, False),
    ("net_vgg7_b4", True, False)])
def test_against_reference_golden(golden_dir, name, fuse_relu, use_graph):
    rec = np.load(os.path.join(golden_dir, name + ".npz"))
    cfg = ["M" if c == 0 else int(c) for c in rec["cfg"]]
    run_steps(cfg, int(rec["B"]), int(rec["seed"]), bool(rec["dropout"]), int(rec["steps"]), int(rec["mu"]),
              fuse_relu, use_graph, rec)


@pytest.mark.parametrize("keep_gradients", [True, False])
def test_vgg7_three_steps_graph_replay(keep_gradients):
    """Eager warm-up step, capture, then replays: the captured step must keep matching the oracle, with the
    gradients kept for comparison and in the default mode (accumulating weight-gradient kernels, bucket cleared
    by the update launch)."""
    run_steps([128, 128, "M", 256, 256, "M", 512, 512, "M"], 8, 4321, True, 3, 5, True, True, keep_gradients=keep_gradients,
              prefetch=not keep_gradients)


def test_golden_net_default_trainer_mode(golden_dir):
    rec = np.load(os.path.join(golden_dir, "net_vgg7_b4.npz"))
    cfg = ["M" if c == 0 else int(c) for c in rec["cfg"]]
    run_steps(cfg, int(rec["B"]), int(rec["seed"]), bool(rec["dropout"]), int(rec["steps"]), int(rec["mu"]),
              True, True, rec, keep_gradients=False)


@pytest.mark.parametrize("name,B", [("vgg9_wide", 2), ("vgg13", 4), (8, 2)])
def test_other_layer_lists_one_step(name, B):
    """The layer lists of the benchmark's other configurations (incl. the 64-channel VGG-13 layers) and the
    reference's depth-8 table, one step each."""
    run_steps(list(ti_vgg.cifar_cfg[name]), B, 99, True, 1, 5, True, False)


def test_stochastic_act_err_grad_rounding():
    saved = ti_torch.ACT_ROUND_METHOD, ti_torch.ERROR_ROUND_METHOD, ti_torch.GRAD_ROUND_METHOD
    try:
        ti_torch.ACT_ROUND_METHOD = ti_torch.ERROR_ROUND_METHOD = ti_torch.GRAD_ROUND_METHOD = ti_torch.StoShift
        cfg = [128, "M", 128, "M", 512, "M"]
        model, oracle, rng = build(cfg, 77, True, True, 4)
        oracle.act_mode = oracle.err_mode = oracle.grad_mode = O.STOCHASTIC
        tr = Trainer(model, 4, DEV, use_graph=False, seed=77)
        for step in range(2):
            x = synth_images(rng, 4)
            tgt = rng.integers(0, 10, size=4)
            out_h, exp_h = tr.step(torch.from_numpy(x).pin_memory(), torch.from_numpy(tgt).pin_memory())
            tr.sync()
            x8, xe = O.float_to_int8(x)
            want, want_e = oracle.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=step)
            oracle.backward(tgt, step=step)
            assert np.array_equal(out_h.numpy(), want) and int(exp_h) == want_e
            for i, l in enumerate(model.weighted_layers()):
                assert np.array_equal(l.weight.cpu().numpy(), oracle.w[i]), f"weights {i} step {step}"
    finally:
        ti_torch.ACT_ROUND_METHOD, ti_torch.ERROR_ROUND_METHOD, ti_torch.GRAD_ROUND_METHOD = saved


def test_reference_function_names_and_shift_helpers():
    """RoundShift / StoShift / PstoShift, act/err/grad_calc, int8mm, conv2d_int8 keep the reference's call shapes."""
    rng = np.random.default_rng(1)
    x = rng.integers(-100000, 100000, size=(5, 7, 3)).astype(np.int32)
    xt = torch.from_numpy(x).to(DEV)
    for s in (1, 4, 9):
        assert np.array_equal(ti_torch.RoundShift(xt, s).cpu().numpy(), O.round_shift(x, s))
        assert np.array_equal(ti_torch.PstoShift(xt, s).cpu().numpy(), O.psto_shift(x, s))
    a, e = ti_torch.act_calc(xt, 3)
    wa, we, _ = O.act_calc(x, 3)
    assert np.array_equal(a.cpu().numpy(), wa) and int(e) == we
    a, s = ti_torch.err_calc(xt)
    wa, ws = O.err_calc(x)
    assert np.array_equal(a.cpu().numpy(), wa) and int(s) == ws
    a, s = ti_torch.grad_calc(xt, 5)
    wa, ws = O.grad_calc(x, 5)
    assert np.array_equal(a.cpu().numpy(), wa) and int(s) == ws
    assert ti_torch.RangeEstimate(xt) == O.range_estimate(x)
    l, r = rng.integers(-127, 128, size=(6, 10)).astype(np.int8), rng.integers(-127, 128, size=(10, 9)).astype(np.int8)
    assert np.array_equal(ti_torch.int8mm(torch.from_numpy(l).to(DEV), torch.from_numpy(r).to(DEV)).cpu().numpy(), O.int8_mm(l, r))


def test_state_dict_roundtrip_reference_format():
    model, _, _ = build([16, "M", 32, "M", 512, "M"], 5, True, True, 5)
    sd = model.state_dict()
    assert list(sd.keys())[:2] == ["layers.0.weight", "layers.0.weight_exp"]
    # a reference checkpoint stores weight_exp as a 0-dim float tensor on the host
    ref_style = {k: (v.float().cpu() if k.endswith("weight_exp") else v.cpu()) for k, v in sd.items()}
    model2, _, _ = build([16, "M", 32, "M", 512, "M"], 6, True, True, 5)
    model2.load_state_dict(ref_style)
    for a, b in zip(model.weighted_layers(), model2.weighted_layers()):
        assert torch.equal(a.weight, b.weight) and int(a.weight_exp) == int(b.weight_exp)


def test_eval_mode_forward_and_topk_accuracy():
    """Forward-only use (main.py:82-83 with TRAINING False): TiDropout is the identity and adds nothing to the
    exponent (ti_torch.py:449-450); logits equal the oracle's network without dropout; top-k as meters.accuracy."""
    from niti_b200.meters import accuracy
    cfg = [128, "M", 128, "M", 512, "M"]
    model, _, rng = build(cfg, 5, True, True, 5)
    weights = [l.weight.cpu().numpy() for l in model.weighted_layers()]
    wexps = [int(l.weight_exp) for l in model.weighted_layers()]
    oracle = O.Net(cfg, weights, wexps, dropout=False, mu=5, seed=5)
    x = synth_images(rng, 6)
    tgt = rng.integers(0, 10, size=6)
    try:
        ti_torch.TRAINING = False
        out, out_exp = model(torch.from_numpy(x).to(DEV))
    finally:
        ti_torch.TRAINING = True
    x8, xe = O.float_to_int8(x)
    want, want_e = oracle.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=0)
    assert np.array_equal(out.cpu().numpy(), want) and int(out_exp) == want_e
    top1, top3 = accuracy(out, torch.from_numpy(tgt).to(DEV), (1, 3))
    w32 = want.astype(np.int32)
    own = w32[np.arange(6), tgt][:, None]
    for k, got in ((1, float(top1)), (3, float(top3))):
        sure = 100.0 * np.mean(((w32 >= own).sum(1) - 1) < k)        # hits whatever the order among equal logits
        maybe = 100.0 * np.mean((w32 > own).sum(1) < k)              # hits under the most favourable order
        assert sure - 1e-4 <= got <= maybe + 1e-4, (k, got, sure, maybe)


def test_vgg7_batch128_full_size_step():
    """The benchmark's own configuration (VGG-small-7, batch 128, dropout, grad bit-width 5): one graph-replayed
    step pair against the oracle (exact int8 x int8 -> int32 products through torch._int_mm on the host)."""
    O.set_backend("int_mm")
    try:
        run_steps([128, 128, "M", 256, 256, "M", 512, 512, "M"], 128, 2024, True, 2, 5, True, True, keep_gradients=False,
                  prefetch=True)
    finally:
        O.set_backend("int64")


@pytest.mark.parametrize("name,B", [("vgg9_wide", 32), ("vgg13", 128)])
def test_benchmark_configs_at_their_per_gpu_shard_size(name, B):
    """VGG-small-9 at 32 images (its global batch of 256 over 8 GPUs) and VGG-13 at 128 images (1024 over 8): one
    graph-replayed step pair each against the oracle, as for VGG-small-7 above."""
    O.set_backend("int_mm")
    try:
        run_steps(list(ti_vgg.cifar_cfg[name]), B, 2025, True, 2, 5, True, True, keep_gradients=False, prefetch=True)
    finally:
        O.set_backend("int64")


def test_checkpoint_loaded_after_graph_capture_takes_effect():
    """load_state_dict copies INTO the weight tensors, so the captured graphs (which hold their addresses) train on the
    loaded values: three steps (capture happens on the second), reload the initial weights, and the next step must equal
    the oracle's step from those initial weights with that step's random bits."""
    cfg, B, seed = [128, "M", 128, "M", 512, "M"], 4, 4242
    model, oracle, rng = build(cfg, seed, True, True, 5)
    initial = {k: v.clone() for k, v in model.state_dict().items()}
    w0 = [np.array(w) for w in oracle.w]
    tr = Trainer(model, B, DEV, use_graph=True, seed=seed, warmup_steps=1)
    for step in range(3):
        x, tgt = synth_images(rng, B), rng.integers(0, 10, size=B)
        tr.step(torch.from_numpy(x).pin_memory(), torch.from_numpy(tgt).pin_memory())
    tr.sync()
    assert tr._graphs is not None
    ptrs = [l.weight.data_ptr() for l in model.weighted_layers()]
    model.load_state_dict(initial)
    assert ptrs == [l.weight.data_ptr() for l in model.weighted_layers()], "weights must be loaded in place"
    x, tgt = synth_images(rng, B), rng.integers(0, 10, size=B)
    out_h, exp_h = tr.step(torch.from_numpy(x).pin_memory(), torch.from_numpy(tgt).pin_memory())
    tr.sync()
    fresh = O.Net(cfg, w0, oracle.w_exp, dropout=True, mu=5, seed=seed)
    x8, xe = O.float_to_int8(x)
    want, want_e = fresh.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=3)
    fresh.backward(tgt, step=3)
    assert np.array_equal(out_h.numpy(), want) and int(exp_h) == want_e
    for i, l in enumerate(model.weighted_layers()):
        assert np.array_equal(l.weight.cpu().numpy(), fresh.w[i]), f"weights {i}"


def test_a_reported_wait_expiry_is_sticky():
    """A non-zero status word after a step surfaces in StepResult.wait and the trainer then refuses further steps until
    reset_exchange() (here the word is set by hand: no kernel is made to give up)."""
    from niti_b200 import ops
    model, _, rng = build([128, "M", 128, "M", 512, "M"], 7, True, True, 5)
    tr = Trainer(model, 4, DEV, use_graph=False, seed=7)
    x, tgt = synth_images(rng, 4), rng.integers(0, 10, size=4)
    xh, th = torch.from_numpy(x).pin_memory(), torch.from_numpy(tgt).pin_memory()
    tr.step(xh, th).wait()
    ops.status_word(DEV).copy_(torch.tensor([9, 1, 1, 0], dtype=torch.int32))
    try:
        res = tr.step(xh, th)
        with pytest.raises(RuntimeError, match="gave up waiting for rank 1"):
            res.wait()
        with pytest.raises(RuntimeError, match="no further steps"):
            tr.step(xh, th)
        tr.reset_exchange()
        tr.step(xh, th).wait()
    finally:
        ops.status_word(DEV).zero_()
