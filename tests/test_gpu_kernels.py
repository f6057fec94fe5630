"""Kernel-level parity: every C-ABI entry point against the CPU oracle, bit-exact."""
import numpy as np
import pytest
import torch

from oracle import niti_oracle as O, philox

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from niti_b200 import ops  # noqa: E402

DEV = "cuda:0"


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def rnd8(rng, shape, lo=-127, hi=128):
    return rng.integers(lo, hi, size=shape).astype(np.int8)


def describe_mismatch(got, want):
    bad = np.argwhere(got != want)
    return f"{len(bad)} of {got.size} differ; first {bad[:5].tolist()} got {got[tuple(bad[0])]} want {want[tuple(bad[0])]}" \
        if len(bad) else "equal"


def assert_same(got_t, want, what):
    got = got_t.cpu().numpy()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.array_equal(got, want), f"{what}: {describe_mismatch(got, want.astype(got.dtype))}"
    ops.check_status(DEV)


# ----------------------------------------------------------------------------- GEMM
GEMM_CASES = [
    # M, N, K, trans_a, trans_b
    (128, 128, 128, 0, 1), (256, 128, 256, 0, 1), (384, 256, 512, 0, 1), (200, 144, 272, 0, 1),
    (1024, 512, 1024, 0, 1), (128, 128, 128, 0, 0), (256, 256, 384, 0, 0), (200, 144, 272, 0, 0),
    (128, 128, 128, 1, 0), (256, 384, 512, 1, 0), (208, 144, 272, 1, 0), (128, 128, 256, 1, 1),
    # reduction or output narrower than one 128-byte TMA box (the patch-matrix GEMMs of the first layer)
    (256, 128, 32, 0, 1), (300, 64, 48, 0, 1), (128, 32, 4096, 1, 0), (64, 32, 640, 1, 0),
    # CUDA-core shapes of the 10-class FC layer: forward, error, gradient
    (64, 10, 8192, 0, 1), (64, 8192, 10, 0, 0), (10, 8192, 64, 1, 0), (7, 5, 33, 0, 1), (7, 5, 33, 1, 1),
]


@pytest.mark.parametrize("M,N,K,ta,tb", GEMM_CASES)
def test_gemm(M, N, K, ta, tb):
    rng = np.random.default_rng(M * 7 + N * 3 + K + ta * 2 + tb)
    a = rnd8(rng, (K, M) if ta else (M, K))
    b = rnd8(rng, (N, K) if tb else (K, N))
    want = O.int8_mm(a.T if ta else a, b.T if tb else b)
    c32, mx = ops.gemm_acc(cu(a), cu(b), bool(ta), bool(tb))
    assert_same(c32, want.astype(np.int32), "gemm accumulators")
    assert int(mx.item()) == int(np.abs(want).max())


# ----------------------------------------------------------------------------- convolution
CONV_CASES = [
    # N, H, W, C, K
    (2, 8, 8, 128, 128), (4, 32, 32, 128, 128), (3, 16, 16, 128, 256), (5, 8, 8, 256, 512), (9, 4, 4, 256, 128),
    (2, 12, 20, 128, 144), (1, 2, 2, 128, 128), (16, 2, 2, 128, 128),
    (4, 32, 32, 3, 128), (3, 8, 8, 3, 32), (2, 8, 8, 16, 32), (2, 6, 10, 5, 7),
    # channel counts that are multiples of 16 but not of 128: partial 128-byte blocks, TMA zero fill
    (6, 16, 16, 64, 64), (3, 8, 8, 192, 64), (2, 8, 8, 48, 80), (4, 8, 8, 64, 320),
]


@pytest.mark.parametrize("N,H,W,C,K", CONV_CASES)
def test_conv_fprop(N, H, W, C, K):
    rng = np.random.default_rng(N + H * 3 + C * 5 + K)
    x, w = rnd8(rng, (N, H, W, C)), rnd8(rng, (K, 3, 3, C))
    want = O.conv_fprop(x, w)
    y32, mx = ops.conv_fprop_acc(cu(x), cu(w))
    assert_same(y32, want.astype(np.int32), "conv fprop accumulators")
    assert int(mx.item()) == int(np.abs(want).max())


@pytest.mark.parametrize("N,H,W,C,K", CONV_CASES)
def test_conv_dgrad(N, H, W, C, K):
    rng = np.random.default_rng(N + H * 3 + C * 5 + K + 1)
    err, w = rnd8(rng, (N, H, W, K)), rnd8(rng, (K, 3, 3, C))
    want = O.conv_dgrad(err, w)
    e32, mx = ops.conv_dgrad_acc(cu(err), cu(w))
    assert_same(e32, want.astype(np.int32), "conv dgrad accumulators")
    assert int(mx.item()) == int(np.abs(want).max())


@pytest.mark.parametrize("N,H,W,C,K", CONV_CASES)
@pytest.mark.parametrize("tma_reduce", [True, False])
def test_conv_wgrad(N, H, W, C, K, tma_reduce):
    rng = np.random.default_rng(N + H * 3 + C * 5 + K + 2)
    x, err = rnd8(rng, (N, H, W, C)), rnd8(rng, (N, H, W, K))
    want = O.conv_wgrad(x, err)
    old = ops.set_wgrad_tma_reduce(tma_reduce)
    try:
        g32, mx = ops.conv_wgrad_acc(cu(x), cu(err))
        assert_same(g32, want.astype(np.int32), "conv wgrad accumulators")
        assert int(mx.item()) == int(np.abs(want).max())
    finally:
        ops.set_wgrad_tma_reduce(old)


def test_conv_rejects_stride():
    x, w = cu(np.zeros((1, 8, 8, 128), np.int8)), cu(np.zeros((128, 3, 3, 128), np.int8))
    with pytest.raises(RuntimeError):
        ops.conv_fprop_acc(x, w, pad=1, stride=2)


# ----------------------------------------------------------------------------- requantisation
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("mx", [0, 1, 100, 127, 128, 129, 1000, 65536, 65537, 3000000, 2 ** 30])
def test_requant_act(mode, mx):
    rng = np.random.default_rng(mx % 1000 + mode)
    n = 16 * 1000 + 7
    acc = rng.integers(-mx, mx + 1, size=n).astype(np.int32)
    acc[5] = mx
    acc[n - 1] = -mx
    words = philox.random_u32_tensor(99, 3, (n,), offset=8)
    want, want_exp, _ = O.act_calc(acc, -4, mode, words)
    a = cu(acc)
    seed = ops.seed_tensor(99, DEV)
    e_in = torch.tensor(-4, dtype=torch.int32, device=DEV)
    out, e_out, sh = ops.requant(a, ops.absmax(a), ops.CALC_ACT, 7, mode, seed, 3, 8, exp_a=e_in, want_shift=True)
    assert_same(out, want, f"requant mode {mode} max {mx}")
    assert int(e_out.item()) == want_exp


def test_requant_unaligned_rng_offset_and_relu():
    rng = np.random.default_rng(5)
    acc = rng.integers(-50000, 50000, size=4099).astype(np.int32)
    words = philox.random_u32_tensor(7, 1, acc.shape, offset=13)
    want, sh = O.err_calc(acc, O.STOCHASTIC, words)
    a = cu(acc)
    out, e_out, s = ops.requant(a, ops.absmax(a), ops.CALC_ERR, 7, 1, ops.seed_tensor(7, DEV), 1, 13, relu=True, want_shift=True)
    assert_same(out, np.maximum(want, 0), "requant + relu")
    assert int(s.item()) == sh and int(e_out.item()) == sh


@pytest.mark.parametrize("mu", [5, 4, 3])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_update(mu, mode):
    rng = np.random.default_rng(mu + mode)
    K, R, S, C = 32, 3, 3, 16
    w = rnd8(rng, (K, R, S, C))
    for mx in (0, 3, 31, 40000):
        g = rng.integers(-mx, mx + 1, size=w.shape).astype(np.int32)
        words = philox.random_u32_tensor(21, 2, w.shape)
        want_w, _, _ = O.weight_update(w, g, mu, mode, words)
        w_dev, g_dev = cu(w), cu(g)
        ops.update(w_dev, g_dev, ops.absmax(g_dev), mu, mode, ops.seed_tensor(21, DEV), 2)
        assert_same(w_dev, want_w, f"updated weights mx={mx}")


# ----------------------------------------------------------------------------- memory-bound layers
@pytest.mark.parametrize("shape", [(4, 32, 32, 128), (3, 8, 8, 16), (2, 6, 10, 5), (1, 2, 2, 512)])
def test_maxpool_relu(shape):
    rng = np.random.default_rng(sum(shape))
    x = np.maximum(rnd8(rng, shape, -128, 128), -20 if shape[3] == 5 else 0).astype(np.int8)  # many ties
    y = ops.maxpool_fwd(cu(x))
    assert_same(y, O.maxpool_fwd(x), "maxpool fwd")
    dy = rnd8(rng, y.shape)
    assert_same(ops.maxpool_bwd(cu(x), cu(dy)), O.maxpool_bwd(x, dy), "maxpool bwd")
    assert_same(ops.maxpool_bwd(cu(x), cu(dy), relu_mask=True), O.relu_bwd(x, O.maxpool_bwd(x, dy)), "maxpool bwd + relu mask")
    x2 = rnd8(rng, shape, -128, 128)
    assert_same(ops.relu_fwd(cu(x2)), O.relu_fwd(x2), "relu fwd")
    e = rnd8(rng, shape)
    assert_same(ops.relu_bwd(cu(x2), cu(e)), O.relu_bwd(x2, e), "relu bwd")


def test_maxpool_generic_window():
    rng = np.random.default_rng(3)
    x = rnd8(rng, (2, 9, 9, 4), -5, 6)
    assert_same(ops.maxpool_fwd(cu(x), 3, 2), O.maxpool_fwd(x, 3, 2), "maxpool 3/2 fwd")
    dy = rnd8(rng, (2, 4, 4, 4), -30, 31)
    assert_same(ops.maxpool_bwd(cu(x), cu(dy), 3, 2), O.maxpool_bwd(x, dy, 3, 2), "maxpool 3/2 bwd")
    assert_same(ops.maxpool_bwd(cu(x), cu(dy), 3, 2, True), O.relu_bwd(x, O.maxpool_bwd(x, dy, 3, 2)), "maxpool 3/2 bwd + relu mask")


def test_dropout():
    rng = np.random.default_rng(8)
    x = rnd8(rng, (16, 8192))
    mask = O.dropout_mask(1234, 0xFFFE, 8192)
    assert_same(ops.dropout(cu(x), ops.seed_tensor(1234, DEV), 0xFFFE), x * mask, "dropout")


def test_loss_golden_and_oracle(golden_dir):
    import os
    g = np.load(os.path.join(golden_dir, "layers.npz"))
    for k in range(6):
        out, e, tgt = g[f"loss{k}_out"], int(g[f"loss{k}_exp"]), g[f"loss{k}_tgt"]
        err = ops.loss_err(cu(out), torch.tensor(e, dtype=torch.int32, device=DEV), cu(tgt.astype(np.int64)),
                           ops.seed_tensor(5, DEV))
        assert_same(err, g[f"loss{k}_err"], f"loss vs reference golden {k}")
    rng = np.random.default_rng(77)
    for e in range(-12, 6):
        B = 128
        out = rnd8(rng, (B, 10), -127 // (1 + (e % 3) * 5), 128 // (1 + (e % 3) * 5))
        tgt = rng.integers(0, 10, size=B)
        words = philox.random_u32_tensor(40 + e, 0xFFFF, (B, 10), offset=30)
        want, _ = O.ti_loss(out, e, tgt, words)
        err = ops.loss_err(cu(out), torch.tensor(e, dtype=torch.int32, device=DEV), cu(tgt.astype(np.int64)),
                           ops.seed_tensor(40 + e, DEV), sample_offset=3)
        assert_same(err, want, f"loss exp={e}")


def test_quantize_input():
    from tests.golden.make_golden import synth_images
    rng = np.random.default_rng(11)
    for scale in (1.0, 0.3, 4.0, 2.0 / 2.6402):
        x = (synth_images(rng, 8) * np.float32(scale)).astype(np.float32)
        want8, want_e = O.float_to_int8(x)
        x8, e = ops.quantize_input(cu(x))
        assert_same(x8, np.ascontiguousarray(want8.transpose(0, 2, 3, 1)), "input quantisation")
        assert int(e.item()) == want_e


# ----------------------------------------------------------------------------- fused conv + requantisation
@pytest.mark.parametrize("N,H,W,C,K", [(4, 32, 32, 128, 128), (3, 16, 16, 128, 256), (5, 8, 8, 256, 512), (2, 12, 20, 128, 144),
                                        (4, 32, 32, 3, 128), (9, 4, 4, 256, 128), (6, 16, 16, 64, 64), (2, 8, 8, 48, 80)])
@pytest.mark.parametrize("mode,relu", [(0, True), (0, False), (1, False), (2, True)])
@pytest.mark.parametrize("parking", [False, True])
def test_conv_fused_requant(N, H, W, C, K, mode, relu, parking):
    """Fused conv + requantisation against conv + act_calc / err_calc of the oracle.
    parking=False: predicted-shift kernels; the first call mispredicts (state starts at 0) and must
    redo, the second call predicts right.  parking=True: accumulators parked in tensor memory across
    a grid barrier, exact in one launch (all of these shapes are small enough)."""
    old = ops.set_accumulator_parking(parking)
    try:
        _fused_case(N, H, W, C, K, mode, relu, parking and C * 9 > 32)
    finally:
        ops.set_accumulator_parking(old)


def _fused_case(N, H, W, C, K, mode, relu, parked):
    rng = np.random.default_rng(N + H + C + K + mode)
    x, w = rnd8(rng, (N, H, W, C)), rnd8(rng, (K, 3, 3, C))
    seed = ops.seed_tensor(31, DEV)
    acc = O.conv_fprop(x, w)
    words = philox.random_u32_tensor(31, 5, acc.shape, offset=64)
    want, want_e, want_s = O.act_calc(acc, -3 + -9, mode, words)
    if relu:
        want = O.relu_fwd(want)
    st = ops.new_requant_state(DEV)
    ea, eb = torch.tensor(-3, dtype=torch.int32, device=DEV), torch.tensor(-9, dtype=torch.int32, device=DEV)
    for call in range(2):
        y8, e, s = ops.conv_fprop_fused(cu(x), cu(w), st, 1, mode, seed, 5, 64, relu, ea, eb)
        assert_same(y8, want, f"fused fprop call {call}")
        assert int(e.item()) == want_e and int(s.item()) == want_s
        redo_now, redos = (0, 0) if parked else (1 if (call == 0 and want_s != 0) else 0, 1 if want_s != 0 else 0)
        assert st.tolist()[1:6] == [0, redo_now, redos, 0, 0] and st.tolist()[0] == want_s
    if C % 16 == 0 and K % 16 == 0:
        err = rnd8(rng, (N, H, W, K))
        acc = O.conv_dgrad(err, w)
        words = philox.random_u32_tensor(31, 6, acc.shape, offset=128)
        want, want_s = O.err_calc(acc, mode, words)
        st = ops.new_requant_state(DEV)
        for call in range(2):
            e8, e, s = ops.conv_dgrad_fused(cu(err), cu(w), st, 1, mode, seed, 6, 128, ea, eb)
            assert_same(e8, want, f"fused dgrad call {call}")
            assert int(s.item()) == want_s and int(e.item()) == want_s - 12


# ----------------------------------------------------------------------------- single-CTA variants
@pytest.mark.parametrize("pairs", [0, 3])
def test_cta_pair_and_single_cta_kernels_match(pairs):
    """CTA pairs (cta_group::2) are the default for GEMMs and optional for convolutions; with the option
    switch at 0 (one CTA per tile everywhere) and at 3 (pairs wherever shapes allow) the integers must be the same."""
    old = ops.set_cta_pairs(pairs)
    try:
        rng = np.random.default_rng(12)
        for (M, N, K, ta, tb) in [(384, 256, 512, 0, 1), (256, 256, 384, 0, 0), (256, 384, 512, 1, 0)]:
            a = rnd8(rng, (K, M) if ta else (M, K))
            b = rnd8(rng, (N, K) if tb else (K, N))
            c32, mx = ops.gemm_acc(cu(a), cu(b), bool(ta), bool(tb))
            assert_same(c32, O.int8_mm(a.T if ta else a, b.T if tb else b).astype(np.int32), "gemm, single CTA")
        x, w, err = rnd8(rng, (5, 8, 8, 256)), rnd8(rng, (512, 3, 3, 256)), rnd8(rng, (5, 8, 8, 512))
        assert_same(ops.conv_fprop_acc(cu(x), cu(w))[0], O.conv_fprop(x, w).astype(np.int32), "conv fprop, single CTA")
        assert_same(ops.conv_dgrad_acc(cu(err), cu(w))[0], O.conv_dgrad(err, w).astype(np.int32), "conv dgrad, single CTA")
        for parking in (False, True):
            oldp = ops.set_accumulator_parking(parking)
            st = ops.new_requant_state(DEV)
            want, want_e, _ = O.act_calc(O.conv_fprop(x, w), 0)
            for _ in range(2):
                y8, e, s = ops.conv_fprop_fused(cu(x), cu(w), st, 1, 0, None, 0, 0, False,
                                                torch.zeros((), dtype=torch.int32, device=DEV), None)
                assert_same(y8, want, f"fused conv, pairs={pairs}, parking={parking}")
            ops.set_accumulator_parking(oldp)
    finally:
        ops.set_cta_pairs(old)


# ----------------------------------------------------------------------------- fused classifier head
HEAD_CASES = [
    # B, F, J, dropout, (act, err, grad) rounding, exp_x, exp_w, sample_offset
    (128, 8192, 10, True, (0, 0, 2), -5, -8, 0),
    (128, 8192, 10, True, (1, 1, 1), -9, -9, 256),
    (4, 512, 10, True, (0, 0, 2), -6, -7, 0),
    (37, 2048, 16, False, (0, 1, 0), -2, -5, 37),
    (200, 1024, 3, True, (2, 2, 2), -12, -10, 0),
    (300, 160, 10, False, (0, 0, 2), 0, -3, 11),
]


@pytest.mark.gpu
@pytest.mark.parametrize("B,F,J,dropout,modes,exp_x,exp_w,offset", HEAD_CASES)
def test_fc_head_one_kernel_matches_the_separate_calls(B, F, J, dropout, modes, exp_x, exp_w, offset):
    """The one-kernel classifier head against the chain of calls it replaces (each of which is checked
    against the oracle above): dropout, FC forward, requantise, loss, FC error-backward, requantise,
    weight gradient, update, dropout backward."""
    rng = np.random.default_rng(B * 7 + F + J)
    act_mode, err_mode, grad_mode = modes
    x = cu(rnd8(rng, (B, F), 0, 128))
    w = cu(rnd8(rng, (J, F), -40, 41))
    tgt = cu(rng.integers(0, J, size=B).astype(np.int64))
    seed = ops.seed_tensor(99 + B, DEV)
    ex = torch.tensor(exp_x, dtype=torch.int32, device=DEV)
    ew = torch.tensor(exp_w, dtype=torch.int32, device=DEV)
    stream = 16 * 6
    assert ops.fc_head_supported(B, F, J)

    xd = ops.dropout(x, seed, 0xFFFE) if dropout else x
    e_in = ex + 1 if dropout else ex
    acc, mx = ops.gemm_acc(xd, w, trans_b=True)
    out8, out_exp, _ = ops.requant(acc, mx, ops.CALC_ACT, 7, act_mode, seed, stream, offset * J, exp_a=e_in, exp_b=ew)
    err8 = ops.loss_err(out8, out_exp, tgt, seed, 0xFFFF, offset)
    acc2, mx2 = ops.gemm_acc(err8, w)
    zero = torch.zeros((), dtype=torch.int32, device=DEV)
    e8, err_exp, _ = ops.requant(acc2, mx2, ops.CALC_ERR, 7, err_mode, seed, stream + 1, offset * F, exp_a=zero, exp_b=ew)
    if dropout:
        e8 = ops.dropout(e8, seed, 0xFFFE)
    g32, gm = ops.gemm_acc(err8, xd, trans_a=True)
    w_sep = w.clone()
    ops.update(w_sep, g32, gm, 5, grad_mode, seed, stream + 2)

    for update in (False, True):
        w_one = w.clone()
        got = ops.fc_head_train(x, ex, w_one, ew, tgt, seed, stream, dropout=dropout, act_mode=act_mode, err_mode=err_mode,
                                grad_mode=grad_mode, mu=5, update=update, sample_offset=offset)
        o8, oexp, l8, b8, bexp, gg, gmax = got
        assert_same(o8, out8.cpu().numpy(), "head: logits")
        assert int(oexp) == int(out_exp)
        assert_same(l8, err8.cpu().numpy(), "head: loss error")
        assert_same(b8, e8.cpu().numpy(), "head: error to the features")
        assert int(bexp) == int(err_exp)
        assert_same(gg, g32.cpu().numpy(), "head: weight gradient")
        assert int(gmax) == int(gm)
        assert_same(w_one, (w_sep if update else w).cpu().numpy(), f"head: weights, update={update}")


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("count", [1, 7, 19])
def test_update_multi_matches_layer_by_layer(mode, count):
    """One launch for all layers against absmax + update per layer (the latter is checked against the oracle above)."""
    rng = np.random.default_rng(100 * mode + count)
    sizes = [int(rng.integers(1, 40000)) * (4 if i % 3 else 1) + (i % 3 == 0) * 3 for i in range(count)]
    sizes[0] = 128 * 3 * 3 * 256
    seed = ops.seed_tensor(321, DEV)
    ws, gs, want = [], [], []
    for i, n in enumerate(sizes):
        w = cu(rnd8(rng, (n,)))
        scale = [1, 50, 4000, 300000][i % 4]
        g = cu((rng.integers(-scale, scale + 1, size=n) * (i % 5 != 4)).astype(np.int32))
        ref = w.clone()
        mx = ops.absmax(g)
        ops.update(ref, g, mx, 5, mode, seed, 16 * i + 2)
        ws.append(w); gs.append(g); want.append((ref, mx))
    got_mx = ops.update_multi(ws, gs, [16 * i + 2 for i in range(count)], 5, mode, seed, want_max=True)
    for i in range(count):
        assert_same(ws[i], want[i][0].cpu().numpy(), f"update_multi layer {i} of {count}, n={sizes[i]}")
        assert int(got_mx[i]) == int(want[i][1])


@pytest.mark.gpu
def test_update_multi_can_clear_the_accumulators():
    rng = np.random.default_rng(5)
    seed = ops.seed_tensor(1, DEV)
    ws = [cu(rnd8(rng, (n,))) for n in (4096, 1003)]
    gs = [cu(rng.integers(-900, 900, size=n).astype(np.int32)) for n in (4096, 1003)]
    want = []
    for w, g in zip(ws, gs):
        ref = w.clone()
        ops.update(ref, g, ops.absmax(g), 5, 2, seed, 2)
        want.append(ref.cpu().numpy())
    ops.update_multi(ws, gs, [2, 2], 5, 2, seed, clear=True)
    for w, g, r in zip(ws, gs, want):
        assert_same(w, r, "update_multi with clear: weights")
        assert int(g.abs().max()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_dp_update_with_one_rank_equals_update_multi(mode):
    """niti_dp_update_i8 with world = 1 (all three barriers, slice = whole layer) against niti_update_multi_i8 with
    clearing; three launches in a row, so the barrier sequence numbers carry over.  The multi-rank arithmetic is
    checked on two GPUs in test_gpu_dp_peer.py."""
    rng = np.random.default_rng(40 + mode)
    sizes = [128 * 3 * 3 * 3, 128 * 3 * 3 * 128, 4 * 1001, 10 * 8192]
    seed = ops.seed_tensor(99, DEV)
    w_offs, off = [], 0
    for n in sizes:
        w_offs.append(off)
        off += (n + 255) // 256 * 256
    g_off = off
    g_offs, goff = [], 0
    for n in sizes:
        g_offs.append(goff)
        goff += n
    x_off = (g_off + 4 * goff + 255) // 256 * 256
    arena = torch.zeros(x_off + ops.dp_exchange_bytes(), dtype=torch.uint8, device=DEV)
    ws = [arena[o:o + n].view(torch.int8) for o, n in zip(w_offs, sizes)]
    bucket = arena[g_off:g_off + 4 * goff].view(torch.int32)
    gs = [bucket[o:o + n] for o, n in zip(g_offs, sizes)]
    items = [(w_offs[i], g_offs[i], sizes[i], 16 * i + 2) for i in range(len(sizes))]
    base = arena.data_ptr()
    for w in ws:
        w.copy_(cu(rnd8(rng, (w.numel(),))))
    for step in range(3):
        for i, g in enumerate(gs):
            scale = [3, 700, 90000, 0][(i + step) % 4]
            g.copy_(cu(rng.integers(-scale, scale + 1, size=g.numel()).astype(np.int32)))
        ref_w = [w.clone() for w in ws]
        ref_g = [g.clone() for g in gs]
        want_mx = ops.update_multi(ref_w, ref_g, [it[3] for it in items], 5, mode, seed, want_max=True, clear=True)
        got_mx = torch.zeros(len(sizes), dtype=torch.int32, device=DEV)
        ops.dp_update(items, 0, 1, [base], [base + g_off], [base + x_off], 5, mode, seed, DEV, maxabs=got_mx)
        ops.check_status(DEV)
        for i in range(len(sizes)):
            assert_same(ws[i], ref_w[i].cpu().numpy(), f"dp_update step {step} layer {i}")
            assert int(got_mx[i]) == int(want_mx[i])
        assert int(bucket.abs().max()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,W,C,K", [(8, 16, 16, 128, 128), (4, 8, 8, 256, 128), (3, 10, 6, 64, 144)])
def test_conv_wgrad_accumulates_into_the_gradient(N, H, W, C, K):
    """g32 += weight gradient: twice the same call gives base + 2 * gradient (gradient accumulation over micro-batches)."""
    rng = np.random.default_rng(N + H + C)
    x, e = rnd8(rng, (N, H, W, C)), rnd8(rng, (N, H, W, K))
    assert ops.conv_wgrad_accumulate_supported(C, K, 3, 3, 1)
    base = rng.integers(-1000, 1000, size=(K, 3, 3, C)).astype(np.int32)
    g = cu(base.copy())
    ops.conv_wgrad_accumulate(cu(x), cu(e), g)
    ops.conv_wgrad_accumulate(cu(x), cu(e), g)
    want = O.conv_wgrad(x, e, 3, 3, 1)
    assert_same(g, (base.astype(np.int64) + 2 * want).astype(np.int32), "accumulating weight gradient")


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,W,C,K,parking", [(8, 16, 16, 128, 256, True), (4, 8, 8, 256, 128, True), (16, 32, 32, 128, 128, False),
                                               (3, 10, 6, 144, 64, True)])
def test_conv_dgrad_fused_applies_relu_mask(N, H, W, C, K, parking):
    """Error-backward + requantisation + the backward of the ReLU in front of the layer in one kernel: the shift is
    that of the UNMASKED error, the mask zeroes where the layer's forward input was not positive."""
    rng = np.random.default_rng(N * H + C)
    err, w = rnd8(rng, (N, H, W, K)), rnd8(rng, (K, 3, 3, C))
    x = np.maximum(rnd8(rng, (N, H, W, C)), 0)  # a ReLU output: about half zeros
    old = ops.set_accumulator_parking(parking)
    try:
        ea = torch.zeros((), dtype=torch.int32, device=DEV)
        st = ops.new_requant_state(DEV)
        for _ in range(2):  # second call: the shift prediction of the streaming kernel is right
            got, _, shift = ops.conv_dgrad_fused(cu(err), cu(w), st, 1, 0, None, 0, 0, ea, ea, relu_mask=cu(x))
    finally:
        ops.set_accumulator_parking(old)
    acc = O.conv_dgrad(err, w, 1)
    want, s = O.err_calc(acc)
    assert int(shift) == s
    assert_same(got, np.where(x > 0, want, 0).astype(np.int8), "dgrad + requant + relu mask")


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,W,C,K,masked", [(3, 16, 16, 128, 64, False), (2, 8, 8, 48, 144, True), (5, 32, 32, 16, 32, True),
                                              (1, 4, 4, 272, 16, False)])
def test_conv_dgrad_fused_steps_down_one_shift_from_side_codes(N, H, W, C, K, masked):
    """The streaming kernel narrows with the shift it guessed.  With side memory a guess ONE too high is repaired from
    two extra bits per output instead of a second contraction: state[2] reads 2 (not 1), state[3] (second contractions)
    does not grow, the guess stays, and the output is the oracle's for the true shift.  After 12 step-downs in a row the
    guess follows."""
    rng = np.random.default_rng(N * 131 + C)
    w = rnd8(rng, (K, 3, 3, C))
    big = rnd8(rng, (N, H, W, K))
    small = (big.astype(np.int32) // 2).astype(np.int8)  # every sum about half as large: one bit less
    x = np.maximum(rnd8(rng, (N, H, W, C)), 0)
    mask = cu(x) if masked else None
    want = {}
    for name, e in (("big", big), ("small", small)):
        y, sft = O.err_calc(O.conv_dgrad(e, w, 1))
        want[name] = (np.where(x > 0, y, 0).astype(np.int8) if masked else y, sft)
    assert want["small"][1] == want["big"][1] - 1 and want["small"][1] >= 1
    old = ops.set_accumulator_parking(False)
    try:
        nbytes = ops.conv_dgrad_side_bytes(N, H, W, C, K, 3, 3, 1)
        assert nbytes == N * H * W * C // 4
        side = torch.full((nbytes,), 0xA5, dtype=torch.uint8, device=DEV)
        ea = torch.zeros((), dtype=torch.int32, device=DEV)
        st = ops.new_requant_state(DEV)

        def run(name):
            got, _, shift = ops.conv_dgrad_fused(cu(big if name == "big" else small), cu(w), st, 1, 0, None, 0, 0, ea, ea,
                                                 relu_mask=mask, side=side)
            assert int(shift) == want[name][1]
            assert_same(got, want[name][0], f"dgrad + requant ({name})")
            v = st.tolist()
            return v[0], v[2] & 3, (v[2] >> 4) & 15, v[2] >> 8, v[3]

        S = want["big"][1]
        assert run("big") == (S, 1, 0, 0, 1)        # guess 0: contracted again
        assert run("big") == (S, 0, 0, 0, 1)        # right
        assert run("small") == (S, 2, 1, 1, 1)      # one too high: stepped down, the guess stays
        assert run("big") == (S, 0, 0, 1, 1)
        for i in range(11):
            assert run("small") == (S, 2, i + 1, i + 2, 1)
        assert run("small") == (S - 1, 2, 0, 13, 1)  # the twelfth in a row: the guess follows
        assert run("small") == (S - 1, 0, 0, 13, 1)
        assert run("big") == (S, 1, 0, 13, 2)        # one too LOW cannot be repaired: contracted again
    finally:
        ops.set_accumulator_parking(old)


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,W,C,K", [(4, 32, 32, 3, 128), (3, 8, 8, 3, 64), (130, 32, 32, 3, 128), (2, 6, 10, 2, 32)])
def test_first_layer_weight_gradient_from_the_forward_patch_matrix(N, H, W, C, K):
    """A thin layer's forward call leaves its patch matrix in caller-owned scratch; the weight gradient computed from
    it equals the oracle's (and the one computed from the input)."""
    rng = np.random.default_rng(N + 7 * K)
    x, w, err = rnd8(rng, (N, H, W, C)), rnd8(rng, (K, 3, 3, C)), rnd8(rng, (N, H, W, K))
    nbytes = ops.conv_fprop_scratch_bytes(N, H, W, C, K, 3, 3)
    assert nbytes >= N * H * W * 32
    buf = torch.full((nbytes,), 0x5A, dtype=torch.uint8, device=DEV)
    ea = torch.zeros((), dtype=torch.int32, device=DEV)
    st = ops.new_requant_state(DEV)
    y, _, shift = ops.conv_fprop_fused(cu(x), cu(w), st, 1, 0, None, 0, 0, True, ea, ea, scratch_buf=buf)
    want_y, s = O.act_calc(O.conv_fprop(x, w, 1), 0)[0], None
    assert_same(y, np.maximum(want_y, 0).astype(np.int8), "thin forward with caller scratch")
    g, mx = ops.conv_wgrad_from_patches(buf, cu(err), C)
    want = O.conv_wgrad(x, err, 3, 3, 1)
    assert_same(g, want, "weight gradient from patches")
    assert int(mx) == int(np.abs(want).max())
    g2, _ = ops.conv_wgrad_acc(cu(x), cu(err), 3, 3, 1)
    assert torch.equal(g, g2)


@pytest.mark.gpu
@pytest.mark.parametrize("shapes", [
    [(128, 8, 8, 512, 512), (128, 8, 8, 256, 512)],                       # a VGG-small-7 pair: one wave, equal shares
    [(32, 16, 16, 256, 256), (32, 16, 16, 128, 256), (32, 32, 32, 128, 128)],
    [(3, 8, 8, 16, 32), (2, 4, 4, 144, 16), (5, 16, 16, 48, 272), (1, 2, 2, 16, 16)],   # ragged, partial tiles
    [(4, 8, 8, 64, 64)]])
def test_weight_gradients_of_several_layers_in_one_launch(shapes):
    """Every layer's gradient is ADDED into its own buffer by one launch; the sums equal the oracle's plus what the
    buffers held."""
    assert len(shapes) <= ops.conv_wgrad_accumulate_multi_max()
    rng = np.random.default_rng(len(shapes) * 17 + shapes[0][0])
    jobs, want = [], []
    for (N, H, W, C, K) in shapes:
        x, err = rnd8(rng, (N, H, W, C)), rnd8(rng, (N, H, W, K))
        base = rng.integers(-1000, 1000, size=(K, 3, 3, C)).astype(np.int32)
        g = cu(base)
        jobs.append((cu(x), cu(err), g, 3, 3, 1))
        want.append(base + O.conv_wgrad(x, err, 3, 3, 1))
    ops.conv_wgrad_accumulate_multi(jobs)
    ops.check_status(DEV)
    for i, (job, w) in enumerate(zip(jobs, want)):
        assert_same(job[2], w, f"layer {i} of {len(shapes)}")


@pytest.mark.gpu
def test_bounded_grid_barrier_gives_up_and_reports():
    """A grid barrier that cannot be met (one block, two expected) returns after its 0.5 s limit with a status code;
    nothing traps or hangs and the device keeps working afterwards."""
    import time
    from niti_b200._lib import lib, check
    scratch = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    check(lib.niti_selftest_barrier_timeout(scratch.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream), "selftest")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    s = status.tolist()
    assert s[0] == 8 and s[1] == 0 and s[2] == 2 and s[3] == 0, s
    assert 0.3 < dt < 5.0, dt
    x = cu(np.arange(64, dtype=np.int32) - 32)            # the context is alive
    assert int(ops.absmax(x)) == 32


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,W,C,K,mode", [
    (128, 16, 16, 256, 256, 0), (128, 8, 8, 512, 512, 0), (32, 16, 16, 128, 256, 0),   # VGG shapes that park at these batches
    (3, 16, 16, 32, 48, 0), (5, 8, 8, 144, 16, 0), (7, 4, 4, 64, 272, 0), (2, 2, 2, 16, 32, 0), (6, 8, 16, 128, 128, 1)])
def test_conv_fprop_fused_with_pool_in_the_same_launch(N, H, W, C, K, mode):
    """conv + act_calc + ReLU + 2x2 max pooling in one kernel against the oracle's four separate steps; the unpooled
    tensor is written too (the pool's backward routes by it)."""
    assert ops.conv_fprop_pool_fused_supported(N, H, W, C, K, 3, 3, 1)
    rng = np.random.default_rng(N * 7 + H + C + K)
    x, w = rnd8(rng, (N, H, W, C)), rnd8(rng, (K, 3, 3, C))
    seed = ops.seed_tensor(77, DEV)
    ea = torch.full((), -3, dtype=torch.int32, device=DEV)
    st = ops.new_requant_state(DEV)
    for _ in range(2):
        y8, yp, exp_out, shift = ops.conv_fprop_pool_fused(cu(x), cu(w), st, 1, mode, seed, 5, 0, True, ea, ea)
    acc = O.conv_fprop(x, w)
    words = philox.random_u32_tensor(77, 5, acc.shape) if mode == 1 else None
    want, want_e, _ = O.act_calc(acc, -6, mode, words)
    want = O.relu_fwd(want)
    assert int(exp_out) == want_e
    assert_same(y8, want, "fused conv + relu")
    assert_same(yp, O.maxpool_fwd(want), "pooled output of the same launch")


@pytest.mark.gpu
def test_conv_fprop_pool_fusion_is_refused_where_it_cannot_run():
    # 32-pixel-wide images: a pooling window spans two warps' rows of a tile; odd sizes; layers that do not fit in tensor memory
    assert not ops.conv_fprop_pool_fused_supported(8, 32, 32, 128, 128, 3, 3, 1)
    assert not ops.conv_fprop_pool_fused_supported(8, 6, 5, 128, 128, 3, 3, 1)
    assert not ops.conv_fprop_pool_fused_supported(1024, 16, 16, 128, 128, 3, 3, 1)


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,W,C2,K", [(4, 8, 8, 64, 32), (2, 5, 7, 8, 12), (3, 6, 6, 1, 16), (16, 16, 16, 128, 128)])
def test_conv_int4_operands(N, H, W, C2, K):
    """int4 pairs packed per byte (every nibble pattern occurs, -8 included), against the oracle's unpack + convolution."""
    rng = np.random.default_rng(N + C2 + K)
    x4 = rng.integers(0, 256, size=(N, H, W, C2), dtype=np.uint8)
    w4 = rng.integers(0, 256, size=(K, 3, 3, C2), dtype=np.uint8)
    y32, mx = ops.conv_fprop_i4(cu(x4), cu(w4), 1)
    want = O.conv_fprop_int4(x4, w4)
    assert_same(y32, want.astype(np.int32), "int4 convolution")
    assert int(mx) == int(np.abs(want).max())


@pytest.mark.gpu
def test_dp_update_peer_wait_gives_up_and_reports():
    """niti_dp_update_i8 told that there are two ranks, the second one a zeroed local area that nobody signals: the first
    cross-rank barrier runs into its 4 s limit, the kernel returns with status {9, rank waited for, barrier number}, updates
    nothing and the context keeps working.  One process, one GPU, one kernel: nothing waits for another launch."""
    import time
    sizes = [128 * 3 * 3 * 16, 4 * 1000]
    w_offs, off = [], 0
    for n in sizes:
        w_offs.append(off)
        off += (n + 255) // 256 * 256
    g_off = off
    g_offs, goff = [], 0
    for n in sizes:
        g_offs.append(goff)
        goff += n
    x_off = (g_off + 4 * goff + 255) // 256 * 256
    nbytes = x_off + ops.dp_exchange_bytes()
    arenas = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(2)]
    rng = np.random.default_rng(3)
    w0 = cu(rnd8(rng, (g_off,)))
    arenas[0][:g_off].view(torch.int8).copy_(w0)
    arenas[0][g_off:g_off + 4 * goff].view(torch.int32).copy_(cu(rng.integers(-500, 500, size=goff).astype(np.int32)))
    items = [(w_offs[i], g_offs[i], sizes[i], 16 * i + 2) for i in range(len(sizes))]
    seed = ops.seed_tensor(5, DEV)
    status = ops.status_word(DEV)
    status.zero_()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ops.dp_update(items, 0, 2, [a.data_ptr() for a in arenas], [a.data_ptr() + g_off for a in arenas],
                  [a.data_ptr() + x_off for a in arenas], 5, 2, seed, DEV)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    s = status.tolist()
    try:
        assert s[0] == 9 and s[1] == 1 and s[2] == 1, s
        assert 3.0 < dt < 12.0, dt
        with pytest.raises(RuntimeError, match="gave up waiting for rank 1 at barrier 1"):
            ops.check_status(DEV)
        assert torch.equal(arenas[0][:g_off].view(torch.int8), w0), "no weight may change when the exchange did not happen"
    finally:
        status.zero_()
    del arenas  # the exchange areas are discarded: their barrier numbers are meaningless now
    x = cu(np.arange(64, dtype=np.int32) - 32)            # the context is alive
    assert int(ops.absmax(x)) == 32


@pytest.mark.gpu
@pytest.mark.parametrize("N,H,W,C,K", [(128, 32, 32, 128, 128), (128, 8, 8, 512, 512), (256, 16, 16, 256, 256)])
def test_conv_passes_are_adjoint_at_full_size(N, H, W, C, K):
    """At the benchmark's full sizes, where the oracle is out of reach: the three passes must satisfy, exactly in
    integers, <conv(x, w), e> = <x, dgrad(e, w)> = <w, wgrad(x, e)> (the oracle satisfies the same identity, see
    tests/test_oracle_properties.py), and max|acc| reported by each pass must be the tensor's."""
    g = torch.Generator().manual_seed(N + C)
    x = torch.randint(-127, 128, (N, H, W, C), dtype=torch.int8, generator=g).to(DEV)
    w = torch.randint(-127, 128, (K, 3, 3, C), dtype=torch.int8, generator=g).to(DEV)
    e = torch.randint(-127, 128, (N, H, W, K), dtype=torch.int8, generator=g).to(DEV)
    y32, my = ops.conv_fprop_acc(x, w)
    d32, md = ops.conv_dgrad_acc(e, w)
    g32, mg = ops.conv_wgrad_acc(x, e)
    lhs = int((y32.to(torch.int64) * e.to(torch.int64)).sum())
    assert lhs == int((d32.to(torch.int64) * x.to(torch.int64)).sum()), "forward vs error-backward"
    assert lhs == int((g32.to(torch.int64) * w.to(torch.int64)).sum()), "forward vs weight gradient"
    for acc, m in ((y32, my), (d32, md), (g32, mg)):
        assert int(m) == int(acc.abs().max())
    ops.check_status(DEV)
    # the fused forms agree with narrowing the int32 tensors by the same shift
    st = ops.new_requant_state(DEV)
    ea = torch.zeros((), dtype=torch.int32, device=DEV)
    for _ in range(2):
        y8, _, shift = ops.conv_fprop_fused(x, w, st, 1, 0, None, 0, 0, True, ea, ea)
    want8, _, _ = ops.requant(y32, my, ops.CALC_ACT, 7, 0, None, 0, 0, relu=True)
    assert torch.equal(y8, want8)


@pytest.mark.gpu
def test_single_conv_layer_step_full_size_stochastic():
    """The single-layer benchmark configuration at full size (N=128, 32x32, C=K=128, 3x3, pad 1): forward, error-backward,
    weight gradient and update with stochastic rounding from the seeded stream, against the oracle (torch._int_mm
    products on the host)."""
    O.set_backend("int_mm")
    try:
        rng = np.random.default_rng(1234)
        N, H, W, C, K = 128, 32, 32, 128, 128
        x, w, e = rnd8(rng, (N, H, W, C)), rnd8(rng, (K, 3, 3, C)), rnd8(rng, (N, H, W, K))
        seed = ops.seed_tensor(42, DEV)
        ea = torch.zeros((), dtype=torch.int32, device=DEV)
        xt, wt, et = cu(x), cu(w), cu(e)
        # forward + act_calc (StoShift), stream 32
        st = ops.new_requant_state(DEV)
        for _ in range(2):
            y8, _, s_y = ops.conv_fprop_fused(xt, wt, st, 1, ops.ROUND_STOCHASTIC, seed, 32, 0, False, ea, ea)
        acc = O.conv_fprop(x, w, 1)
        want, _, s = O.act_calc(acc, 0, O.STOCHASTIC, philox.random_u32_tensor(42, 32, acc.shape))
        assert int(s_y) == s
        assert_same(y8, want, "forward, stochastic")
        # error-backward + err_calc (StoShift), stream 33
        st = ops.new_requant_state(DEV)
        for _ in range(2):
            e8, _, s_e = ops.conv_dgrad_fused(et, wt, st, 1, ops.ROUND_STOCHASTIC, seed, 33, 0, ea, ea)
        acc = O.conv_dgrad(e, w, 1)
        want, s = O.err_calc(acc, O.STOCHASTIC, philox.random_u32_tensor(42, 33, acc.shape))
        assert int(s_e) == s
        assert_same(e8, want, "error-backward, stochastic")
        # weight gradient (exact int32) + update with StoShift, stream 34
        g32, mg = ops.conv_wgrad_acc(xt, et)
        gacc = O.conv_wgrad(x, e, 3, 3, 1)
        assert_same(g32, gacc.astype(np.int32), "weight gradient")
        w2 = wt.clone()
        ops.update(w2, g32, mg, 5, ops.ROUND_STOCHASTIC, seed, 34)
        assert_same(w2, O.weight_update(w, gacc, 5, O.STOCHASTIC, philox.random_u32_tensor(42, 34, gacc.shape))[0], "update")
    finally:
        O.set_backend("int64")
