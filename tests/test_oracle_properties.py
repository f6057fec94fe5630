"""Size-independent properties of the oracle (CPU, hypothesis): closed forms of the shifts in plain Python integers,
bounds of the stochastic variants, adjointness of the three convolution passes.  The same adjoint identity is what
the GPU suite checks at the benchmark's full sizes, where the oracle itself would be too slow."""
import numpy as np
from hypothesis import given, settings, strategies as st

from oracle import niti_oracle as O

ints32 = st.integers(min_value=-(2 ** 31) + 1, max_value=2 ** 31 - 1)


def _clamp(v):
    return max(-127, min(127, v))


@settings(max_examples=300, deadline=None)
@given(st.lists(ints32, min_size=1, max_size=64), st.integers(min_value=1, max_value=24))
def test_round_shift_is_round_half_away_from_zero(values, s):
    x = np.array(values, dtype=np.int64)
    got = O.round_shift(x, s)
    for v, g in zip(values, got):
        a = abs(v)
        want = (a + (1 << (s - 1))) >> s
        assert int(g) == _clamp(want if v >= 0 else -want)


@settings(max_examples=300, deadline=None)
@given(st.lists(ints32, min_size=1, max_size=64), st.integers(min_value=1, max_value=24), st.integers(min_value=0, max_value=2 ** 32 - 1))
def test_stochastic_shifts_lie_between_truncation_and_one_more(values, s, word):
    x = np.array(values, dtype=np.int64)
    rnd = np.full(x.shape, word, dtype=np.uint64)
    for got in (O.sto_shift(x, s, rnd), O.psto_shift(x, s)):
        for v, g in zip(values, got):
            q = abs(v) >> s
            lo, hi = _clamp(q), _clamp(q + 1)
            assert lo <= abs(int(g)) <= hi and (int(g) == 0 or (int(g) > 0) == (v > 0))
    # the extreme random words give the two ends
    assert np.array_equal(np.abs(O.sto_shift(x, s, np.full(x.shape, (1 << s) - 1, dtype=np.uint64))),
                          np.minimum(np.abs(x) >> s, 127))
    up = (np.abs(x) & ((1 << s) - 1)) > 0
    assert np.array_equal(np.abs(O.sto_shift(x, s, np.zeros(x.shape, dtype=np.uint64))), np.minimum((np.abs(x) >> s) + up, 127))


@settings(max_examples=200, deadline=None)
@given(st.lists(ints32, min_size=1, max_size=32))
def test_bitwidth_is_bit_length_of_max_minus_one(values):
    x = np.array(values, dtype=np.int64)
    m = int(np.abs(x).max())
    assert O.range_estimate(x) == (0 if m == 0 else (m - 1).bit_length())


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 3), st.integers(2, 7), st.integers(2, 7), st.integers(1, 5), st.integers(1, 5), st.integers(0, 2 ** 31 - 1))
def test_conv_passes_are_adjoint(N, H, W, C, K, seed):
    """<conv(x, w), e> = <x, dgrad(e, w)> = <w, wgrad(x, e)>: exact in integers, whatever the sizes."""
    rng = np.random.default_rng(seed)
    x = rng.integers(-127, 128, size=(N, H, W, C)).astype(np.int8)
    w = rng.integers(-127, 128, size=(K, 3, 3, C)).astype(np.int8)
    e = rng.integers(-127, 128, size=(N, H, W, K)).astype(np.int8)
    lhs = int((O.conv_fprop(x, w, 1).astype(np.int64) * e).sum())
    assert lhs == int((O.conv_dgrad(e, w, 1).astype(np.int64) * x).sum())
    assert lhs == int((O.conv_wgrad(x, e, 3, 3, 1).astype(np.int64) * w).sum())


def test_exact_backends_agree():
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, size=(37, 53)).astype(np.int8)
    b = rng.integers(-127, 128, size=(53, 29)).astype(np.int8)
    O.set_backend("int64")
    r64 = O.int8_mm(a, b)
    try:
        O.set_backend("int_mm")
        assert np.array_equal(O.int8_mm(a, b), r64)
    finally:
        O.set_backend("int64")


def test_int4_unpacking_order_and_sign():
    a = np.array([[0x10, 0x8F, 0x7A]], dtype=np.uint8)      # (lo, hi) = (0, 1), (-1, -8), (-6, 7)
    assert O.unpack_int4(a).tolist() == [[0, 1, -1, -8, -6, 7]]


@settings(max_examples=200, deadline=None)
@given(st.integers(2, 24), st.integers(0, 2 ** 31 - 1))
def test_round_shift_one_lower_follows_from_the_upper_result_and_two_bits(S, seed):
    """What the kernels' repair of a shift guessed one too high rests on (niti_conv_dgrad_requant_side_i8): with
    u = x + 2^(S-1) - [x < 0], y = u >> S is RoundShift(x, S) before clamping and code = (u >> (S-2)) & 3; then
    RoundShift(x, S-1) = clamp(2 y + [code == 3] - [code == 0]) for every x whose magnitude is below 2^(S+6), i.e.
    whenever S - 1 is the shift the tensor really needs."""
    rng = np.random.default_rng(seed)
    lim = 1 << (S + 6)
    x = rng.integers(-(lim - 1), lim, size=4096, dtype=np.int64)
    x[:8] = [lim - 1, -(lim - 1), 0, 1, -1, (1 << (S - 2)), -(1 << (S - 2)), (1 << (S - 1)) - 1]
    u = x + (1 << (S - 1)) - (x < 0)
    y = u >> S
    code = (u >> (S - 2)) & 3
    assert np.array_equal(np.clip(y, -127, 127).astype(np.int8), O.round_shift(x, S))
    lower = np.clip(2 * y + (code == 3) - (code == 0), -127, 127).astype(np.int8)
    assert np.array_equal(lower, O.round_shift(x, S - 1))
