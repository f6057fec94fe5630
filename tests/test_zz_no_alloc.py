"""niti_conv_wgrad_builtin_scratch_i8: the weight gradient for hosts that cannot allocate device memory
(a plugin under an application that owns all of it, a service with a fixed, audited budget).  Called
through the C ABI; its output must equal niti_conv_wgrad_i8's bit for bit, on two calls in a row that
share the library's built-in scratch buffer.  Collected last on purpose (file name): a failure here
cannot hide one elsewhere when the suite stops at the first failure."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from niti_b200._lib import lib  # noqa: E402
from oracle import niti_oracle as O  # noqa: E402

DEV = "cuda:0"
LIMIT = 16 << 20


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def wgrad_both(x, err, pad=1):
    """(g32, max) from the entry point with caller scratch and from the one with built-in scratch."""
    N, H, W, C = x.shape
    K = err.shape[3]
    outs = []
    for builtin in (False, True):
        g32 = torch.full((K, 3, 3, C), 0x5A5A5A5A, dtype=torch.int32, device=DEV)
        mx = torch.full((1,), -1, dtype=torch.int32, device=DEV)
        if builtin:
            rc = lib.niti_conv_wgrad_builtin_scratch_i8(_ptr(x), _ptr(err), _ptr(g32), _ptr(mx), N, H, W, C, K, 3, 3, pad,
                                                        None, _stream())
        else:
            nbytes = lib.niti_conv_wgrad_scratch_bytes(N, H, W, C, K, 3, 3)
            sc = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
            rc = lib.niti_conv_wgrad_i8(_ptr(x), _ptr(err), _ptr(g32), _ptr(mx), _ptr(sc), nbytes, N, H, W, C, K, 3, 3, pad,
                                        None, _stream())
        assert rc == 0, lib.niti_strerror(rc)
        torch.cuda.synchronize()
        outs.append((g32.cpu().numpy(), int(mx.item())))
    return outs


@pytest.mark.parametrize("N,H,W,C,K", [
    (16, 16, 16, 256, 256),   # tensor-core path; the usual 12 splits (28 MB) do not fit: runs with 7
    (8, 8, 8, 128, 128),      # tensor-core path, fits as planned
    (8, 8, 8, 144, 144),      # channel counts that are multiples of 16 but not of 128: the tail tiles are clipped by TMA
    (8, 8, 8, 16, 48),        # a single, mostly clipped tile per tap
    (32, 32, 32, 3, 128),     # first-layer path: patch matrix + split-K partials in the buffer
    (2, 6, 10, 5, 7),         # CUDA-core path: needs no scratch at all
])
def test_matches_caller_scratch_variant_twice_in_a_row(N, H, W, C, K):
    torch.cuda.set_device(0)
    rng = np.random.default_rng(N * 3 + C + K)
    for call in range(2):  # the second call finds the first call's partial sums in the buffer
        xh = rng.integers(-127, 128, size=(N, H, W, C)).astype(np.int8)
        eh = rng.integers(-127, 128, size=(N, H, W, K)).astype(np.int8)
        x, err = torch.from_numpy(xh).to(DEV), torch.from_numpy(eh).to(DEV)
        (g_ref, m_ref), (g_new, m_new) = wgrad_both(x, err)
        assert np.array_equal(g_new, g_ref), f"call {call}: gradients differ"
        assert m_new == m_ref == int(np.abs(g_ref).max())
        if call == 0:  # and against the oracle itself, not only against the sibling entry point
            assert np.array_equal(g_new, O.conv_wgrad(xh, eh, 3, 3, 1).astype(np.int32))


def test_maximum_is_optional_as_in_the_caller_scratch_variant():
    torch.cuda.set_device(0)
    rng = np.random.default_rng(5)
    xh = rng.integers(-127, 128, size=(4, 8, 8, 128)).astype(np.int8)
    eh = rng.integers(-127, 128, size=(4, 8, 8, 128)).astype(np.int8)
    x, err = torch.from_numpy(xh).to(DEV), torch.from_numpy(eh).to(DEV)
    g32 = torch.zeros((128, 3, 3, 128), dtype=torch.int32, device=DEV)
    rc = lib.niti_conv_wgrad_builtin_scratch_i8(_ptr(x), _ptr(err), _ptr(g32), None, 4, 8, 8, 128, 128, 3, 3, 1, None, _stream())
    assert rc == 0, lib.niti_strerror(rc)
    torch.cuda.synchronize()
    assert np.array_equal(g32.cpu().numpy(), O.conv_wgrad(xh, eh, 3, 3, 1).astype(np.int32))


def test_refuses_what_does_not_fit_and_allocates_nothing():
    torch.cuda.set_device(0)
    C = K = 1024  # one unsplit copy of the gradient is 37.7 MB > 16 MiB
    assert C * K * 9 * 4 > LIMIT
    x = torch.zeros((1, 4, 4, C), dtype=torch.int8, device=DEV)
    err = torch.zeros((1, 4, 4, K), dtype=torch.int8, device=DEV)
    g32 = torch.zeros((16,), dtype=torch.int32, device=DEV)  # never written: the call must stop at the size check
    mx = torch.full((1,), 77, dtype=torch.int32, device=DEV)
    rc = lib.niti_conv_wgrad_builtin_scratch_i8(_ptr(x), _ptr(err), _ptr(g32), _ptr(mx), 1, 4, 4, C, K, 3, 3, 1, None, _stream())
    assert rc == -5 and b"built-in" in lib.niti_strerror(rc)
    torch.cuda.synchronize()
    assert int(mx.item()) == 77 and int(g32.abs().sum().item()) == 0
    # a fitting call neither grows nor shrinks the device memory in use (nothing is allocated or freed behind the caller)
    xs = torch.ones((8, 8, 8, 128), dtype=torch.int8, device=DEV)
    es = torch.ones((8, 8, 8, 128), dtype=torch.int8, device=DEV)
    g = torch.zeros((128, 3, 3, 128), dtype=torch.int32, device=DEV)
    lib.niti_conv_wgrad_builtin_scratch_i8(_ptr(xs), _ptr(es), _ptr(g), _ptr(mx), 8, 8, 8, 128, 128, 3, 3, 1, None, _stream())
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert lib.niti_conv_wgrad_builtin_scratch_i8(_ptr(xs), _ptr(es), _ptr(g), _ptr(mx), 8, 8, 8, 128, 128, 3, 3, 1, None, _stream()) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert int(g[0, 1, 1, 0].item()) == 8 * 8 * 8
