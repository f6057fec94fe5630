"""Counter-based random bits for stochastic rounding and dropout (TEST INFRASTRUCTURE).

This file is part of the CPU oracle: only the test-suite, the smoke check and the
benchmark's CPU-baseline leg may import it.  The shipped CUDA kernels carry their
own device implementation of the same generator.

Generator: Philox4x32-10 (Salmon, Moraes, Dror, Shaw, "Parallel random numbers:
as easy as 1, 2, 3", SC'11), restated from the paper.  The reference draws its
random integers with ``torch.randint`` (ti_torch.py:41 for StoShift,
ti_torch.py:446 for TiDropout); a library RNG cannot be reproduced bit-for-bit
across devices, so both sides of the parity tests use this keyed generator and
the reference is fed the same numbers by substituting ``torch.randint``.

Word for element ``idx`` of stream ``stream`` under ``seed``::

    block   = philox4x32_10(counter=(lo32(idx>>2), hi32(idx>>2), stream, 0),
                            key=(lo32(seed), hi32(seed)))
    u32     = block[idx & 3]
"""
import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_S32 = np.uint64(32)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Ten rounds of Philox-4x32 on arrays of uint32 counters; returns 4 uint32 arrays."""
    c0 = np.asarray(c0, dtype=np.uint64) & _MASK
    c1 = np.asarray(c1, dtype=np.uint64) & _MASK
    c2 = np.asarray(c2, dtype=np.uint64) & _MASK
    c3 = np.asarray(c3, dtype=np.uint64) & _MASK
    k0 = int(k0) & 0xFFFFFFFF
    k1 = int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> _S32, p0 & _MASK
        hi1, lo1 = p1 >> _S32, p1 & _MASK
        c0, c1, c2, c3 = (hi1 ^ c1 ^ np.uint64(k0)), lo1, (hi0 ^ c3 ^ np.uint64(k1)), lo0
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return (c0.astype(np.uint32), c1.astype(np.uint32),
            c2.astype(np.uint32), c3.astype(np.uint32))


def random_u32(seed, stream, idx):
    """uint32 word for each global element index in ``idx`` (any integer array)."""
    idx = np.asarray(idx, dtype=np.uint64)
    blk = idx >> np.uint64(2)
    lane = (idx & np.uint64(3)).astype(np.int64)
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    out = philox4x32_10(blk & _MASK, blk >> _S32,
                        np.full(blk.shape, int(stream) & 0xFFFFFFFF, dtype=np.uint64),
                        np.zeros(blk.shape, dtype=np.uint64),
                        seed & 0xFFFFFFFF, seed >> 32)
    stacked = np.stack(out, axis=-1)
    return np.take_along_axis(stacked, lane[..., None], axis=-1)[..., 0]


def random_u32_tensor(seed, stream, shape, offset=0):
    """Words for a C-contiguous tensor of ``shape`` whose first element has global index ``offset``."""
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    idx = np.arange(n, dtype=np.uint64) + np.uint64(offset)
    return random_u32(seed, stream, idx).reshape(shape)
