"""CPU oracle for NITI's int8 training hot path (TEST INFRASTRUCTURE, not product code).

Only ``tests/``, the smoke check and the benchmark's CPU-baseline / reference legs may
import this module; the shipped package never does.  Every function restates, in exact
integer arithmetic on NumPy arrays, one function of the reference (cited as file:line
within the reference project).  Conventions fixed here where the reference leaves them
open:

* ``//`` on tensors truncates toward zero, as it did in the torch 1.7 the reference was
  written for (Dockerfile:2); the closed forms below are what RoundShift / StoShift /
  PstoShift (ti_torch.py:23-69) evaluate to under that semantics.
* bit-width of a tensor = ``0 if max|x|==0 else bit_length(max|x|-1)``: the exact-integer
  value of ``ceil(log2(max|x|))`` (ti_torch.py:366-377).
* contractions are exact integer sums (the reference's CUTLASS epilogue rounds through
  fp32, cutlassconv_kernel.cu:46,159; not reproduced).
* max-pool backward routes dy to the FIRST window position, scanning rows then columns,
  that equals the window maximum.  The reference leaves this to cuDNN on fp16 copies
  (int8pool_kernel.cu:82-138); its tie rule is not observable here: parity unpinned
  for ties at that boundary.
* 2**s for fractional s in TiLoss (ti_loss.py:23) is evaluated by ``exp2_det`` below, a
  fixed sequence of IEEE double operations, then rounded to float32.

Contraction backend: ``int64`` (of record) or ``int_mm`` (torch._int_mm on int8, exact
int32, used for full-size timing runs); both give identical results whenever no
accumulator exceeds int32, which ``check_acc`` asserts.
"""
import numpy as np

from . import philox

BITWIDTH = 7  # ti_torch.py:458

ROUND, STOCHASTIC, PSEUDO_STOCHASTIC = 0, 1, 2  # RoundShift / StoShift / PstoShift

_BACKEND = "int64"


def set_backend(name):
    global _BACKEND
    assert name in ("int64", "int_mm")
    _BACKEND = name


# --------------------------------------------------------------------------------------
# requantisation (ti_torch.py:23-72, 103-147, 366-377)
# --------------------------------------------------------------------------------------

def bitwidth_of_max(m):
    """ti_torch.py:366-377 (RangeEstimate/TensorBitwidth) as exact integers."""
    m = int(m)
    return 0 if m == 0 else (m - 1).bit_length()


def range_estimate(x):
    x = np.asarray(x)
    if x.size == 0:
        return 0
    return bitwidth_of_max(np.max(np.abs(x.astype(np.int64))))


def int8_clip(x, clip_val=127):
    """ti_torch.py:71-72."""
    return np.clip(x, -clip_val, clip_val).astype(np.int8)


def _split(x, shift):
    x = np.asarray(x).astype(np.int64)
    a = np.abs(x)
    sg = np.sign(x)
    q = a >> shift
    lo = a & ((1 << shift) - 1)
    return sg, q, lo


def round_shift(x, shift):
    """RoundShift, ti_torch.py:23-31: round half away from zero, clamp to +-127."""
    sg, q, lo = _split(x, shift)
    return int8_clip(sg * (q + (lo >> (shift - 1))))


def sto_shift(x, shift, rand_u32):
    """StoShift, ti_torch.py:33-46.  ``rand_u32``: one uint32 word per element; the
    reference's ``randint(0, 2**shift)`` is its low ``shift`` bits."""
    sg, q, lo = _split(x, shift)
    r = np.asarray(rand_u32).astype(np.int64) & ((1 << shift) - 1)
    return int8_clip(sg * (q + (lo > r)))


def psto_shift(x, shift):
    """PstoShift, ti_torch.py:48-69: the low half of the dropped bits plays the random number."""
    sg, q, lo = _split(x, shift)
    h = shift // 2
    qp = lo >> h
    pr = lo & ((1 << h) - 1)
    if shift % 2 == 1:
        pr = pr * 2
    return int8_clip(sg * (q + (qp > pr)))


def apply_shift(x, shift, mode, rand_u32=None):
    if mode == ROUND:
        return round_shift(x, shift)
    if mode == STOCHASTIC:
        return sto_shift(x, shift, rand_u32)
    if mode == PSEUDO_STOCHASTIC:
        return psto_shift(x, shift)
    raise ValueError(mode)


def wrap_int8(x):
    """``tensor.type(torch.int8)`` on an int32 tensor: two's-complement wrap (ti_torch.py:115)."""
    return np.asarray(x).astype(np.int64).astype(np.int8)


def act_calc(acc, exp_in, mode=ROUND, rand_u32=None):
    """ti_torch.py:103-117.  Returns (int8, exp_out, shift)."""
    b = range_estimate(acc)
    shift = b - BITWIDTH
    if shift > 0:
        return apply_shift(acc, shift, mode, rand_u32), exp_in + shift, shift
    return wrap_int8(acc), exp_in, 0


def err_calc(acc, mode=ROUND, rand_u32=None):
    """ti_torch.py:119-133.  Returns (int8, shift)."""
    b = range_estimate(acc)
    shift = b - BITWIDTH
    if shift > 0:
        return apply_shift(acc, shift, mode, rand_u32), shift
    return wrap_int8(acc), 0


def grad_calc(acc, mu, mode=PSEUDO_STOCHASTIC, rand_u32=None):
    """ti_torch.py:135-147.  Returns (int8, shift)."""
    b = range_estimate(acc)
    shift = b - mu
    if b == 0:
        return np.zeros(np.shape(acc), dtype=np.int8), 0
    if shift < 1:
        return wrap_int8(acc), 0
    return apply_shift(acc, shift, mode, rand_u32), shift


def weight_update(w, grad_acc, mu, mode=PSEUDO_STOCHASTIC, rand_u32=None):
    """UpdateWeight.weight_update, ti_torch.py:16-21.  Returns (new int8 weights, int8 grad, shift)."""
    g, shift = grad_calc(grad_acc, mu, mode, rand_u32)
    new_w = int8_clip(w.astype(np.int16) - g.astype(np.int16))
    return new_w, g, shift


# --------------------------------------------------------------------------------------
# contractions
# --------------------------------------------------------------------------------------

def check_acc(acc):
    m = int(np.max(np.abs(acc))) if acc.size else 0
    assert m < 2 ** 31, "accumulator exceeds int32: the int8 path is not defined for this input"
    return acc


def _matmul_exact(a, b):
    """[m,k] int8 x [k,n] int8 -> int64 [m,n], exact."""
    if _BACKEND == "int_mm":
        import torch
        c = torch._int_mm(torch.from_numpy(np.ascontiguousarray(a, dtype=np.int8)),
                          torch.from_numpy(np.ascontiguousarray(b, dtype=np.int8)))
        return c.numpy().astype(np.int64)
    # float64 products of int8 are exact and sums stay below 2**53 for any k < 2**39
    c = np.matmul(np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64))
    return c.astype(np.int64)


def int8_mm(a, b):
    """int8mm, ti_torch.py:152-176 -> int8mm_cuda.int8_mm (int8mm_kernel.cu:8-34): exact a @ b."""
    return check_acc(_matmul_exact(a, b))


def _im2col(x, R, S, pad):
    """x [N,H,W,C] -> [N*H*W, R*S*C] for stride 1, same-size output when pad=(R-1)/2."""
    N, H, W, C = x.shape
    P = H + 2 * pad - R + 1
    Q = W + 2 * pad - S + 1
    xp = np.zeros((N, H + 2 * pad, W + 2 * pad, C), dtype=x.dtype)
    xp[:, pad:pad + H, pad:pad + W, :] = x
    cols = np.empty((N, P, Q, R, S, C), dtype=x.dtype)
    for r in range(R):
        for s in range(S):
            cols[:, :, :, r, s, :] = xp[:, r:r + P, s:s + Q, :]
    return cols.reshape(N * P * Q, R * S * C), (N, P, Q)


def conv_fprop(x, w, pad=1, stride=1):
    """conv2d_int8, ti_torch.py:178-192 -> cutlassconv_cuda.sp_conv_optimized
    (cutlassconv_kernel.cu:38-177): cross-correlation, NHWC x [K,R,S,C] -> int32 [N,P,Q,K]."""
    assert stride == 1, "the oracle restates the stride-1 path the reference models use"
    K, R, S, C = w.shape
    acc = None
    N = x.shape[0]
    step = max(1, (1 << 24) // max(1, x.shape[1] * x.shape[2] * R * S * C))
    outs = []
    for n0 in range(0, N, step):
        cols, (n, P, Q) = _im2col(x[n0:n0 + step], R, S, pad)
        outs.append(_matmul_exact(cols, w.reshape(K, R * S * C).T).reshape(n, P, Q, K))
    acc = np.concatenate(outs, axis=0) if outs else np.zeros((0,) + x.shape[1:3] + (K,), np.int64)
    return check_acc(acc)


def unpack_int4(a):
    """Bytes holding two signed 4-bit values each, even element in the low nibble (cutlass int4b_t arrays,
    include/cutlass/array_subbyte.h:116-124) -> int8 with twice as many entries along the last axis."""
    b = np.asarray(a).view(np.uint8)
    lo = (b & 15).astype(np.int8)
    hi = (b >> 4).astype(np.int8)
    lo = np.where(lo > 7, lo - 16, lo).astype(np.int8)
    hi = np.where(hi > 7, hi - 16, hi).astype(np.int8)
    return np.stack([lo, hi], axis=-1).reshape(b.shape[:-1] + (2 * b.shape[-1],))


def conv_fprop_int4(x4, w4, pad=1):
    """cutlassconv_cuda.int4_conv (cutlassconv_kernel.cu:602-884): the int8 convolution of the unpacked operands."""
    return conv_fprop(unpack_int4(x4), unpack_int4(w4), pad=pad)


def flip_transpose(w):
    """ti_torch.py:404: torch.flip(w,[1,2]).transpose(0,3) -> [C,R,S,K]."""
    return np.ascontiguousarray(np.flip(w, axis=(1, 2)).transpose(3, 1, 2, 0))


def conv_dgrad(err, w, pad=1):
    """TiConv2d.backward error path, ti_torch.py:403-405: err (x) flipped/transposed w = dX."""
    return conv_fprop(err, flip_transpose(w), pad=w.shape[1] - 1 - pad)


def conv_wgrad(x, err, R=3, S=3, pad=1):
    """TiConv2d.backward gradient path, ti_torch.py:429-432 (and the first-layer group-conv
    form, ti_torch.py:194-233, which equals the same sum):
    g[k,r,s,c] = sum_{n,p,q} err[n,p,q,k] * x[n,p+r-pad,q+s-pad,c]."""
    N, H, W, C = x.shape
    K = err.shape[3]
    xp = np.zeros((N, H + 2 * pad, W + 2 * pad, C), dtype=np.int8)
    xp[:, pad:pad + H, pad:pad + W, :] = x
    P, Q = err.shape[1], err.shape[2]
    e2 = err.reshape(N * P * Q, K)
    g = np.empty((K, R, S, C), dtype=np.int64)
    for r in range(R):
        for s in range(S):
            xs = np.ascontiguousarray(xp[:, r:r + P, s:s + Q, :]).reshape(N * P * Q, C)
            g[:, r, s, :] = _matmul_exact(np.ascontiguousarray(e2.T), xs)
    return check_acc(g)


# --------------------------------------------------------------------------------------
# memory-bound layers
# --------------------------------------------------------------------------------------

def relu_fwd(x):
    """TiReLU.forward, ti_torch.py:272-279."""
    return np.maximum(x, np.int8(0))


def relu_bwd(act_in, err):
    """TiReLU.backward, ti_torch.py:281-290."""
    return np.where(act_in > 0, err, np.int8(0)).astype(np.int8)


def maxpool_fwd(x, k=2, stride=2):
    """TiMaxpool2d.forward, ti_torch.py:302-307 (int8pool_kernel.cu:28-80), pad 0."""
    N, H, W, C = x.shape
    P = (H - k) // stride + 1
    Q = (W - k) // stride + 1
    y = np.full((N, P, Q, C), -128, dtype=np.int8)
    for i in range(k):
        for j in range(k):
            y = np.maximum(y, x[:, i:i + stride * P:stride, j:j + stride * Q:stride, :])
    return y


def maxpool_bwd(x, dy, k=2, stride=2):
    """TiMaxpool2d.backward, ti_torch.py:309-316; first-max tie rule (module docstring).
    Overlapping windows (stride < k) accumulate with int8 wrap, as an int8 sum would."""
    N, H, W, C = x.shape
    y = maxpool_fwd(x, k, stride)
    P, Q = y.shape[1], y.shape[2]
    dx = np.zeros(x.shape, dtype=np.int64)
    taken = np.zeros(y.shape, dtype=bool)
    for i in range(k):
        for j in range(k):
            xs = x[:, i:i + stride * P:stride, j:j + stride * Q:stride, :]
            hit = (xs == y) & ~taken
            taken |= hit
            dx[:, i:i + stride * P:stride, j:j + stride * Q:stride, :] += np.where(hit, dy, 0)
    return dx.astype(np.int8)


def dropout_mask(seed, stream, features):
    """TiDropout.forward, ti_torch.py:446: one Bernoulli(1/2) bit per feature, shared by the batch."""
    return (philox.random_u32_tensor(seed, stream, (features,)) & 1).astype(np.int8)


# --------------------------------------------------------------------------------------
# input quantisation and loss
# --------------------------------------------------------------------------------------

def float_bitwidth(r):
    """ceil(log2(r)) for a positive float32 r, from its exponent and mantissa (exact)."""
    m, e = np.frexp(np.float32(r))  # r = m * 2**e, m in [0.5, 1)
    return int(e) - 1 if m == 0.5 else int(e)


def float_to_int8(x):
    """TiFloatToInt8, ti_torch.py:341-356.  x float32 -> (int8, exp)."""
    x = np.asarray(x, dtype=np.float32)
    r = np.max(np.abs(x))
    b = float_bitwidth(r)
    norm = x * np.float32(2.0 ** (BITWIDTH - b))
    q = np.clip(np.rint(norm), -128, 127).astype(np.int8)
    return q, b - BITWIDTH


_LN2 = 0.6931471805599453  # nearest double to ln 2


def exp2_det(s):
    """2**s for 0 <= s (float64 array) by a fixed sequence of IEEE-754 double operations:
    split s = i + f, Horner-evaluate sum_{j<=17} (f ln2)^j / j! with separate multiplies
    and adds (no fused multiply-add), scale by 2**i."""
    s = np.asarray(s, dtype=np.float64)
    i = np.floor(s)
    t = (s - i) * _LN2
    acc = np.full(s.shape, 1.0 / 355687428096000.0)  # 1/17!
    fact = 355687428096000.0
    for j in range(17, 0, -1):
        fact = fact / j  # (j-1)!
        acc = acc * t + (1.0 / fact)
    return np.ldexp(acc, i.astype(np.int64))


def ti_loss(out_val, out_exp, target, rand_u32):
    """TiLoss.forward, ti_loss.py:6-36.  out_val int8 [B,classes], out_exp int, target [B];
    ``rand_u32`` [B,classes] words for the closing StoShift(.,4).  float32 steps follow the
    reference's order of operations."""
    B, n = out_val.shape
    s = out_val.astype(np.int64)
    f32 = np.float32
    if out_exp > -7:
        sf = (s * 47274).astype(f32) / f32(2 ** 15)
        if out_exp >= 0:
            sf = sf * f32(2.0 ** out_exp)
        else:
            sf = sf / f32(2.0 ** (-out_exp))
        out_max = sf.max(axis=1)
        offset = out_max - f32(10)
        sf = sf - offset[:, None]
        sf = np.maximum(sf, f32(0))
        out_grad = exp2_det(sf.astype(np.float64)).astype(f32) - f32(1)
        out_sum = out_grad.astype(np.int64).sum(axis=1)
    else:
        e = int(out_exp)
        gi = (2 ** (1 - 2 * e)) + s * (2 ** (1 - e)) + s * s
        out_sum = gi.sum(axis=1)
        out_grad = gi.astype(f32)  # int64 -> float32 happens inside the true division below
    out_grad = (out_grad * f32(2 ** 11)) / out_sum.astype(f32)[:, None]
    row_sum = out_grad.astype(np.int64).sum(axis=1)
    rows = np.arange(B)
    out_grad[rows, target] = out_grad[rows, target] - row_sum.astype(f32)
    g32 = out_grad.astype(np.int64)  # .type(torch.int32): truncation toward zero
    return sto_shift(g32, 4, rand_u32), 0


# --------------------------------------------------------------------------------------
# model-level restatement (ti_net.py:17-32, ti_vgg.py:10-42)
# --------------------------------------------------------------------------------------

VGG_CFGS = {
    # ti_vgg.py:10-14
    "ref7": [128, 128, "M", 256, 256, "M", 512, 512, "M"],
    "ref8": [128, 128, 128, "M", 256, 256, "M", 512, 512, "M"],
    "ref9": [128, 128, 128, "M", 256, 256, 256, "M", 512, 512, "M"],
}


class Layer:
    pass


class Net:
    """Layer-by-layer restatement of TiNet.forward/backward over ti_vgg's layer list.

    Stream ids for random bits: the l-th weighted layer (convs in order, then the FC) uses
    streams 16*l + {0: act, 1: err, 2: grad}; dropout uses 0xFFFE and the loss 0xFFFF; the
    generator's seed is ``seed + step``.  Element indices are global (sample offset times
    per-sample size) so that a batch shard draws the bits of its own samples.
    """

    def __init__(self, cfg, weights, weight_exps, in_hw=32, classes=10, dropout=True,
                 act_mode=ROUND, err_mode=ROUND, grad_mode=PSEUDO_STOCHASTIC, mu=5, seed=0):
        self.cfg, self.dropout = list(cfg), dropout
        self.w = [np.array(w, dtype=np.int8) for w in weights]
        self.w_exp = list(weight_exps)
        self.act_mode, self.err_mode, self.grad_mode, self.mu, self.seed = act_mode, err_mode, grad_mode, mu, seed
        self.trace = {}

    def _rand(self, mode, stream, shape, step, offset=0):
        if mode != STOCHASTIC:
            return None
        return philox.random_u32_tensor(self.seed + step, stream, shape, offset)

    def forward(self, x8, x_exp, step=0, sample_offset=0, training=True):
        """x8 int8 NHWC, x_exp int.  Returns (logits int8, exp)."""
        t = self.trace = {"saved": []}
        a, e = x8, x_exp
        li = 0
        for c in self.cfg:
            if c == "M":
                t["saved"].append(("pool", a))
                a = maxpool_fwd(a)
            else:
                acc = conv_fprop(a, self.w[li])
                per = acc[0].size if acc.shape[0] else 0
                r = self._rand(self.act_mode, 16 * li, acc.shape, step, sample_offset * per)
                y, e2, sh = act_calc(acc, e + self.w_exp[li], self.act_mode, r)
                t["saved"].append(("conv", li, a, e))
                t["saved"].append(("relu", y))
                a, e = relu_fwd(y), e2
                li += 1
        t["saved"].append(("flat", a.shape))
        a = a.reshape(a.shape[0], -1)
        if self.dropout and training:
            m = dropout_mask(self.seed + step, 0xFFFE, a.shape[1])
            t["saved"].append(("drop", m))
            a, e = a * m, e + 1
        acc = int8_mm(a, self.w[li].T)
        r = self._rand(self.act_mode, 16 * li, acc.shape, step, sample_offset * acc.shape[1])
        y, e2, sh = act_calc(acc, e + self.w_exp[li], self.act_mode, r)
        t["saved"].append(("fc", li, a, e))
        t["out"], t["out_exp"] = y, e2
        return y, e2

    def backward(self, target, step=0, sample_offset=0, update=True):
        """TiNet.backward (ti_net.py:25-32).  Returns {layer: int64 grad accumulators}; updates weights
        in place unless ``update`` is False (data-parallel callers sum accumulators first)."""
        t = self.trace
        B, n = t["out"].shape
        r = philox.random_u32_tensor(self.seed + step, 0xFFFF, (B, n), sample_offset * n)
        err, e_exp = ti_loss(t["out"], t["out_exp"], target, r)
        t["loss_err"] = err
        grads = {}
        t["errs"] = {}
        for item in reversed(t["saved"]):
            kind = item[0]
            if kind == "fc":
                _, li, a, a_exp = item
                acc = int8_mm(err, self.w[li])
                rr = self._rand(self.err_mode, 16 * li + 1, acc.shape, step, sample_offset * acc.shape[1])
                e_out, sh = err_calc(acc, self.err_mode, rr)
                grads[li] = int8_mm(np.ascontiguousarray(err.T), a)
                e_exp = e_exp + sh + self.w_exp[li]
                err = e_out
            elif kind == "drop":
                err = err * item[1]
            elif kind == "flat":
                err = err.reshape(item[1])
            elif kind == "pool":
                err = maxpool_bwd(item[1], err)
            elif kind == "relu":
                err = relu_bwd(item[1], err)
            elif kind == "conv":
                _, li, a, a_exp = item
                grads[li] = conv_wgrad(a, err)
                if li != 0:
                    acc = conv_dgrad(err, self.w[li])
                    per = acc[0].size
                    rr = self._rand(self.err_mode, 16 * li + 1, acc.shape, step, sample_offset * per)
                    e_out, sh = err_calc(acc, self.err_mode, rr)
                    e_exp = e_exp + sh + self.w_exp[li]
                    err = e_out
                    t["errs"][li] = err
        if update:
            self.apply_grads(grads, step)
        return grads

    def apply_grads(self, grads, step=0):
        for li, g in grads.items():
            rr = self._rand(self.grad_mode, 16 * li + 2, g.shape, step)
            self.w[li], _, _ = weight_update(self.w[li], g, self.mu, self.grad_mode, rr)
