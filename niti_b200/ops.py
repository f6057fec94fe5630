"""torch-tensor front end of the C ABI: allocates outputs with torch, launches on torch's
current stream of the tensors' device, never synchronises.

Shapes and layouts are those of the reference's extension calls (NHWC int8 activations,
[K,R,S,C] int8 filters); per-tensor exponents, shifts and max|acc| words are 0-dim / 1-element
int32 CUDA tensors so that nothing here reads a value back to the host.
"""
import torch

import ctypes

from ._lib import lib, check, FcHeadArgs, UpdateItem, DpItem, DpUpdateArgs, WgradItem

ROUND_NEAREST, ROUND_STOCHASTIC, ROUND_PSEUDO_STOCHASTIC = 0, 1, 2
CALC_ACT, CALC_ERR, CALC_GRAD = 0, 1, 2

_status = {}
_scratch = {}
_scratch_retired = []

# Launch accounting.  LAUNCHES counts kernels of this library enqueued through this module.
# PROFILE, when set to a list (eager execution only, never under graph capture), makes every
# call record (name, algorithmic ops, algorithmic bytes, start event, end event) on the
# launching stream.
LAUNCHES = 0
PROFILE = None


def _call(name, kernels, algo_ops, algo_bytes, fn, *args):
    global LAUNCHES
    LAUNCHES += kernels
    if PROFILE is None:
        check(fn(*args), name)
        return
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    check(fn(*args), name)
    b.record()
    PROFILE.append((name, algo_ops, algo_bytes, a, b))


def _st():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            raise RuntimeError("niti_b200 ops need contiguous CUDA tensors (there is no CPU path)")


def status_word(device):
    """int32[4] the tensor-core kernels write if one of their bounded waits expires."""
    key = torch.device(device).index
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[key]


def status_message(s):
    """Text for a non-zero status word (a list of its four values)."""
    if s[0] == 9:
        who = f"rank {s[1]}" if s[1] >= 0 else "the blocks of its own grid"
        return (f"niti_b200 data-parallel update gave up waiting for {who} at barrier {s[2]}: "
                "the replicas are out of step")
    return f"niti_b200 kernel gave up waiting: code={s[0]} block={s[1]} role={s[2]}"


def check_status(device):
    """Synchronises and raises if a kernel reported a timed-out wait."""
    s = status_word(device).tolist()
    if s[0] != 0:
        raise RuntimeError(status_message(s))


def scratch(device, nbytes):
    """Grow-only per-device scratch arena (stream-ordered reuse on the current stream).  An arena that is outgrown is
    kept alive, not freed: a captured CUDA graph may still hold its address."""
    key = torch.device(device).index
    cur = _scratch.get(key)
    if cur is None or cur.numel() < nbytes:
        if cur is not None:
            _scratch_retired.append(cur)
        cur = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = cur
    return cur


def seed_tensor(value, device):
    """uint64 seed word on the device (stored in an int64 tensor)."""
    return torch.tensor([int(value)], dtype=torch.int64, device=device)


# ------------------------------------------------------------------ contractions
def conv_fprop_acc(x, w, pad=1, stride=1):
    _need_cuda(x, w)
    N, H, W, C = x.shape
    K, R, S, C2 = w.shape
    assert C == C2 and x.dtype == torch.int8 and w.dtype == torch.int8
    P, Q = H + 2 * pad - R + 1, W + 2 * pad - S + 1
    y32 = torch.empty((N, P, Q, K), dtype=torch.int32, device=x.device)
    mx = torch.empty(1, dtype=torch.int32, device=x.device)
    nbytes = lib.niti_conv_fprop_scratch_bytes(N, H, W, C, K, R, S)
    sc = scratch(x.device, nbytes) if nbytes else None
    _call("niti_conv_fprop_i8", 2 if nbytes else 1, 2 * N * P * Q * K * R * S * C, x.numel() + w.numel() + 4 * y32.numel(),
          lib.niti_conv_fprop_i8, _p(x), _p(w), _p(y32), _p(mx), _p(sc), sc.numel() if nbytes else 0,
          N, H, W, C, K, R, S, pad, stride, _p(status_word(x.device)), _st())
    return y32, mx


def conv_fprop_i4(x4, w4, pad=1):
    """int4 convolution: x4 uint8 [N,H,W,C/2] and w4 uint8 [K,R,S,C/2] hold two signed 4-bit channels per byte (even channel
    in the low nibble) -> (int32 [N,P,Q,K], max|y|).  The reference's cutlassconv_cuda.int4_conv."""
    _need_cuda(x4, w4)
    assert x4.dtype == torch.uint8 and w4.dtype == torch.uint8
    N, H, W, C2 = x4.shape
    K, R, S, _ = w4.shape
    P, Q = H + 2 * pad - R + 1, W + 2 * pad - S + 1
    y32 = torch.empty((N, P, Q, K), dtype=torch.int32, device=x4.device)
    mx = torch.empty(1, dtype=torch.int32, device=x4.device)
    nbytes = lib.niti_conv_fprop_i4_scratch_bytes(N, H, W, C2, K, R, S)
    sc = scratch(x4.device, nbytes)
    _call("niti_conv_fprop_i4", 3, 2 * N * P * Q * K * R * S * 2 * C2, x4.numel() + w4.numel() + 4 * y32.numel(),
          lib.niti_conv_fprop_i4, _p(x4), _p(w4), _p(y32), _p(mx), _p(sc), sc.numel(), N, H, W, C2, K, R, S, pad,
          _p(status_word(x4.device)), _st())
    return y32, mx


def set_accumulator_parking(enabled):
    """Switch the single-launch (accumulators parked in tensor memory) fused kernels on or off; returns the old setting."""
    return bool(lib.niti_set_option(1, int(bool(enabled))))


def set_cooperative_launch(enabled):
    """Cooperative (default) or plain launches for the kernels with a grid barrier; returns the old setting."""
    return bool(lib.niti_set_option(5, int(bool(enabled))))


def set_cta_pairs(mask):
    """CTA pairs (tcgen05 cta_group::2): bit 0 for GEMMs (default on), bit 1 for convolutions (default off);
    True = both, False = none.  Returns the old mask."""
    if isinstance(mask, bool):
        mask = 3 if mask else 0
    return lib.niti_set_option(4, int(mask))


def set_wgrad_tma_reduce(enabled):
    """Tensor-core weight gradient: add tiles into the gradient with TMA reductions (default) or go through
    partial sums in scratch; returns the old setting."""
    return bool(lib.niti_set_option(2, int(bool(enabled))))


def new_requant_state(device):
    """int32[8] a fused conv + requantisation call keeps per layer and direction:
    [0] shift (prediction in, true value out), [1] max|acc|, [2] redo flag, [3] redo count, [4] block ticket."""
    return torch.zeros(8, dtype=torch.int32, device=device)


def conv_fprop_fused_supported(C, K, R, S, pad):
    return bool(lib.niti_conv_fprop_requant_supported(C, K, R, S, pad))


def conv_dgrad_fused_supported(C, K, R, S, pad):
    return bool(lib.niti_conv_dgrad_requant_supported(C, K, R, S, pad))


def conv_fprop_scratch_bytes(N, H, W, C, K, R, S):
    """Scratch bytes of a forward convolution (non-zero for thin layers: their patch matrix [N*H*W][32] + padded filters)."""
    return int(lib.niti_conv_fprop_scratch_bytes(N, H, W, C, K, R, S))


def conv_fprop_fused(x, w, state, pad=1, mode=ROUND_NEAREST, seed=None, rng_stream=0, rng_offset=0, relu=False,
                     exp_a=None, exp_b=None, scratch_buf=None):
    """Convolution + act_calc in one pass.  Returns (int8 [N,H,W,K], exp_out, shift).  scratch_buf: a uint8 tensor of
    conv_fprop_scratch_bytes() bytes owned by the caller instead of the shared scratch; a thin layer's patch matrix
    then survives in its first N*H*W*32 bytes for conv_wgrad_from_patches."""
    _need_cuda(x, w, state, scratch_buf)
    N, H, W, C = x.shape
    K, R, S, _ = w.shape
    y8 = torch.empty((N, H, W, K), dtype=torch.int8, device=x.device)
    exp_out = torch.empty((), dtype=torch.int32, device=x.device)
    shift_out = torch.empty((), dtype=torch.int32, device=x.device)
    nbytes = lib.niti_conv_fprop_scratch_bytes(N, H, W, C, K, R, S)
    sc = (scratch_buf if scratch_buf is not None else scratch(x.device, nbytes)) if nbytes else None
    _call("niti_conv_fprop_requant_i8", 3 if nbytes else 2, 2 * N * H * W * K * R * S * C, x.numel() + w.numel() + y8.numel(),
          lib.niti_conv_fprop_requant_i8, _p(x), _p(w), _p(y8), _p(state), _p(sc), sc.numel() if nbytes else 0,
          N, H, W, C, K, R, S, pad, mode, _p(seed), rng_stream, rng_offset, int(relu), _p(exp_a), _p(exp_b),
          _p(exp_out), _p(shift_out), _p(status_word(x.device)), _st())
    return y8, exp_out, shift_out


def conv_fprop_pool_fused_supported(N, H, W, C, K, R, S, pad):
    return bool(lib.niti_conv_fprop_requant_pool_supported(N, H, W, C, K, R, S, pad))


def conv_fprop_pool_fused(x, w, state, pad=1, mode=ROUND_NEAREST, seed=None, rng_stream=0, rng_offset=0, relu=False,
                          exp_a=None, exp_b=None):
    """Convolution + act_calc (+ ReLU) + 2x2 max pooling in one launch.  Returns (int8 [N,H,W,K], int8 [N,H/2,W/2,K],
    exp_out, shift)."""
    _need_cuda(x, w, state)
    N, H, W, C = x.shape
    K, R, S, _ = w.shape
    y8 = torch.empty((N, H, W, K), dtype=torch.int8, device=x.device)
    yp = torch.empty((N, H // 2, W // 2, K), dtype=torch.int8, device=x.device)
    exp_out = torch.empty((), dtype=torch.int32, device=x.device)
    shift_out = torch.empty((), dtype=torch.int32, device=x.device)
    _call("niti_conv_fprop_requant_pool_i8", 1, 2 * N * H * W * K * R * S * C, x.numel() + w.numel() + y8.numel() + yp.numel(),
          lib.niti_conv_fprop_requant_pool_i8, _p(x), _p(w), _p(y8), _p(yp), _p(state),
          N, H, W, C, K, R, S, pad, mode, _p(seed), rng_stream, rng_offset, int(relu), _p(exp_a), _p(exp_b),
          _p(exp_out), _p(shift_out), _p(status_word(x.device)), _st())
    return y8, yp, exp_out, shift_out


def conv_dgrad_side_bytes(N, H, W, C, K, R, S, pad):
    """Bytes of per-layer side memory conv_dgrad_fused can use for this shape (0: the single-launch kernel serves it)."""
    return int(lib.niti_conv_dgrad_requant_side_bytes(N, H, W, C, K, R, S, pad))


def conv_dgrad_fused(err, w, state, pad=1, mode=ROUND_NEAREST, seed=None, rng_stream=0, rng_offset=0, exp_a=None, exp_b=None,
                     relu_mask=None, side=None):
    """Error-backward convolution + err_calc in one pass (+ the backward of the ReLU in front of the layer when
    relu_mask, the layer's forward input, is given).  side: optional uint8 tensor of conv_dgrad_side_bytes() bytes kept
    with the layer; with it a shift guessed one too high is repaired by a cheap pass instead of a second contraction.
    Returns (int8 [N,H,W,C], exp_out, shift)."""
    _need_cuda(err, w, state, relu_mask, side)
    N, H, W, K = err.shape
    K2, R, S, C = w.shape
    e8 = torch.empty((N, H, W, C), dtype=torch.int8, device=err.device)
    exp_out = torch.empty((), dtype=torch.int32, device=err.device)
    shift_out = torch.empty((), dtype=torch.int32, device=err.device)
    _call("niti_conv_dgrad_requant_i8", 2, 2 * N * H * W * K * R * S * C, err.numel() + w.numel() + e8.numel(),
          lib.niti_conv_dgrad_requant_side_i8, _p(err), _p(w), _p(e8), _p(state), _p(side), side.numel() if side is not None else 0,
          N, H, W, C, K, R, S, pad, mode, _p(seed),
          rng_stream, rng_offset, _p(exp_a), _p(exp_b), _p(exp_out), _p(shift_out), _p(relu_mask),
          _p(status_word(err.device)), _st())
    return e8, exp_out, shift_out


def conv_dgrad_acc(err, w, pad=1):
    """err [N,H,W,K] with the layer's own filters w [K,R,S,C] -> int32 [N,H,W,C] (error w.r.t. the input)."""
    _need_cuda(err, w)
    N, H, W, K = err.shape
    K2, R, S, C = w.shape
    assert K == K2
    e32 = torch.empty((N, H, W, C), dtype=torch.int32, device=err.device)
    mx = torch.empty(1, dtype=torch.int32, device=err.device)
    _call("niti_conv_dgrad_i8", 1, 2 * N * H * W * K * R * S * C, err.numel() + w.numel() + 4 * e32.numel(),
          lib.niti_conv_dgrad_i8, _p(err), _p(w), _p(e32), _p(mx), N, H, W, C, K, R, S, pad,
          _p(status_word(err.device)), _st())
    return e32, mx


def conv_wgrad_acc(x, err, R=3, S=3, pad=1, out=None, want_max=True):
    """Weight gradient accumulators and max|g32| (None when want_max is False: update_multi finds it)."""
    _need_cuda(x, err, out)
    N, H, W, C = x.shape
    K = err.shape[3]
    g32 = out if out is not None else torch.empty((K, R, S, C), dtype=torch.int32, device=x.device)
    mx = torch.empty(1, dtype=torch.int32, device=x.device) if want_max else None
    nbytes = lib.niti_conv_wgrad_scratch_bytes(N, H, W, C, K, R, S)
    sc = scratch(x.device, nbytes)
    _call("niti_conv_wgrad_i8", 2 if C % 16 == 0 else 3, 2 * N * H * W * K * R * S * C, x.numel() + err.numel() + 4 * g32.numel(),
          lib.niti_conv_wgrad_i8, _p(x), _p(err), _p(g32), _p(mx), _p(sc), sc.numel(), N, H, W, C, K, R, S, pad,
          _p(status_word(x.device)), _st())
    return g32, mx


def conv_wgrad_from_patches(patches, err, C, R=3, S=3, out=None, want_max=True):
    """Weight gradient of a thin layer (R*S*C <= 32) from the patch matrix its forward call left in `patches` (see
    conv_fprop_fused(scratch_buf=...)): same result as conv_wgrad_acc on the layer's input, without gathering again."""
    _need_cuda(patches, err, out)
    N, H, W, K = err.shape
    g32 = out if out is not None else torch.empty((K, R, S, C), dtype=torch.int32, device=err.device)
    mx = torch.empty(1, dtype=torch.int32, device=err.device) if want_max else None
    nbytes = lib.niti_conv_wgrad_patches_scratch_bytes(N, H, W, C, K, R, S)
    sc = scratch(err.device, nbytes)
    _call("niti_conv_wgrad_patches_i8", 2, 2 * N * H * W * K * R * S * C, N * H * W * 32 + err.numel() + 4 * g32.numel(),
          lib.niti_conv_wgrad_patches_i8, _p(patches), _p(err), _p(g32), _p(mx), _p(sc), sc.numel(), N, H, W, C, K, R, S,
          _p(status_word(err.device)), _st())
    return g32, mx


def conv_wgrad_accumulate_supported(C, K, R, S, pad):
    return bool(lib.niti_conv_wgrad_accumulate_supported(C, K, R, S, pad))


def conv_wgrad_accumulate(x, err, g32, R=3, S=3, pad=1):
    """g32 += weight gradient (no clearing pass: the caller keeps g32 zeroed between steps, see update_multi)."""
    _need_cuda(x, err, g32)
    N, H, W, C = x.shape
    K = err.shape[3]
    assert g32.dtype == torch.int32 and g32.numel() == K * R * S * C
    _call("niti_conv_wgrad_accumulate_i8", 1, 2 * N * H * W * K * R * S * C, x.numel() + err.numel() + 4 * g32.numel(),
          lib.niti_conv_wgrad_accumulate_i8, _p(x), _p(err), _p(g32), N, H, W, C, K, R, S, pad,
          _p(status_word(x.device)), _st())
    return g32


def conv_wgrad_accumulate_multi_max():
    return int(lib.niti_conv_wgrad_accumulate_multi_max())


def conv_wgrad_accumulate_multi(jobs):
    """[(x, err, g32, R, S, pad), ...] (at most conv_wgrad_accumulate_multi_max() layers): every g32 += its layer's weight
    gradient, all in one launch whose thread blocks are shared out by work."""
    items = (WgradItem * len(jobs))()
    algo_ops = algo_bytes = 0
    for i, (x, err, g32, R, S, pad) in enumerate(jobs):
        _need_cuda(x, err, g32)
        N, H, W, C = x.shape
        K = err.shape[3]
        assert g32.dtype == torch.int32 and g32.numel() == K * R * S * C
        items[i] = WgradItem(_p(x), _p(err), _p(g32), N, H, W, C, K, R, S, pad)
        algo_ops += 2 * N * H * W * K * R * S * C
        algo_bytes += x.numel() + err.numel() + 4 * g32.numel()
    dev = jobs[0][0].device
    _call("niti_conv_wgrad_accumulate_i8", 1, algo_ops, algo_bytes, lib.niti_conv_wgrad_accumulate_multi_i8, items, len(jobs),
          _p(status_word(dev)), _st())


def gemm_acc(a, b, trans_a=False, trans_b=False, out=None):
    """C32[M,N] = op(a) @ op(b); a is [M,K] ([K,M] if trans_a), b is [K,N] ([N,K] if trans_b)."""
    _need_cuda(a, b, out)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    assert (b.shape[1] if trans_b else b.shape[0]) == K
    c32 = out if out is not None else torch.empty((M, N), dtype=torch.int32, device=a.device)
    mx = torch.empty(1, dtype=torch.int32, device=a.device)
    _call("niti_gemm_i8", 1, 2 * M * N * K, a.numel() + b.numel() + 4 * c32.numel(),
          lib.niti_gemm_i8, _p(a), _p(b), _p(c32), _p(mx), M, N, K, int(trans_a), int(trans_b),
          _p(status_word(a.device)), _st())
    return c32, mx


def group_conv1(inp, wt, pad):
    """Grouped cross-correlation, one input channel per group, batch 1: inp [1,H,W,G] int8, wt [G*Kg,R,S,1] int8
    -> int32 [1,P,Q,G*Kg] (what the reference's conv2d_weight_int8 asks of int8conv_cuda.group_conv)."""
    _need_cuda(inp, wt)
    _, H, W, G = inp.shape
    GK, R, S, one = wt.shape
    assert inp.shape[0] == 1 and one == 1 and GK % G == 0 and inp.dtype == torch.int8 and wt.dtype == torch.int8
    P, Q = H + 2 * pad - R + 1, W + 2 * pad - S + 1
    out = torch.empty((1, P, Q, GK), dtype=torch.int32, device=inp.device)
    _call("niti_group_conv1_i8", 1, 2 * GK * P * Q * R * S, inp.numel() + wt.numel() + 4 * out.numel(),
          lib.niti_group_conv1_i8, _p(inp), _p(wt), _p(out), H, W, G, GK // G, R, S, pad, _st())
    return out


# ------------------------------------------------------------------ requantisation
def requant(acc, maxabs, kind, target_bits, mode=ROUND_NEAREST, seed=None, rng_stream=0, rng_offset=0, relu=False,
            exp_a=None, exp_b=None, want_shift=False):
    """int32 -> int8 by the tensor-wide shift.  Returns (out8, exp_out, shift_out)."""
    _need_cuda(acc, maxabs)
    out = torch.empty(acc.shape, dtype=torch.int8, device=acc.device)
    exp_out = torch.empty((), dtype=torch.int32, device=acc.device)
    shift_out = torch.empty((), dtype=torch.int32, device=acc.device) if want_shift else None
    _call("niti_requant_i8", 1, 0, 5 * acc.numel(),
          lib.niti_requant_i8, _p(acc), _p(out), _p(maxabs), acc.numel(), kind, target_bits, mode, _p(seed), rng_stream,
          rng_offset, int(relu), _p(exp_a), _p(exp_b), _p(exp_out), _p(shift_out), _st())
    return out, exp_out, shift_out


def absmax(acc):
    _need_cuda(acc)
    mx = torch.empty(1, dtype=torch.int32, device=acc.device)
    _call("niti_absmax_i32", 1, 0, 4 * acc.numel(), lib.niti_absmax_i32, _p(acc), acc.numel(), _p(mx), _st())
    return mx


# ------------------------------------------------------------------ memory-bound layers
def maxpool_fwd(x, k=2, stride=2):
    _need_cuda(x)
    N, H, W, C = x.shape
    y = torch.empty((N, (H - k) // stride + 1, (W - k) // stride + 1, C), dtype=torch.int8, device=x.device)
    _call("niti_maxpool_fwd_i8", 1, 0, x.numel() + y.numel(), lib.niti_maxpool_fwd_i8, _p(x), _p(y), N, H, W, C, k, stride, _st())
    return y


def maxpool_bwd(x, dy, k=2, stride=2, relu_mask=False):
    """dx of max pooling; relu_mask also applies the backward of the ReLU that produced x (zero where x <= 0)."""
    _need_cuda(x, dy)
    N, H, W, C = x.shape
    dx = torch.empty_like(x)
    _call("niti_maxpool_bwd_i8", 1, 0, 2 * x.numel() + dy.numel(), lib.niti_maxpool_bwd_i8, _p(x), _p(dy), _p(dx), N, H, W, C, k, stride, int(relu_mask), _st())
    return dx


def relu_fwd(x):
    _need_cuda(x)
    y = torch.empty_like(x)
    _call("niti_relu_fwd_i8", 1, 0, 2 * x.numel(), lib.niti_relu_fwd_i8, _p(x), _p(y), x.numel(), _st())
    return y


def relu_bwd(act, err):
    _need_cuda(act, err)
    out = torch.empty_like(err)
    _call("niti_relu_bwd_i8", 1, 0, 3 * err.numel(), lib.niti_relu_bwd_i8, _p(act), _p(err), _p(out), err.numel(), _st())
    return out


def dropout(x, seed, rng_stream):
    _need_cuda(x, seed)
    y = torch.empty_like(x)
    _call("niti_dropout_i8", 1, 0, 2 * x.numel(), lib.niti_dropout_i8, _p(x), _p(y), x.shape[0], x.numel() // x.shape[0],
          _p(seed), rng_stream, _st())
    return y


def loss_err(out8, out_exp, target, seed, rng_stream=0xFFFF, sample_offset=0):
    _need_cuda(out8, out_exp, target, seed)
    assert target.dtype == torch.int64 and out_exp.dtype == torch.int32
    err = torch.empty_like(out8)
    _call("niti_loss_i8", 1, 0, 2 * out8.numel(), lib.niti_loss_i8, _p(out8), _p(out_exp), _p(target), _p(err),
          out8.shape[0], out8.shape[1], _p(seed), rng_stream, sample_offset, _st())
    return err


def fc_head_supported(B, F, J):
    return bool(lib.niti_fc_head_supported(B, F, J))


def fc_head_train(x, exp_x, w, exp_w, target, seed, layer_stream, *, dropout=True, bits=7, act_mode=ROUND_NEAREST,
                  err_mode=ROUND_NEAREST, grad_mode=ROUND_PSEUDO_STOCHASTIC, mu=5, update=True, sample_offset=0,
                  g32=None, dropout_stream=0xFFFE, loss_stream=0xFFFF):
    """Dropout + FC forward + loss error + FC backward (+ update of w in place) in one kernel.
    Returns (out8, exp_out, err8, e8, exp_err, g32, grad_maxabs)."""
    _need_cuda(x, exp_x, w, exp_w, target, seed, g32)
    B, F = x.shape
    J = w.shape[0]
    assert x.dtype == torch.int8 and w.dtype == torch.int8 and target.dtype == torch.int64 and w.shape[1] == F
    dev = x.device
    out8 = torch.empty((B, J), dtype=torch.int8, device=dev)
    err8 = torch.empty((B, J), dtype=torch.int8, device=dev)
    e8 = torch.empty_like(x)
    exps = torch.empty(2, dtype=torch.int32, device=dev)
    if g32 is None:
        g32 = torch.empty((J, F), dtype=torch.int32, device=dev)
    gm = torch.empty(1, dtype=torch.int32, device=dev)
    nbytes = lib.niti_fc_head_scratch_bytes(B, F, J)
    sc = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    a = FcHeadArgs(_p(x), _p(exp_x), _p(w), _p(exp_w), _p(target), _p(out8), exps[0:1].data_ptr(), _p(err8), _p(e8),
                   exps[1:2].data_ptr(), _p(g32), _p(gm), _p(sc), nbytes, B, F, J, int(dropout), bits, act_mode, err_mode,
                   grad_mode, mu, int(update), _p(seed), layer_stream, dropout_stream, loss_stream, sample_offset,
                   _p(status_word(dev)))
    _call("niti_fc_head_train_i8", 1, 6 * B * F * J, 2 * x.numel() + 6 * w.numel(), lib.niti_fc_head_train_i8,
          ctypes.byref(a), _st())
    return out8, exps[0], err8, e8, exps[1], g32, gm


def update(w, g32, maxabs, mu, mode=ROUND_PSEUDO_STOCHASTIC, seed=None, rng_stream=0):
    """In-place integer SGD update of the int8 weights from their int32 gradient accumulators."""
    _need_cuda(w, g32, maxabs)
    _call("niti_update_i8", 1, 0, 6 * w.numel(), lib.niti_update_i8, _p(w), _p(g32), _p(maxabs),
          w.numel(), mu, mode, _p(seed), rng_stream, _st())


def update_multi(ws, g32s, streams, mu, mode=ROUND_PSEUDO_STOCHASTIC, seed=None, want_max=False, clear=False):
    """All layers' integer SGD updates in one launch: per layer max|g32| -> shift -> w -= narrow(g32); `clear`
    also zeroes the accumulators afterwards.  Returns the per-layer maxima (int32[len(ws)]) when want_max."""
    _need_cuda(seed, *ws, *g32s)
    dev = ws[0].device
    n = len(ws)
    mx = torch.empty(n, dtype=torch.int32, device=dev) if want_max else None
    items = (UpdateItem * n)()
    for i, (w, g, st) in enumerate(zip(ws, g32s, streams)):
        assert w.dtype == torch.int8 and g.dtype == torch.int32 and g.numel() == w.numel()
        items[i] = UpdateItem(_p(w), _p(g), mx[i:i + 1].data_ptr() if want_max else None, w.numel(), st)
    nbytes = lib.niti_update_multi_scratch_bytes()
    sc = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    total = sum(w.numel() for w in ws)
    _call("niti_update_multi_i8", (n + 15) // 16, 0, 10 * total, lib.niti_update_multi_i8, items, n, mu, mode, int(clear), _p(seed),
          _p(sc), nbytes, _p(status_word(dev)), _st())
    return mx


def dp_exchange_bytes():
    return int(lib.niti_dp_exchange_bytes())


def dp_update(items, rank, world, weight_ptrs, grad_ptrs, exchange_ptrs, mu, mode, seed, device, maxabs=None):
    """One rank's part of the data-parallel update over peer memory (niti_dp_update_i8): `items` is a list of
    (w_offset bytes, g_offset elements, n, rng_stream); the three pointer lists hold one device address per rank."""
    _need_cuda(seed, maxabs)
    n = len(items)
    arr = (DpItem * n)()
    for i, it in enumerate(items):  # (w_offset, g_offset, n, rng_stream[, staged pointers per rank or None])
        arr[i].w_offset, arr[i].g_offset, arr[i].n, arr[i].rng_stream = int(it[0]), int(it[1]), int(it[2]), int(it[3])
        if len(it) > 4 and it[4] is not None:
            for r, ptr in enumerate(it[4]):
                arr[i].staged[r] = ptr
    vp = ctypes.c_void_p * world
    w, g, x = vp(*weight_ptrs), vp(*grad_ptrs), vp(*exchange_ptrs)
    args = DpUpdateArgs(ctypes.cast(arr, ctypes.c_void_p), n, rank, world, ctypes.cast(w, ctypes.c_void_p),
                        ctypes.cast(g, ctypes.c_void_p), ctypes.cast(x, ctypes.c_void_p), mu, mode, _p(seed), _p(maxabs),
                        _p(status_word(device)))
    total = sum(it[2] for it in items)
    _call("niti_dp_update_i8", 1, 0, 9 * total, lib.niti_dp_update_i8, ctypes.byref(args), _st())


def peer_copy(dst_ptr, src_ptr, nbytes):
    """Device-to-device copy between raw addresses (own or peer-mapped arenas) on the current stream."""
    check(lib.niti_peer_copy(ctypes.c_void_p(dst_ptr), ctypes.c_void_p(src_ptr), nbytes, _st()), "niti_peer_copy")


def quantize_input(x, reduce_max=None):
    """float32 NCHW -> (int8 NHWC, exponent).  ``reduce_max(t)``: optional hook that replaces the int32[1] word
    holding the bit pattern of max|x| by its maximum over a process group, in place."""
    _need_cuda(x)
    assert x.dtype == torch.float32
    N, C, H, W = x.shape
    x8 = torch.empty((N, H, W, C), dtype=torch.int8, device=x.device)
    e = torch.empty((), dtype=torch.int32, device=x.device)
    tmp = torch.empty(1, dtype=torch.int32, device=x.device)
    if reduce_max is not None:
        _call("niti_absmax_f32", 1, 0, 4 * x.numel(), lib.niti_absmax_f32, _p(x), x.numel(), _p(tmp), _st())
        reduce_max(tmp)
        _call("niti_quantize_input_with_max_f32", 1, 0, 5 * x.numel(), lib.niti_quantize_input_with_max_f32, _p(x), _p(x8), _p(e),
              _p(tmp), N, C, H, W, _st())
        return x8, e
    _call("niti_quantize_input_f32", 2, 0, 9 * x.numel(), lib.niti_quantize_input_f32, _p(x), _p(x8), _p(e), _p(tmp), N, C, H, W, _st())
    return x8, e
