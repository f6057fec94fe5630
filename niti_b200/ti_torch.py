"""Drop-in for the reference's ``ti_torch`` module (integer layers of NITI) on the B200 kernels.

Same public names, argument meaning and ``(int8 tensor, exponent)`` tuple convention as the
reference's ti_torch.py; file:line citations below are to that file.  What differs, on purpose:

* exponents and shift amounts are 0-dim ``int32`` CUDA tensors (the reference mixes Python ints
  and float tensors and reads the bit-width back to the host twice per layer, :366-377); nothing
  here synchronises, so a whole training step can be captured in a CUDA graph;
* the four extension modules (``cutlassconv_cuda``, ``int8mm_cuda``, ``int8pool_cuda``,
  ``int8conv_cuda``) are replaced by one C-ABI library (``niti_b200.ops``); there is no CPU or
  PyTorch fallback: without the built library importing this module raises;
* ``//`` follows the torch release the reference was written for (truncation toward zero);
* accumulators are exact int32 (the reference's CUTLASS epilogue rounds through fp32);
* random bits (StoShift, TiDropout) come from a counter-based generator keyed by ``RNG_SEED``
  (a device word, advanced once per training step), a per-layer stream id and the GLOBAL element
  index, so a batch shard draws the bits of its own samples.
"""
import torch
from torch.nn.modules import Module

from . import ops


class UpdateWeight(Module):
    """Parameter update shared by TiConv2d and TiLinear (:11-21)."""

    layer_id = 0          # index among the weighted layers; selects the random-bit streams
    grad_buffer = None    # optional preallocated int32 view the weight gradient is written into
    defer_update = False  # data-parallel trainers sum gradients across ranks before updating
    grad_accumulate = False  # the weight gradient is ADDED into grad_buffer, which weight_update_all zeroes after use
    wgrad_stream = None      # optional side stream for the (accumulating) weight-gradient kernel; the owner joins it
    grad_ready = None     # optional callback(layer), called as soon as grad_int32acc has been enqueued

    def weight_update(self):
        """vanilla SGD on int8 weights: w <- clamp(w - grad_calc(grad_int32acc, GRAD_BITWIDTH))"""
        ops.update(self.weight, self.grad_int32acc, self.grad_maxabs, GRAD_BITWIDTH, _mode(GRAD_ROUND_METHOD),
                   RNG_SEED(self.weight.device), 16 * self.layer_id + 2)


def weight_update_all(layers, clear=False):
    """The updates of all `layers` (UpdateWeight modules whose grad_int32acc is set) in one launch; each
    layer's maximum is recomputed from its accumulators, so this also serves gradients summed across ranks.
    `clear` zeroes the accumulators afterwards (layers with grad_accumulate add into them at the next step)."""
    dev = layers[0].weight.device
    ops.update_multi([l.weight for l in layers], [l.grad_int32acc for l in layers], [16 * l.layer_id + 2 for l in layers],
                     GRAD_BITWIDTH, _mode(GRAD_ROUND_METHOD), RNG_SEED(dev), clear=clear)


def _fake_max(shift):
    # a max|x| whose bit-width is exactly shift + BITWIDTH, so the kernel picks `shift`
    return 1 << (shift + BITWIDTH)


def _shift_with(mode, input, shift, stream=0):
    if shift <= 0:
        raise ValueError("shift must be positive")
    mx = torch.full((1,), _fake_max(shift), dtype=torch.int32, device=input.device)
    out, _, _ = ops.requant(input.contiguous(), mx, ops.CALC_ACT, BITWIDTH, mode, RNG_SEED(input.device), stream)
    return out


def RoundShift(input, shift):
    """Shift right with round-half-away-from-zero, clamp to +-127 (:23-31)."""
    return _shift_with(ops.ROUND_NEAREST, input, shift)


def StoShift(input, shift):
    """Shift right with stochastic rounding (:33-46); random bits from the keyed generator."""
    return _shift_with(ops.ROUND_STOCHASTIC, input, shift)


def PstoShift(input, shift):
    """Shift right with pseudo-stochastic rounding: the dropped low bits are the random number (:48-69)."""
    return _shift_with(ops.ROUND_PSEUDO_STOCHASTIC, input, shift)


def _mode(method):
    return {RoundShift: ops.ROUND_NEAREST, StoShift: ops.ROUND_STOCHASTIC, PstoShift: ops.ROUND_PSEUDO_STOCHASTIC}[method]


def int8_clip(input, clip_val=127):
    return torch.clamp(input, -clip_val, clip_val).type(torch.int8)


def Int8Tensor(val):
    return torch.tensor(val, dtype=torch.int8).to(GPU)


def Int8zeros(size):
    return torch.zeros(size=size, dtype=torch.int8, device=GPU)


def exp_tensor(e, device=None):
    """Exponent as a 0-dim int32 tensor on the device (accepts ints, floats, tensors)."""
    device = device or GPU
    if isinstance(e, torch.Tensor):
        return e.to(device=device, dtype=torch.int32).reshape(())
    return torch.full((), int(e), dtype=torch.int32, device=device)  # a fill kernel: legal under graph capture


def UniformWeights(size):
    """xavier-uniform float init on the host, then weight_quant (:77-85)."""
    if len(size) == 4:
        temp = torch.zeros(size).permute(0, 3, 1, 2).contiguous()
        torch.nn.init.xavier_uniform_(temp)
        return weight_quant(temp.permute(0, 2, 3, 1).contiguous())
    temp = torch.zeros(size)
    torch.nn.init.xavier_uniform_(temp)
    return weight_quant(temp)


def NormalWeight(size):
    if len(size) == 4:
        temp = torch.zeros(size).permute(0, 3, 1, 2).contiguous()
        torch.nn.init.xavier_normal_(temp)
        return weight_quant(temp.permute(0, 2, 3, 1).contiguous())
    temp = torch.zeros(size)
    torch.nn.init.xavier_normal_(temp)
    return weight_quant(temp)


def weight_quant(input):
    """float weights -> (int8 on the device, exponent) (:334-339); setup only, runs on the host."""
    input_range = torch.max(torch.abs(input))
    input_bitwidth = torch.ceil(torch.log2(input_range))
    act_exp = input_bitwidth - 7
    round_val = torch.round(input / input_range * (2 ** 7 - 1)).type(torch.int8).to(GPU)
    return round_val, exp_tensor(act_exp)


def _global_max(word):
    """Global-exact data-parallel mode: replace a max word by its maximum over GLOBAL_MAX_GROUP, in place."""
    import torch.distributed as dist
    dist.all_reduce(word, op=dist.ReduceOp.MAX, group=None if GLOBAL_MAX_GROUP is True else GLOBAL_MAX_GROUP)


def _calc(int32_acc, kind, target_bits, method, stream, exp_a=None, exp_b=None, maxabs=None, relu=False, offset=0):
    acc = int32_acc.contiguous()
    if maxabs is None:
        maxabs = ops.absmax(acc)
    if GLOBAL_MAX_GROUP is not None and kind != ops.CALC_GRAD:
        _global_max(maxabs)  # activations / errors of the whole (sharded) batch share one shift
    return ops.requant(acc, maxabs, kind, target_bits, _mode(method), RNG_SEED(acc.device), stream, offset,
                       relu=relu, exp_a=exp_a, exp_b=exp_b, want_shift=True)


def act_calc(int32_acc, exp_in, maxabs=None, rng_stream=0, relu=False, rng_offset=0, exp_b=None):
    """int32 accumulators -> (int8, exp_out) by the tensor's bit-width (:103-117)."""
    out, exp_out, _ = _calc(int32_acc, ops.CALC_ACT, BITWIDTH, ACT_ROUND_METHOD, rng_stream,
                            exp_tensor(exp_in, int32_acc.device), exp_b, maxabs, relu, rng_offset)
    return out, exp_out


def err_calc(int32_acc, maxabs=None, rng_stream=0, rng_offset=0):
    """int32 accumulators -> (int8, shift) (:119-133)."""
    out, _, shift = _calc(int32_acc, ops.CALC_ERR, BITWIDTH, ERROR_ROUND_METHOD, rng_stream, None, None, maxabs, False, rng_offset)
    return out, shift


def grad_calc(int32_acc, mu, maxabs=None, rng_stream=0):
    """int32 gradient accumulators -> (int8, shift) with target bit-width mu (:135-147)."""
    out, _, shift = _calc(int32_acc, ops.CALC_GRAD, mu, GRAD_ROUND_METHOD, rng_stream, None, None, maxabs)
    return out, shift


def roundoff4(size):
    return (size + 3) // 4 * 4


def int8mm(lhs, rhs):
    """[m,k] int8 @ [k,n] int8 -> int32 [m,n] (:152-176); no padding to multiples of 4 is needed."""
    return ops.gemm_acc(lhs.contiguous(), rhs.contiguous())[0]


def conv2d_int8(input, weight, stride=1, padding=1):
    """NHWC int8 conv -> int32 (:178-192); any channel count (the reference pads C to 16)."""
    return ops.conv_fprop_acc(input.contiguous(), weight.contiguous(), padding, stride)[0]


def conv2d_weight_int8(input, weight_size, grad_output, stride=1, padding=0, dilation=1):
    """Weight gradient of a convolution -> int32 [K,R,S,C] (:194-233); exact integers, any batch size."""
    if stride != 1 or dilation != 1:
        raise RuntimeError("conv2d_weight_int8: only stride 1 / dilation 1 are implemented")
    return ops.conv_wgrad_acc(input.contiguous(), grad_output.contiguous(), weight_size[1], weight_size[2], padding)[0]


class TiLinear(UpdateWeight):
    def __init__(self, in_features, out_features, last_layer=False):
        super(TiLinear, self).__init__()
        self.weight, self.weight_exp = WEIGHT_INIT_METHOD(torch.Size([out_features, in_features]))
        self.last_layer = last_layer

    def forward(self, input):
        """(act int8 [B,in], exp) -> (act int8 [B,out], exp) (:241-253)"""
        self.act_in = input
        act_in, exp_in = input
        acc, mx = ops.gemm_acc(act_in, self.weight, trans_b=True)
        per = acc.shape[1]
        return act_calc(acc, exp_in, mx, 16 * self.layer_id, rng_offset=SAMPLE_OFFSET * per, exp_b=self.weight_exp)

    def backward(self, input):
        """(err int8 [B,out], exp) -> (err int8 [B,in], exp); updates the weights (:255-266)"""
        err_in, err_exp = input
        act, self.act_in_exp = self.act_in
        acc, mx = ops.gemm_acc(err_in, self.weight)
        err_out, self.err_exp, _ = _calc(acc, ops.CALC_ERR, BITWIDTH, ERROR_ROUND_METHOD, 16 * self.layer_id + 1,
                                         exp_tensor(err_exp, acc.device), self.weight_exp, mx, False,
                                         SAMPLE_OFFSET * acc.shape[1])
        self.grad_int32acc, self.grad_maxabs = ops.gemm_acc(err_in, act, trans_a=True, out=self.grad_buffer)
        if self.grad_ready is not None:
            self.grad_ready(self)
        if not self.defer_update:
            self.weight_update()
        return err_out, self.err_exp


class TiReLU(Module):
    """Integer ReLU (:268-290).  ``fused=True`` marks a ReLU whose forward was already applied by
    the preceding convolution's requantisation; backward is the same either way because
    x > 0 exactly where max(x, 0) > 0."""

    def __init__(self, fused=False):
        super(TiReLU, self).__init__()
        self.fused = fused
        # set by a model builder when the next layer (a TiMaxpool2d or TiConv2d with relu_backward_fused) applies
        # this ReLU's backward mask itself
        self.backward_in_next_layer = False

    def forward(self, input):
        act_in, exp_in = input
        act_out = act_in if self.fused else ops.relu_fwd(act_in)
        self.act_in = (act_out if self.fused else act_in, exp_in)
        return act_out, exp_in

    def backward(self, input):
        err_in, err_exp = input
        if self.backward_in_next_layer:
            return err_in, err_exp
        act, _ = self.act_in
        return ops.relu_bwd(act, err_in.contiguous()), err_exp


class TiMaxpool2d(Module):
    """Integer max pooling (:292-316), int8 in both directions."""

    def __init__(self, kernel_size, stride, padding=0):
        super(TiMaxpool2d, self).__init__()
        if padding != 0:
            raise RuntimeError("TiMaxpool2d: padding is not implemented (the reference models use 0)")
        self.kernel_size = kernel_size
        self.stride = stride
        self.padding = padding
        # True when this layer's input is the output of a TiReLU whose backward mask is applied here
        # (x > 0 on the ReLU's output exactly where its input was > 0): one pass instead of two
        self.relu_backward_fused = False
        # (input tensor, pooled tensor) left by a convolution whose kernel already pooled its output
        self.precomputed = None

    def forward(self, input):
        self.act_in, exp_in = input
        pre, self.precomputed = self.precomputed, None
        if pre is not None and pre[0] is self.act_in:
            self.act_out = pre[1]
        else:
            self.act_out = ops.maxpool_fwd(self.act_in, self.kernel_size, self.stride)
        return self.act_out, exp_in

    def backward(self, input):
        err_in, err_exp = input
        return ops.maxpool_bwd(self.act_in, err_in.contiguous(), self.kernel_size, self.stride,
                               self.relu_backward_fused), err_exp


class TiFlat(Module):
    """Flatten everything but the batch dimension (:318-332)."""

    def forward(self, input):
        self.act_in = input
        act_in, exp_in = input
        return act_in.view(-1, act_in.nelement() // act_in.size(0)), exp_in

    def backward(self, input):
        err_in, err_exp = input
        act, _ = self.act_in
        return err_in.view_as(act), err_exp


def TiFloatToInt8(input):
    """float tensor -> (int8, exponent) with exponent = ceil(log2(max|x|)) - 7 (:341-356).
    4-D inputs are taken as NCHW and returned NHWC (the permute of ti_net.py:19 is fused in)."""
    x = input.to(GPU, dtype=torch.float32).contiguous()
    hook = _global_max if GLOBAL_MAX_GROUP is not None else None
    if x.dim() == 4:
        return ops.quantize_input(x, hook)
    q, e = ops.quantize_input(x.reshape(1, 1, 1, -1), hook)
    return q.reshape(x.shape), e


def TiInt8ToFloat(input):
    act_in, exp_in = input
    return act_in.float() * (2 ** (exp_tensor(exp_in, act_in.device).float()))


def TensorBitwidth(val):
    m = int(val)
    return 0 if m == 0 else (m - 1).bit_length()


def RangeEstimate(input):
    """Bit-width of max|x| (:366-377) as a Python int.  Synchronises: for inspection, not the hot path."""
    return TensorBitwidth(ops.absmax(input.contiguous().to(torch.int32)).item())


# weight gradients waiting for company: layers that run their gradient on a side stream hand it in here, and every
# WGRAD_GROUP of them go out as ONE launch (ops.conv_wgrad_accumulate_multi), issued when the last one's inputs exist
_WGRAD_PENDING = []
# called after a FULL group has been launched, with (stream, layers of the group): behind that launch on `stream` the
# gradients of these layers are complete while most of the backward pass is still to come.  A data-parallel trainer
# starts moving them to their owners there.
WGRAD_FLUSH_HOOK = None


def flush_wgrad(full_group=False):
    """Launch the weight gradients collected so far (a group that filled up, a layer without a successor in its group,
    the end of a step)."""
    if not _WGRAD_PENDING:
        return
    stream, fork = _WGRAD_PENDING[-1][0], _WGRAD_PENDING[-1][1]  # the last layer's inputs are the last to be enqueued
    jobs = [j for _, _, j, _ in _WGRAD_PENDING]
    layers = [l for _, _, _, l in _WGRAD_PENDING]
    del _WGRAD_PENDING[:]
    stream.wait_event(fork)
    with torch.cuda.stream(stream):
        if len(jobs) == 1:
            ops.conv_wgrad_accumulate(*jobs[0])
        else:
            ops.conv_wgrad_accumulate_multi(jobs)
    if full_group and WGRAD_FLUSH_HOOK is not None:
        WGRAD_FLUSH_HOOK(stream, layers)


class TiConv2d(UpdateWeight):
    """3x3 (or RxR) convolution, stride 1, NHWC (:379-437).  ``fuse_relu`` applies the following
    TiReLU inside the requantisation kernel (pair it with ``TiReLU(fused=True)``)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=1, first_layer=False, fuse_relu=False):
        super(TiConv2d, self).__init__()
        self.weight, self.weight_exp = WEIGHT_INIT_METHOD(torch.Size([out_channels, kernel_size, kernel_size, in_channels]))
        self.first_layer = first_layer
        self.stride = stride
        self.padding = padding
        self.fuse_relu = fuse_relu
        # True when this layer's input is the output of a TiReLU whose backward mask this layer's error-backward
        # kernel applies (set by a model builder together with that TiReLU's backward_in_next_layer)
        self.relu_backward_fused = False
        # the TiMaxpool2d that follows this layer's (fused) ReLU, when a model builder found one: where the kernel
        # can, the forward launch also writes the pooled tensor and hands it to that layer
        self.pool_layer = None
        # shift predictions of the fused conv + requantisation kernels (forward, error-backward)
        self._fwd_state = None
        self._bwd_state = None
        self._bwd_side, self._bwd_side_shape = None, None
        self._patches, self._patches_of = None, None

    def forward(self, input):
        self.act, self.act_in_exp = input
        K, R, S, C = self.weight.shape
        per = self.act.shape[1] * self.act.shape[2] * K
        if FUSE_REQUANT and GLOBAL_MAX_GROUP is None and self.stride == 1 and ops.conv_fprop_fused_supported(C, K, R, S, self.padding):
            # conv2d_int8 + act_calc (:393-395) in one kernel; see ops.conv_fprop_fused
            if self._fwd_state is None:
                self._fwd_state = ops.new_requant_state(self.act.device)
            pool = self.pool_layer
            if (pool is not None and FUSE_POOL and self.fuse_relu and pool.kernel_size == 2 and pool.stride == 2
                    and ops.conv_fprop_pool_fused_supported(*self.act.shape, K, R, S, self.padding)):
                # conv2d_int8 + act_calc + ReLU (:393-395, :268-277) and the pool's forward (:302-307) in one kernel
                out, pooled, exp_out, _ = ops.conv_fprop_pool_fused(self.act, self.weight, self._fwd_state, self.padding,
                                                                    _mode(ACT_ROUND_METHOD), RNG_SEED(self.act.device),
                                                                    16 * self.layer_id, SAMPLE_OFFSET * per, True,
                                                                    exp_tensor(self.act_in_exp, self.act.device), self.weight_exp)
                pool.precomputed = (out, pooled)
                return out, exp_out
            self._patches_of = None
            if TRAINING and KEEP_PATCHES and self.first_layer:
                # a thin layer runs as a GEMM over a patch matrix; kept in memory of its own it also serves the weight
                # gradient of this step (the reference gathers its first-layer operands twice, :412-428)
                nbytes = ops.conv_fprop_scratch_bytes(*self.act.shape, K, R, S)
                if nbytes:
                    if self._patches is None or self._patches.numel() < nbytes or self._patches.device != self.act.device:
                        self._patches = torch.empty(nbytes, dtype=torch.uint8, device=self.act.device)
                    self._patches_of = self.act
            out, exp_out, _ = ops.conv_fprop_fused(self.act, self.weight, self._fwd_state, self.padding, _mode(ACT_ROUND_METHOD),
                                                   RNG_SEED(self.act.device), 16 * self.layer_id, SAMPLE_OFFSET * per,
                                                   self.fuse_relu, exp_tensor(self.act_in_exp, self.act.device), self.weight_exp,
                                                   scratch_buf=self._patches if self._patches_of is not None else None)
            return out, exp_out
        acc, mx = ops.conv_fprop_acc(self.act, self.weight, self.padding, self.stride)
        return act_calc(acc, self.act_in_exp, mx, 16 * self.layer_id, self.fuse_relu, SAMPLE_OFFSET * per, self.weight_exp)

    def backward(self, input):
        err_in, self.err_exp = input
        err_in = err_in.contiguous()
        err_out = None
        fork = None
        if self.wgrad_stream is not None and not self.first_layer:
            fork = torch.cuda.Event()
            fork.record()  # the weight gradient needs only what has been enqueued up to here
        if not self.first_layer:
            # the reference builds flip(w).transpose(0,3) here (:404); the kernels read w in place
            K, R, S, C = self.weight.shape
            per = self.act[0].numel()
            if FUSE_REQUANT and GLOBAL_MAX_GROUP is None and ops.conv_dgrad_fused_supported(C, K, R, S, self.padding):
                if self._bwd_state is None:
                    self._bwd_state = ops.new_requant_state(err_in.device)
                n, h, w_ = err_in.shape[:3]
                if STEP_DOWN_CODES and (self._bwd_side is None or self._bwd_side_shape != (n, h, w_)):
                    # layers whose output does not fit in tensor memory guess their shift; two more bits per output
                    # make a guess one too high a cheap repair instead of a second contraction
                    nbytes = ops.conv_dgrad_side_bytes(n, h, w_, C, K, R, S, self.padding)
                    self._bwd_side = torch.empty(nbytes, dtype=torch.uint8, device=err_in.device) if nbytes else None
                    self._bwd_side_shape = (n, h, w_)
                err_out, self.err_exp, _ = ops.conv_dgrad_fused(err_in, self.weight, self._bwd_state, self.padding,
                                                                _mode(ERROR_ROUND_METHOD), RNG_SEED(err_in.device),
                                                                16 * self.layer_id + 1, SAMPLE_OFFSET * per,
                                                                exp_tensor(self.err_exp, err_in.device), self.weight_exp,
                                                                relu_mask=self.act if self.relu_backward_fused else None,
                                                                side=self._bwd_side if STEP_DOWN_CODES else None)
            else:
                acc, mx = ops.conv_dgrad_acc(err_in, self.weight, self.padding)
                err_out, self.err_exp, _ = _calc(acc, ops.CALC_ERR, BITWIDTH, ERROR_ROUND_METHOD, 16 * self.layer_id + 1,
                                                 exp_tensor(self.err_exp, acc.device), self.weight_exp, mx, False,
                                                 SAMPLE_OFFSET * per)
                if self.relu_backward_fused:
                    err_out = ops.relu_bwd(self.act, err_out)
        K, R, S, C = self.weight.shape
        if self.first_layer:
            flush_wgrad()
        if (self.grad_accumulate and self.defer_update and self.grad_buffer is not None
                and ops.conv_wgrad_accumulate_supported(C, K, R, S, self.padding)):
            if fork is not None:
                # error-backward and weight gradient are independent: on two streams the SMs one kernel leaves idle
                # (its last wave, its epilogue) are taken by the other
                self._wgrad_inputs = (self.act, err_in)  # referenced until the owner of the side stream has joined it
                _WGRAD_PENDING.append((self.wgrad_stream, fork, (self.act, err_in, self.grad_buffer, R, S, self.padding), self))
                if len(_WGRAD_PENDING) >= min(WGRAD_GROUP, ops.conv_wgrad_accumulate_multi_max()):
                    flush_wgrad(full_group=True)
                self.grad_int32acc, self.grad_maxabs = self.grad_buffer, None
            else:
                self.grad_int32acc, self.grad_maxabs = ops.conv_wgrad_accumulate(self.act, err_in, self.grad_buffer, R, S, self.padding), None
        elif getattr(self, "_patches_of", None) is self.act and self._patches is not None:
            # the patch matrix of this step's forward pass is still there
            self.grad_int32acc, self.grad_maxabs = ops.conv_wgrad_from_patches(self._patches, err_in, C, R, S, out=self.grad_buffer,
                                                                               want_max=not self.defer_update)
            self._patches_of = None
        else:
            # a deferred update finds max|g| itself (weight_update_all)
            self.grad_int32acc, self.grad_maxabs = ops.conv_wgrad_acc(self.act, err_in, R, S, self.padding, out=self.grad_buffer,
                                                                      want_max=not self.defer_update)
        if self.grad_ready is not None:
            self.grad_ready(self)
        if not self.defer_update:
            self.weight_update()
        if not self.first_layer:
            return err_out, self.err_exp


class TiDropout(Module):
    """Integer dropout (:439-455): one Bernoulli(1/2) bit per feature, shared by the whole batch."""

    def forward(self, input):
        if TRAINING:
            act_in, exp_in = input
            self.seed_used = RNG_SEED(act_in.device).clone()
            return ops.dropout(act_in.contiguous(), self.seed_used, 0xFFFE), exp_tensor(exp_in, act_in.device) + 1
        return input

    def backward(self, input):
        err_in, err_exp = input
        return ops.dropout(err_in.contiguous(), self.seed_used, 0xFFFE), err_exp


# ------------------------------------------------------------------------------------- globals
GPU = 'cuda'
BITWIDTH = 7

ACT_ROUND_METHOD = RoundShift
ERROR_ROUND_METHOD = RoundShift

GRAD_ROUND_METHOD = PstoShift
WEIGHT_INIT_METHOD = UniformWeights

FUSE_REQUANT = True    # convolutions narrow to int8 inside their own kernel (predicted shift, verified, redone if wrong)
STEP_DOWN_CODES = True  # error-backward layers that guess their shift keep two more bits per output (see ops.conv_dgrad_fused)
WGRAD_GROUP = 4        # side-stream weight gradients leave in groups of this many layers, one launch per group
KEEP_PATCHES = True    # the first layer's patch matrix is kept from the forward pass for its weight gradient
FUSE_POOL = True       # conv -> ReLU -> 2x2 pool: the convolution's kernel also writes the pooled tensor where it can
FUSE_HEAD = True       # TiNet.train_step runs [dropout,] FC, loss, FC backward and update as one kernel
GRAD_BITWIDTH = 5      # the reference's training loop injects this per epoch (main.py:73-77)
TRAINING = True        # likewise (main.py:147-149)
SAMPLE_OFFSET = 0      # global index of this process's first sample (data-parallel shards)
# Global-exact data-parallel mode: a torch.distributed group (or True for the default group).  Every tensor-wide
# maximum behind an activation / error shift (and the input quantisation) is MAX-reduced over the group, so k ranks on
# shards of a batch compute exactly what one rank computes on the whole batch.  The convolutions then take the
# two-pass route (int32 accumulators, all-reduce of one word, requantise) and the classifier head runs layer by layer.
GLOBAL_MAX_GROUP = None

_seed_words = {}


def RNG_SEED(device=None):
    """The device word (int64[1]) that keys the random bits on ``device``."""
    dev = torch.device(device or GPU)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    if dev.index not in _seed_words:
        _seed_words[dev.index] = torch.zeros(1, dtype=torch.int64, device=dev)
    return _seed_words[dev.index]


def set_seed(value, device=None):
    RNG_SEED(device).fill_(int(value))


def advance_seed(device=None):
    """Next training step: a device-side increment, safe inside CUDA-graph capture."""
    RNG_SEED(device).add_(1)
