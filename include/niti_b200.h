/*
 * niti_b200 -- C ABI of the B200 (sm_100a) kernels behind NITI's int8 training path.
 *
 * One shared library replaces the reference's four PyTorch extensions
 * (pytorch/cutlass-extension, pytorch/int8mm-extension, pytorch/int8pool-extension,
 * pytorch/int8conv-extension) and the element-wise torch code of ti_torch.py / ti_loss.py
 * that sits between their calls.  File:line citations name the reference interface each
 * entry point stands in for.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host;
 *   - activations / errors are int8 NHWC, conv weights int8 [K][R][S][C], FC weights [out][in];
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it on the CURRENT device,
 *     nothing synchronises the host, nothing is allocated, nothing calls exit();
 *   - every function returns 0 on success or a negative NITI_ERR_* code
 *     (niti_strerror gives the text); CUDA launch errors come back as NITI_ERR_CUDA;
 *   - `status` is a device int32[4] the tensor-core kernels write when a bounded wait inside
 *     them expires (word 0: error code, 1: block, 2: role, 3: detail); zero it once, read it
 *     whenever the host synchronises anyway.  It may be NULL.
 *   - `maxabs` words are REDUCED INTO with an unsigned atomic max: the contraction entry points
 *     clear them on the stream before launching their kernel.
 *   - exponents and shifts live on the device as int32 scalars so that a training step never
 *     has to synchronise (the reference reads them back twice per layer, ti_torch.py:366-377).
 *   - `seed` arguments are device pointers to one uint64 that the kernel reads when it runs, so a
 *     step captured in a CUDA graph draws fresh random bits after the host (or a kernel in the
 *     graph) advances the word.
 */
#ifndef NITI_B200_H
#define NITI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NITI_API __attribute__((visibility("default")))
#else
#define NITI_API
#endif

#define NITI_OK 0
#define NITI_ERR_BAD_ARG (-1)      /* null pointer, non-positive size, misaligned pointer */
#define NITI_ERR_UNSUPPORTED (-2)  /* shape outside what the kernels implement (message says which) */
#define NITI_ERR_CUDA (-3)         /* a CUDA runtime / driver call failed; see niti_last_cuda_error */
#define NITI_ERR_SCRATCH (-4)      /* scratch buffer too small */
#define NITI_ERR_TOO_LARGE (-5)    /* needs more scratch than the library's built-in buffer (see below) */

/* rounding of the int32 -> int8 shift: RoundShift / StoShift / PstoShift (ti_torch.py:23-69) */
#define NITI_ROUND_NEAREST 0
#define NITI_ROUND_STOCHASTIC 1
#define NITI_ROUND_PSEUDO_STOCHASTIC 2

/* which of act_calc / err_calc / grad_calc (ti_torch.py:103-147) picks the shift */
#define NITI_CALC_ACT 0
#define NITI_CALC_ERR 1
#define NITI_CALC_GRAD 2

/* Process-wide tuning switch; returns the previous value (or NITI_ERR_BAD_ARG for an unknown option).
 * NITI_OPT_ACCUMULATOR_PARKING (default 1): let the fused conv + requantisation entry points use the
 * single-launch kernel that keeps all accumulators in tensor memory across a grid barrier whenever
 * the problem is small enough; 0 forces the predict / verify / redo kernels.  Results are identical. */
#define NITI_OPT_ACCUMULATOR_PARKING 1
/* NITI_OPT_WGRAD_TMA_REDUCE (default 1): the tensor-core weight gradient adds every thread block's tiles
 * straight into the zeroed gradient with TMA reductions at the L2; 0: partial sums per pixel range go to
 * scratch and a second kernel folds them.  Same integers either way. */
#define NITI_OPT_WGRAD_TMA_REDUCE 2
/* NITI_OPT_STAGE_CAP (default 0 = all): use at most this many shared-memory stages in the GEMM / conv
 * main loops (measurement aid: separates latency-bound from bandwidth-bound behaviour). */
#define NITI_OPT_STAGE_CAP 3
/* NITI_OPT_CTA_PAIRS (bit 0: GEMMs, bit 1: convolutions; default 1): run the kernels as pairs of
 * thread blocks that issue 256-row MMAs together (tcgen05 cta_group::2), each fetching half of the B
 * operand, which cuts the L2 -> shared-memory traffic per output; 0: one thread block per 128-row tile. */
#define NITI_OPT_CTA_PAIRS 4
/* NITI_OPT_COOPERATIVE_LAUNCH (default 1): the kernels that contain a grid barrier (accumulator parking,
 * classifier head, multi-layer update) are launched cooperatively, i.e. the driver guarantees that all their
 * thread blocks are resident together.  0: plain launches of the same one-wave grids; a barrier that is not met
 * (something else held SMs for more than 0.5 s) then ends in the status word's error, never in a hang. */
#define NITI_OPT_COOPERATIVE_LAUNCH 5
NITI_API int niti_set_option(int option, int value);

NITI_API int niti_version(void);
NITI_API const char* niti_strerror(int code);
/* text of the last CUDA error seen by this thread inside the library ("" if none) */
NITI_API const char* niti_last_cuda_error(void);

/* ---------------------------------------------------------------- contractions (int8 x int8 -> int32)
 *
 * niti_conv_fprop_i8: cutlassconv_cuda.sp_conv_optimized / sp_conv (cutlassconv.cpp:57-73,
 * cutlassconv_kernel.cu:38-319) as called from conv2d_int8 (ti_torch.py:178-192).
 * x [N][H][W][C], w [K][R][S][C] -> y32 [N][P][Q][K], cross-correlation, stride 1, P = H+2*pad-R+1.
 * Unlike the reference no channel padding to 16 is needed (C = 3 is accepted).  *maxabs = max |y32|.
 * Kernel choice: implicit GEMM on the tensor cores when C % 16 == 0 (and R = S = 2*pad+1, K % 4 == 0);
 * R*S*C <= 32 (3-channel first layer) goes through a patch matrix in `scratch`
 * (niti_conv_fprop_scratch_bytes, 0 for the other paths; scratch may then be NULL) and the
 * tensor-core GEMM; anything else runs on CUDA cores.
 */
NITI_API size_t niti_conv_fprop_scratch_bytes(int N, int H, int W, int C, int K, int R, int S);
NITI_API int niti_conv_fprop_i8(const int8_t* x, const int8_t* w, int32_t* y32, uint32_t* maxabs,
                       void* scratch, size_t scratch_bytes,
                       int N, int H, int W, int C, int K, int R, int S, int pad, int stride,
                       int32_t* status, void* stream);

/* cutlassconv_cuda.int4_conv / int4_conv_optimized (cutlassconv.cpp:83-97, cutlassconv_kernel.cu:602-884), which the
 * reference exports but never calls from ti_torch.py: a 3x3 (RxS) convolution of int4 operands packed two per byte along
 * the channels, element 2i in the low nibble (CUTLASS' int4b_t arrays, include/cutlass/array_subbyte.h:116-124), signed.
 * x4 [N][H][W][C2] bytes = 2*C2 channels, w4 [K][R][S][C2] -> y32 [N][P][Q][K] exact int32 (the reference's epilogue
 * saturates, which cannot trigger: |sum| <= 64*R*S*2*C2), stride 1.  The tensor cores of this part have no int4 integer
 * MMA (tcgen05 kind::i8 takes 8-bit integers): the operands are widened to int8 in `scratch` and go through
 * niti_conv_fprop_i8's kernels.  Parity unpinned at the nibble order: the reference has no caller and no test for it. */
NITI_API size_t niti_conv_fprop_i4_scratch_bytes(int N, int H, int W, int C2, int K, int R, int S);
NITI_API int niti_conv_fprop_i4(const uint8_t* x4, const uint8_t* w4, int32_t* y32, uint32_t* maxabs,
                       void* scratch, size_t scratch_bytes,
                       int N, int H, int W, int C2, int K, int R, int S, int pad,
                       int32_t* status, void* stream);

/* Error back-propagation of a convolution: TiConv2d.backward's
 * conv2d_int8(err, flip(w,[1,2]).transpose(0,3)) (ti_torch.py:403-405) WITHOUT the flipped,
 * transposed copy of the weights: the kernel reads w [K][R][S][C] in place (as the reduction
 * operand, taps mirrored).  err [N][H][W][K] -> e32 [N][H][W][C]; R = S = 2*pad+1.
 * Tensor cores when K % 16 == 0 and C % 16 == 0.
 */
NITI_API int niti_conv_dgrad_i8(const int8_t* err, const int8_t* w, int32_t* e32, uint32_t* maxabs,
                       int N, int H, int W, int C, int K, int R, int S, int pad,
                       int32_t* status, void* stream);

/* Weight gradient of a convolution: the transposed-operand conv of ti_torch.py:429-432 and the
 * first-layer group-conv form conv2d_weight_int8 (ti_torch.py:194-233, int8conv_kernel.cu:248-334):
 * g32[k][r][s][c] = sum_{n,p,q} err[n][p][q][k] * x[n][p+r-pad][q+s-pad][c], exact int32, read
 * straight from the NHWC tensors (no transposes).  On the tensor-core paths the reduction over
 * pixels is split across thread blocks, which add their tiles into g32 with TMA reductions (exact,
 * order-independent); the first-layer path and the NITI_OPT_WGRAD_TMA_REDUCE = 0 mode put partial
 * sums in `scratch` (niti_conv_wgrad_scratch_bytes) and fold them.  *maxabs = max |g32|; maxabs may
 * be null when the caller finds the maximum later (niti_update_multi_i8 does).
 */
NITI_API size_t niti_conv_wgrad_scratch_bytes(int N, int H, int W, int C, int K, int R, int S);
NITI_API int niti_conv_wgrad_i8(const int8_t* x, const int8_t* err, int32_t* g32, uint32_t* maxabs,
                       void* scratch, size_t scratch_bytes,
                       int N, int H, int W, int C, int K, int R, int S, int pad,
                       int32_t* status, void* stream);

/* The weight gradient of a thin layer (R*S*C <= 32: the 3-channel first layer) from the patch matrix that the
 * layer's forward call already built: niti_conv_fprop_i8 / niti_conv_fprop_requant_i8 leave it in the first
 * N*H*W*32 bytes of THEIR scratch ([pixel][32]: the R*S*C bytes of the pixel's receptive field, zero padded), so a
 * caller that gives the forward call a scratch buffer of its own and keeps it until the backward pass saves the
 * second gather (TiConv2d.backward's first-layer branch, ti_torch.py:412-428, rebuilds its operands from the input
 * every time).  Same result as niti_conv_wgrad_i8 on the layer's input.  scratch:
 * niti_conv_wgrad_patches_scratch_bytes() bytes (split-reduction partial sums), nothing to zero.
 * NITI_ERR_UNSUPPORTED for layers that are not thin. */
NITI_API size_t niti_conv_wgrad_patches_scratch_bytes(int N, int H, int W, int C, int K, int R, int S);
NITI_API int niti_conv_wgrad_patches_i8(const int8_t* patches, const int8_t* err, int32_t* g32, uint32_t* maxabs,
                       void* scratch, size_t scratch_bytes,
                       int N, int H, int W, int C, int K, int R, int S,
                       int32_t* status, void* stream);
/* The same contraction ADDED into g32: g32 += sum err * x, with no clearing pass, no scratch and no maximum.
 * The caller has zeroed g32 (niti_update_multi_i8 with clear_gradients does) or keeps the gradient of earlier
 * micro-batches in it.  Tensor-core shapes only (niti_conv_wgrad_accumulate_supported); x, err, g32 16-byte aligned. */
NITI_API int niti_conv_wgrad_accumulate_supported(int C, int K, int R, int S, int pad);
NITI_API int niti_conv_wgrad_accumulate_i8(const int8_t* x, const int8_t* err, int32_t* g32,
                                  int N, int H, int W, int C, int K, int R, int S, int pad,
                                  int32_t* status, void* stream);

/* niti_conv_wgrad_accumulate_i8 for up to niti_conv_wgrad_accumulate_multi_max() layers in ONE launch: every item's
 * gradient is added into its g32.  The thread blocks of the launch are dealt to the layers so that each walks about the
 * same number of pixels, which lets two layers of a step share one wave of the GPU (and one launch, one prologue and
 * one flush of the accumulators) where each alone would leave its blocks short of work.  Every item must satisfy
 * niti_conv_wgrad_accumulate_supported; results are those of `count` single calls in any order (integer sums).  No
 * counterpart in the reference, which computes one layer's gradient at a time (ti_torch.py:429-432). */
typedef struct niti_wgrad_item {
    const int8_t* x; const int8_t* err; int32_t* g32;
    int32_t N, H, W, C, K, R, S, pad;
} niti_wgrad_item;
NITI_API int niti_conv_wgrad_accumulate_multi_max(void);
NITI_API int niti_conv_wgrad_accumulate_multi_i8(const niti_wgrad_item* items, int count, int32_t* status, void* stream);

/* niti_conv_wgrad_i8 for callers that cannot hand over scratch memory.  This entry point has no
 * counterpart in the reference.  Some hosts of this library are not able to call cudaMalloc at all:
 * a plugin inside an application that owns every byte of device memory and offers no allocator, or a
 * service whose device-memory budget is fixed and audited at start-up.  For them the split-reduction
 * scratch of the weight gradient lives in a buffer that is part of the library image
 * (NITI_BUILTIN_SCRATCH_BYTES, held by every GPU context that loads the library until it exits); the
 * call allocates nothing, neither through CUDA nor through any library.
 *  - Same arguments (minus scratch), same result bit for bit as niti_conv_wgrad_i8: when the usual
 *    number of pixel-range splits would not fit, fewer splits are used (integer sums do not depend on
 *    the split), and a problem that does not fit even unsplit (K*R*S*C*4 bytes above the limit, or a
 *    first-layer patch matrix N*H*W*32 bytes above it) is refused with NITI_ERR_TOO_LARGE before
 *    anything is launched.
 *  - The first call on each device looks up the buffer's device address (cudaGetSymbolAddress, with that
 *    device current); make that first call during set-up, before any stream capture is begun.  `stream` must
 *    belong to the current device.  The address is remembered per device ordinal: a process that resets a
 *    device (cudaDeviceReset) must not use this entry point on it afterwards.  Concurrent first calls from
 *    several host threads are safe.  maxabs may be null, as in niti_conv_wgrad_i8.
 *  - All calls on a device share the one buffer and it keeps the previous call's contents; this entry
 *    point needs none of it zeroed, but two calls whose kernels overlap on the GPU (different streams
 *    without ordering) race on it: keep calls stream-ordered.
 */
#define NITI_BUILTIN_SCRATCH_BYTES (16u << 20)
NITI_API int niti_conv_wgrad_builtin_scratch_i8(const int8_t* x, const int8_t* err, int32_t* g32, uint32_t* maxabs,
                       int N, int H, int W, int C, int K, int R, int S, int pad,
                       int32_t* status, void* stream);

/* Convolution and requantisation in ONE pass over the output: TiConv2d.forward's
 * conv2d_int8 + act_calc (ti_torch.py:391-397) and TiConv2d.backward's error path conv2d_int8 +
 * err_calc (ti_torch.py:403-407).  The shift depends on the max of the whole int32 tensor, which
 * is only known when the contraction has finished, so the kernel narrows with a PREDICTED shift
 * (the one this layer needed last time, state[0]) while it reduces the true max|acc|; the thread
 * block that finishes last derives the true shift, and only if the prediction was wrong the
 * contraction is launched again (that second launch returns at once otherwise).  The result is
 * always the exact one; the int32 tensor never touches memory.  When the whole output is at most
 * 148 x (512 / tile width) tiles, all accumulators fit in tensor memory at once and a single
 * cooperative launch does it without any prediction: reduce max, grid barrier, narrow (state[0]
 * still receives the shift; state[2] stays 0).
 *   state: device int32[8], 8-byte aligned, owned by the caller, one per layer and direction, zeroed once:
 *          [0] shift (in: prediction, out: true value), [1] max|acc| (zero between calls), [2] 1 if
 *          the last call had to redo (bits 0-1; see niti_conv_dgrad_requant_side_i8), [3] number of redos so far, [4] block ticket, [5..7] grid-barrier
 *          words of the single-launch kernel (all zero between calls).
 *   kind is ACT for fprop (exp_out = shift + *exp_a + *exp_b) and ERR for dgrad; target 7 bits.
 * Shapes: niti_conv_*_requant_supported() != 0 (the tensor-core shapes of the entry points above
 * with 16-byte-multiple output channels); otherwise NITI_ERR_UNSUPPORTED and the caller uses
 * niti_conv_fprop_i8 / niti_conv_dgrad_i8 + niti_requant_i8.  `scratch` as for niti_conv_fprop_i8.
 */
NITI_API int niti_conv_fprop_requant_supported(int C, int K, int R, int S, int pad);
NITI_API int niti_conv_dgrad_requant_supported(int C, int K, int R, int S, int pad);
NITI_API int niti_conv_fprop_requant_i8(const int8_t* x, const int8_t* w, int8_t* y8, int32_t* state,
                       void* scratch, size_t scratch_bytes,
                       int N, int H, int W, int C, int K, int R, int S, int pad,
                       int round_mode, const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset, int relu,
                       const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                       int32_t* status, void* stream);
NITI_API int niti_conv_dgrad_requant_i8(const int8_t* err, const int8_t* w, int8_t* e8, int32_t* state,
                       int N, int H, int W, int C, int K, int R, int S, int pad,
                       int round_mode, const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset,
                       const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                       const int8_t* relu_mask, int32_t* status, void* stream);
/* relu_mask (may be null): the int8 tensor [N][H][W][C] this layer received in the forward pass, i.e. the output of
 * the ReLU in front of it.  Where it is <= 0 the error is zeroed: TiReLU.backward (ti_torch.py:279-290) folded into
 * the kernel.  The mask is applied after the requantisation, so the shift is that of the unmasked error, exactly as
 * when the two run one after the other. */

/* niti_conv_dgrad_requant_i8 with `side`, niti_conv_dgrad_requant_side_bytes() bytes of caller-owned device memory
 * (16-byte aligned, contents irrelevant) that belongs to the layer like `state`.  A layer whose max |error| hovers
 * around a power of two needs shift S in some steps and S - 1 in others, and every wrong guess costs a second
 * contraction.  With `side` the first launch (round-to-nearest only) also stores bits S-1 and S-2 of every rounded
 * sum, 2 bits per output; when the true shift turns out to be S - 1 the second launch rewrites the int8 output from
 * them (exactly: sign(x) * ((|x| + 2^(S-2)) >> (S-1)) follows from x's value at shift S and those two bits) instead of
 * contracting again, and the guess stays S until the lower shift has applied 12 times in a row.  state[2] then
 * reads: bits 0-1 = 0 right / 1 contracted again / 2 stepped down, bits 4-7 = step-downs in a row, bits 8-31 = step-downs so
 * far; state[3] counts second contractions only.  niti_conv_dgrad_requant_side_bytes returns 0 when the single-launch
 * kernel serves the shape (nothing is predicted there); side may be null (= niti_conv_dgrad_requant_i8).  No counterpart in
 * the reference. */
NITI_API size_t niti_conv_dgrad_requant_side_bytes(int N, int H, int W, int C, int K, int R, int S, int pad);
NITI_API int niti_conv_dgrad_requant_side_i8(const int8_t* err, const int8_t* w, int8_t* e8, int32_t* state,
                       void* side, size_t side_bytes,
                       int N, int H, int W, int C, int K, int R, int S, int pad,
                       int round_mode, const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset,
                       const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                       const int8_t* relu_mask, int32_t* status, void* stream);

/* niti_conv_fprop_requant_i8 that ALSO writes the 2x2 / stride-2 max-pooled output, y8_pooled [N][H/2][W/2][K]:
 * TiConv2d.forward + TiReLU.forward + TiMaxpool2d.forward (ti_torch.py:391-397, 268-277, 302-307;
 * int8pool_cuda.int8_pool, int8pool_kernel.cu:28-80) in one launch.  The unpooled y8 is still written: the pool's
 * backward routes by it.  Only where the single-launch (accumulator-parking) kernel takes the layer and every
 * pooling window lies within one warp's rows of an output tile: niti_conv_fprop_requant_pool_supported() != 0
 * (H, W even; images at most 16 pixels wide); elsewhere NITI_ERR_UNSUPPORTED and the caller runs niti_maxpool_fwd_i8. */
NITI_API int niti_conv_fprop_requant_pool_supported(int N, int H, int W, int C, int K, int R, int S, int pad);
NITI_API int niti_conv_fprop_requant_pool_i8(const int8_t* x, const int8_t* w, int8_t* y8, int8_t* y8_pooled, int32_t* state,
                       int N, int H, int W, int C, int K, int R, int S, int pad,
                       int round_mode, const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset, int relu,
                       const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                       int32_t* status, void* stream);

/* int8mm_cuda.int8_mm (int8mm.cpp:9-18, int8mm_kernel.cu:8-34) as used by TiLinear
 * (ti_torch.py:241-266), without the padding / .contiguous() copies around it:
 * C32[M][N] = op(A) * op(B); trans_a == 0: A is [M][K], else [K][M];
 * trans_b == 0: B is [K][N], else [N][K].  Forward a*W^T: (0,1); error e*W: (0,0);
 * gradient e^T*a: (1,0).  Tensor-core path when every row pitch is a multiple of 16 bytes,
 * M >= 64 and N, K >= 32; otherwise a CUDA-core path (the 10-class FC layer).
 */
NITI_API int niti_gemm_i8(const int8_t* A, const int8_t* B, int32_t* C32, uint32_t* maxabs,
                 int M, int N, int K, int trans_a, int trans_b, int32_t* status, void* stream);

/* ---------------------------------------------------------------- requantisation
 *
 * act_calc / err_calc / grad_calc + RoundShift / StoShift / PstoShift + int8_clip
 * (ti_torch.py:23-72,103-147), with RangeEstimate (ti_torch.py:366-377) already reduced into
 * *maxabs by the producing kernel.  bits = 0 if max==0 else bit_length(max-1);
 * shift = max(bits - target_bits, 0); shift == 0 wraps (tensor.type(int8)), otherwise round
 * and clamp to +-127; kind GRAD with bits == 0 writes zeros.
 * Random word of element i (stochastic mode): Philox4x32-10 keyed by *seed, stream `rng_stream`,
 * element index rng_offset + i.  If relu != 0, max(.,0) is applied after narrowing
 * (TiReLU.forward, ti_torch.py:272-279).
 * *exp_out = shift + (exp_a ? *exp_a : 0) + (exp_b ? *exp_b : 0); *shift_out = shift (each optional).
 */
NITI_API int niti_requant_i8(const int32_t* acc, int8_t* out, const uint32_t* maxabs, int64_t n,
                    int kind, int target_bits, int round_mode,
                    const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset, int relu,
                    const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                    void* stream);

/* max |acc| over n int32 values, reduced into *maxabs (cleared first).  RangeEstimate for
 * tensors that did not come out of a contraction kernel (e.g. all-reduced gradients). */
NITI_API int niti_absmax_i32(const int32_t* acc, int64_t n, uint32_t* maxabs, void* stream);

/* int8conv_cuda.group_conv (int8conv.cpp:35-45, int8conv_kernel.cu:248-334) in the one form the reference
 * calls it: conv2d_weight_int8 (ti_torch.py:194-233) folds batch and input channels into G = N*C groups of one
 * channel each and turns the error maps into G*Kg filters as large as the image, so that the "convolution"
 * yields every sample's own weight gradient.  in [H][W][G], wt [G*Kg][R][S] (one channel), stride 1, dilation 1:
 * out32[p][q][g*Kg+k] = sum_{r,s} in[p+r-pad][q+s-pad][g] * wt[g*Kg+k][r][s], P = H+2*pad-R+1, exact int32
 * (the reference accumulates in float32).  Batch and channels cannot be told apart from G alone, which is why this
 * form cannot be handed to niti_conv_wgrad_i8; code written against this library calls that entry point directly.
 */
NITI_API int niti_group_conv1_i8(const int8_t* in, const int8_t* wt, int32_t* out32, int H, int W, int G, int Kg,
                        int R, int S, int pad, void* stream);

/* ---------------------------------------------------------------- memory-bound layers
 * int8pool_cuda.int8_pool / int8_pool_backward (int8pool.cpp, int8pool_kernel.cu:28-138) as
 * used by TiMaxpool2d (ti_torch.py:292-316); int8 throughout (no fp16 copies), pad 0.
 * Backward recomputes the window maximum from x and routes dy to the first position, scanning
 * rows then columns, that holds it.  relu_mask != 0 additionally zeroes dx where x <= 0, i.e. it
 * applies the TiReLU.backward (ti_torch.py:281-290) of a ReLU whose output x is (x > 0 exactly where
 * the ReLU's input was > 0), saving that layer's separate pass.
 */
NITI_API int niti_maxpool_fwd_i8(const int8_t* x, int8_t* y, int N, int H, int W, int C, int k, int stride, void* stream);
NITI_API int niti_maxpool_bwd_i8(const int8_t* x, const int8_t* dy, int8_t* dx, int N, int H, int W, int C, int k, int stride,
                        int relu_mask, void* stream);
/* TiReLU.forward / backward (ti_torch.py:268-290) */
NITI_API int niti_relu_fwd_i8(const int8_t* x, int8_t* y, int64_t n, void* stream);
NITI_API int niti_relu_bwd_i8(const int8_t* act, const int8_t* err, int8_t* out, int64_t n, void* stream);
/* TiDropout (ti_torch.py:439-455): y[b][f] = x[b][f] * bit(f), bit = low bit of the Philox word of
 * element f in stream rng_stream; the same call serves forward and backward. */
NITI_API int niti_dropout_i8(const int8_t* x, int8_t* y, int64_t rows, int64_t features,
                    const uint64_t* seed, uint32_t rng_stream, void* stream);

/* TiLoss.forward (ti_loss.py:6-36): integer cross-entropy error.  out8 [B][classes] int8, *out_exp its
 * exponent, target int64 [B]; err8 [B][classes].  classes <= 32.  The closing StoShift(.,4) draws the
 * Philox word of element (sample_offset + b) * classes + c from stream rng_stream. */
NITI_API int niti_loss_i8(const int8_t* out8, const int32_t* out_exp, const int64_t* target, int8_t* err8,
                 int B, int classes, const uint64_t* seed, uint32_t rng_stream, uint64_t sample_offset, void* stream);

/* UpdateWeight.weight_update (ti_torch.py:16-21): g8 = grad_calc(g32, mu); w = clamp(w - g8, +-127).
 * *maxabs = max |g32| (from niti_conv_wgrad_i8 / niti_gemm_i8 / niti_absmax_i32). */
NITI_API int niti_update_i8(int8_t* w, const int32_t* g32, const uint32_t* maxabs, int64_t n,
                   int mu, int round_mode, const uint64_t* seed, uint32_t rng_stream, void* stream);

/* Every weighted layer's update in one (cooperative) launch: for each item max |g32| is found, written to
 * *maxabs when that is not null, and w updated exactly as niti_update_i8 would with that maximum and the
 * item's rng_stream.  scratch: niti_update_multi_scratch_bytes() bytes.  status as in niti_fc_head_train_i8
 * (code 7).  clear_gradients != 0 also zeroes every g32 after use, which is what niti_conv_wgrad_accumulate_i8
 * wants to find at the next step.  No counterpart in the reference, which updates layer by layer
 * (ti_torch.py:16-21). */
typedef struct niti_update_item {
    int8_t* w; int32_t* g32; uint32_t* maxabs; int64_t n; uint32_t rng_stream;
} niti_update_item;
NITI_API size_t niti_update_multi_scratch_bytes(void);
NITI_API int niti_update_multi_i8(const niti_update_item* items, int count, int mu, int round_mode, int clear_gradients,
                         const uint64_t* seed, void* scratch, size_t scratch_bytes, int32_t* status, void* stream);

/* The update of a data-parallel step as ONE (cooperative) kernel per rank over peer memory, in place of an
 * all-reduce of the gradients followed by niti_update_multi_i8.  Every rank (one process per GPU, all GPUs of one
 * node with peer access) calls it once per step, on buffers that hold the same layout on every rank:
 *   weights[r]  rank r's weight arena: layer i's int8 weights start w_offset bytes in (a multiple of 4);
 *   grads[r]    rank r's int32 gradient bucket: layer i's accumulators start g_offset ELEMENTS in (a multiple of 4);
 *   exchange[r] niti_dp_exchange_bytes() bytes of rank r, zeroed ONCE by its owner before any rank's first call.
 * weights / grads / exchange are host arrays of `world` device pointers valid in the calling process (the caller's
 * own allocation at index `rank`, the peers' through CUDA IPC or any other peer mapping).  The kernel
 *   1. waits until every rank's earlier work on the stream has finished (flags in the exchange areas),
 *   2. sums slice `rank` of every layer (word groups [G rank / world, G (rank + 1) / world) of its G = n / 4 groups)
 *      over all ranks' buckets with plain peer loads, and sends the slice's max |sum| per layer to every rank,
 *   3. takes each layer's maximum over the ranks, updates ITS slice of the weights exactly as niti_update_i8 would
 *      (same shift, same random words: they are indexed by the element's position in the layer) and stores the new
 *      bytes into every rank's arena; zeroes its own bucket,
 *   4. waits until every rank's stores have landed.
 * Afterwards all replicas hold the weights one process would hold after niti_update_multi_i8 on the summed
 * gradients (integer addition is associative), and every bucket is zero.  maxabs (nullable): uint32[count], each
 * layer's max |summed g32|.  n must be a multiple of 4, count <= 16, world <= 8.  Every wait is bounded (0.5 s for
 * the blocks of the own GPU, 4 s for a peer): on expiry status receives {9, rank it waited for or -1, barrier
 * number}, the kernel returns, and the replicas must be considered out of step.  The ranks must therefore reach the
 * call within 4 s of each other.  Never run two ranks on ONE GPU: their kernels would wait for each other without
 * being co-resident.  No counterpart in the reference (single GPU). */
/* Peer-visible device memory for niti_dp_update_i8, owned by the library.  niti_peer_arena_create allocates `bytes`
 * of zeroed device memory on the current device and fills `handle` (NITI_PEER_HANDLE_BYTES bytes, to be sent to the
 * other processes of the node by any host channel); niti_peer_arena_open maps another process's arena into the
 * calling process for kernels of the CURRENT device (peer access to the owner's GPU is switched on by the mapping);
 * niti_peer_arena_close unmaps it, niti_peer_arena_destroy frees an own arena (after every peer has closed it).
 * Plain CUDA IPC mappings: the memory is not bound to a multicast object. */
#define NITI_PEER_HANDLE_BYTES 64
NITI_API int niti_peer_arena_create(size_t bytes, void** ptr, void* handle);
NITI_API int niti_peer_arena_open(const void* handle, void** ptr);
NITI_API int niti_peer_arena_close(void* ptr);
NITI_API int niti_peer_arena_destroy(void* ptr);
/* staged (all null, or one pointer per rank < world; the own rank's entry is ignored): the gradients of this layer that
 * rank r computed for THIS rank's slice already lie in this rank's memory, pushed there by r (niti_peer_copy, a copy
 * engine transfer under r's backward pass, stream-ordered before r's call of niti_dp_update_i8); staged[r] is the address
 * the layer's word group 0 would have if the whole layer had been pushed (slice start minus 16 * first group of the
 * slice), 16-byte aligned.  The kernel then sums local memory for this layer instead of reading the peers' buckets over
 * NVLink after the backward pass; the ranks' own buckets are still read, zeroed and must hold the layer as before. */
typedef struct niti_dp_item { int64_t w_offset; int64_t g_offset; int64_t n; uint32_t rng_stream; const void* staged[8]; } niti_dp_item;
typedef struct niti_dp_update_args {
    const niti_dp_item* items; int32_t count;
    int32_t rank, world;
    void* const* weights; void* const* grads; void* const* exchange;
    int32_t mu, round_mode;
    const uint64_t* seed;
    uint32_t* maxabs;
    int32_t* status;
} niti_dp_update_args;
NITI_API size_t niti_dp_exchange_bytes(void);
/* bytes device bytes from src to dst on `stream` (cudaMemcpyAsync, device to device): both may lie in any arena mapped
 * into the calling process, so this is how a rank pushes a finished gradient slice into its owner's staging memory. */
NITI_API int niti_peer_copy(void* dst, const void* src, size_t bytes, void* stream);
NITI_API int niti_dp_update_i8(const niti_dp_update_args* args, void* stream);

/* The classifier head of a training step in one (cooperative) kernel: TiDropout.forward
 * (ti_torch.py:439-455), TiLinear.forward (:241-253), TiLoss.forward (ti_loss.py:6-36), TiLinear.backward
 * (:255-266) with UpdateWeight.weight_update (:16-21), and TiDropout.backward.  Same integers as the calls
 *   niti_dropout_i8, niti_gemm_i8 (x W^T), niti_requant_i8 (act), niti_loss_i8, niti_gemm_i8 (err W),
 *   niti_requant_i8 (err), niti_gemm_i8 (err^T x), niti_update_i8, niti_dropout_i8
 * made one after the other with the streams / offsets named below.
 *   x [B][F] int8 features (before dropout), *exp_x their exponent; w [J][F] int8 (updated in place when
 *   `update` != 0), *exp_w; target int64 [B];
 *   out8 [B][J] logits with *exp_out; err8 [B][J] the loss's error (exponent 0);
 *   e8 [B][F] the error handed to the layer before the head (dropout bits applied), *exp_err;
 *   g32 [J][F] the weight gradient's accumulators, *grad_maxabs = max |g32|.
 *   dropout != 0: one keep bit per feature from stream dropout_stream (and the +1 on the exponent);
 *   bits: target bit-width of activations and errors (7); mu: of the gradient;
 *   act / err / grad rounding draw from streams layer_stream, layer_stream + 1, layer_stream + 2 with the
 *   element indices niti_requant_i8 / niti_update_i8 would use (samples offset by sample_offset);
 *   the loss's StoShift draws from loss_stream.
 * scratch: niti_fc_head_scratch_bytes(B, F, J) bytes, 16-byte aligned.  Shapes: J <= 16, F % 16 == 0 and
 * J * F small enough for shared memory (niti_fc_head_supported says).  status: int32[4] or null; a grid
 * barrier that is not met within 0.5 s writes code 6 there and the kernel returns. */
typedef struct niti_fc_head_args {
    const int8_t* x; const int32_t* exp_x;
    int8_t* w; const int32_t* exp_w;
    const int64_t* target;
    int8_t* out8; int32_t* exp_out;
    int8_t* err8;
    int8_t* e8; int32_t* exp_err;
    int32_t* g32; uint32_t* grad_maxabs;
    void* scratch; size_t scratch_bytes;
    int32_t B, F, J;
    int32_t dropout, bits, act_round, err_round, grad_round, mu, update;
    const uint64_t* seed;
    uint32_t layer_stream, dropout_stream, loss_stream;
    uint64_t sample_offset;
    int32_t* status;
} niti_fc_head_args;
NITI_API int niti_fc_head_supported(int B, int F, int J);
NITI_API size_t niti_fc_head_scratch_bytes(int B, int F, int J);
NITI_API int niti_fc_head_train_i8(const niti_fc_head_args* args, void* stream);

/* TiFloatToInt8 + the NCHW -> NHWC permute of TiNet.forward (ti_torch.py:341-356, ti_net.py:18-19):
 * x f32 [N][C][H][W] -> x8 int8 [N][H][W][C], *exp_out = ceil(log2(max|x|)) - 7.
 * `scratch` is one uint32 word (cleared by the call). */
NITI_API int niti_quantize_input_f32(const float* x, int8_t* x8, int32_t* exp_out, uint32_t* scratch,
                            int N, int C, int H, int W, void* stream);

/* Self-test of the bounded waits: launches one thread block that waits at a grid barrier expecting two blocks.  The
 * wait gives up after its 0.5 s limit, writes {8, block index, expected arrivals} to status[0..2] (int32[4], zeroed by
 * the caller) and the kernel returns normally: the context stays usable.  scratch: one int32 word. */
NITI_API int niti_selftest_barrier_timeout(int32_t* scratch, int32_t* status, void* stream);

/* The two halves of niti_quantize_input_f32, for callers that put something between them: *maxbits = the IEEE bit
 * pattern of max |x| (non-negative floats order like their bit patterns, so a MAX reduction over ranks on the
 * uint32 word gives the global maximum: what the global-exact data-parallel mode does). */
NITI_API int niti_absmax_f32(const float* x, int64_t n, uint32_t* maxbits, void* stream);
NITI_API int niti_quantize_input_with_max_f32(const float* x, int8_t* x8, int32_t* exp_out, const uint32_t* maxbits,
                                     int N, int C, int H, int W, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NITI_B200_H */
