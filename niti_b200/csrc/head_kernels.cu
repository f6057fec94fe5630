// The classifier head of a training step in ONE cooperative kernel: dropout, the FC layer's forward GEMM,
// its requantisation, the integer cross-entropy error, the FC layer's error-backward GEMM with its
// requantisation and the dropout mask, the FC weight gradient and the weight update.
//
// In the reference this is TiDropout.forward (ti_torch.py:439-455), TiLinear.forward (:241-253),
// TiLoss.forward (ti_loss.py:6-36), TiLinear.backward (:255-266) with UpdateWeight.weight_update (:16-21)
// and TiDropout.backward: eleven launches of a few microseconds of work each when run one by one, all of
// them bound by launch latency.  Here every thread block keeps the (small) weight matrix in shared memory
// and the three tensor-wide maxima that pick the shifts are met with three grid barriers.
//
// Every grid barrier is bounded (0.5 s): a block that gives up writes the status word and leaves.
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/niti_b200.h"
#include "internal.h"
#include "requant.cuh"
#include "loss_math.cuh"
#include "grid_barrier.cuh"

namespace niti {
namespace {

constexpr int HEAD_THREADS = 256;
constexpr int HEAD_MAX_CLASSES = 16;
constexpr int HEAD_RED_INTS = 16 * 16 * 16;  // [batch group][class][feature of the chunk]
constexpr size_t HEAD_MAX_SMEM = 200 * 1024;

struct HeadParams {
    const int8_t* x; const int32_t* exp_x; int8_t* w; const int32_t* exp_w; const long long* target;
    int8_t* out8; int32_t* exp_out; int8_t* err8; int8_t* e8; int32_t* exp_err; int32_t* g32; unsigned* grad_maxabs;
    int32_t* out32;  // scratch: B*J accumulators of the forward GEMM
    int32_t* state;  // scratch: {max|out32|, max|e32|, max|g32|, barrier arrivals}, zero at launch
    int B, F, J, dropout, bits, act_mode, err_mode, grad_mode, mu, update;
    const unsigned long long* seed;
    unsigned layer_stream, dropout_stream, loss_stream;
    unsigned long long sample_offset;
    int32_t* status;
};

__device__ __forceinline__ unsigned iabs32(int x) { return static_cast<unsigned>(x < 0 ? -x : x); }
// four mask bits -> four bytes of 0xFF / 0x00
__device__ __forceinline__ uint32_t expand4(unsigned b) {
    return ((b & 1u) | ((b & 2u) << 7) | ((b & 4u) << 14) | ((b & 8u) << 21)) * 0xFFu;
}
__device__ __forceinline__ long long warp_sum_ll(long long v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}

// max over the block -> one atomic (every thread calls; `scratch` holds 8 words)
__device__ __forceinline__ void block_max(unsigned* dst, unsigned m, int32_t* scratch) {
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = static_cast<int32_t>(m);
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned x = 0;
#pragma unroll
        for (int i = 0; i < HEAD_THREADS / 32; ++i) x = max(x, static_cast<unsigned>(scratch[i]));
        if (x != 0) atomicMax(dst, x);
    }
    __syncthreads();
}

// e[k] = sum_j err[j] * W[j][16 c + k]: one 16-feature chunk of the error that goes back to the features.
// The loop over classes stays rolled: this code runs once or twice per launch, so every instruction is an
// instruction-cache miss and straight-line unrolling costs more than the loop overhead it saves.
__device__ __forceinline__ void dgrad_chunk(const uint4* sW, const int8_t* err, int J, int F16, int c, int (&e)[16]) {
#pragma unroll
    for (int k = 0; k < 16; ++k) e[k] = 0;
#pragma unroll 1
    for (int j = 0; j < J; ++j) {
        const int ej = err[j];
        const uint4 wv = sW[j * F16 + c];
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int r = 0; r < 4; ++r) e[q * 4 + r] += ej * static_cast<int>(static_cast<int8_t>(ww[q] >> (8 * r)));
    }
}

#ifdef NITI_HEAD_TIMING
#define HEAD_STAMP(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<unsigned long long*>(p.state + 4 + ((p.B * p.J + 1) & ~1))[i] = grid_timer_ns(); } while (0)
#else
#define HEAD_STAMP(i) do { } while (0)
#endif

__global__ void __launch_bounds__(HEAD_THREADS, 1) fc_head_kernel(const HeadParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int F = p.F, F16 = F >> 4, J = p.J, B = p.B, G = gridDim.x;
    // shared memory: W [J][F] | keep bits, one uint16 per 16 features | err8 [B][J] | err8 transposed | reduction scratch | flag
    uint4* sW = reinterpret_cast<uint4*>(smem);
    size_t off = static_cast<size_t>(J) * F;
    uint16_t* sMask = reinterpret_cast<uint16_t*>(smem + off);
    off = (off + 2 * static_cast<size_t>(F16) + 15) & ~static_cast<size_t>(15);
    int8_t* sErr = reinterpret_cast<int8_t*>(smem + off);
    off = (off + static_cast<size_t>(B) * J + 15) & ~static_cast<size_t>(15);
    const int S = (((B + 3) >> 2) + 3) & ~3;  // samples per batch group of the weight gradient (a multiple of 4)
    int8_t* sErrT = reinterpret_cast<int8_t*>(smem + off);  // err8 transposed, [J][4 S], zero beyond B
    off += static_cast<size_t>(J) * 4 * S;
    int32_t* sRed = reinterpret_cast<int32_t*>(smem + off);
    int* sFlag = reinterpret_cast<int*>(sRed + HEAD_RED_INTS);

    HEAD_STAMP(0);
    const unsigned long long seed = *p.seed;
    unsigned* umax = reinterpret_cast<unsigned*>(p.state);

    {   // the weights (read by this block until the end, whatever the other blocks write back) and the dropout bits
        const uint4* W4 = reinterpret_cast<const uint4*>(p.w);
        for (int i = t; i < J * F16; i += HEAD_THREADS) sW[i] = W4[i];
        for (int c = t; c < F16; c += HEAD_THREADS) {
            unsigned bits = 0xFFFFu;
            if (p.dropout) {
                bits = 0;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t r[4];
                    random_block(seed, p.dropout_stream, static_cast<unsigned long long>(c) * 4 + q, r);
                    bits |= ((r[0] & 1u) | ((r[1] & 1u) << 1) | ((r[2] & 1u) << 2) | ((r[3] & 1u) << 3)) << (4 * q);
                }
            }
            sMask[c] = static_cast<uint16_t>(bits);
        }
    }
    __syncthreads();
    HEAD_STAMP(1);

    // ---- forward GEMM: out32[b][j] = sum_f drop(x)[b][f] * W[j][f], one sample per block at a time
    unsigned fwd_max = 0;
    for (int b = blockIdx.x; b < B; b += G) {
        int acc[HEAD_MAX_CLASSES];
#pragma unroll
        for (int j = 0; j < HEAD_MAX_CLASSES; ++j) acc[j] = 0;
        const uint4* x4 = reinterpret_cast<const uint4*>(p.x) + static_cast<size_t>(b) * F16;
        for (int c = t; c < F16; c += HEAD_THREADS) {
            uint4 xv = __ldg(x4 + c);
            const unsigned bits = sMask[c];
            xv.x &= expand4(bits); xv.y &= expand4(bits >> 4); xv.z &= expand4(bits >> 8); xv.w &= expand4(bits >> 12);
#pragma unroll
            for (int j = 0; j < HEAD_MAX_CLASSES; ++j)
                if (j < J) {
                    const uint4 wv = sW[j * F16 + c];
                    int a = acc[j];
                    a = __dp4a(static_cast<int>(xv.x), static_cast<int>(wv.x), a);
                    a = __dp4a(static_cast<int>(xv.y), static_cast<int>(wv.y), a);
                    a = __dp4a(static_cast<int>(xv.z), static_cast<int>(wv.z), a);
                    a = __dp4a(static_cast<int>(xv.w), static_cast<int>(wv.w), a);
                    acc[j] = a;
                }
        }
#pragma unroll
        for (int j = 0; j < HEAD_MAX_CLASSES; ++j)
            if (j < J) {
                const int v = __reduce_add_sync(0xFFFFFFFFu, acc[j]);
                if (lane == 0) sRed[warp * HEAD_MAX_CLASSES + j] = v;
            }
        __syncthreads();
        if (warp == 0) {
            int v = 0;
            if (lane < J) {
#pragma unroll
                for (int wq = 0; wq < HEAD_THREADS / 32; ++wq) v += sRed[wq * HEAD_MAX_CLASSES + lane];
                p.out32[b * J + lane] = v;
            }
            fwd_max = max(fwd_max, __reduce_max_sync(0xFFFFFFFFu, iabs32(v)));
        }
        __syncthreads();
    }
    if (t == 0 && fwd_max != 0) atomicMax(&umax[0], fwd_max);  // one atomic per block: they serialise at the L2
    HEAD_STAMP(2);
    if (!bounded_grid_barrier(&p.state[3], G, p.status, 6, sFlag)) return;

    HEAD_STAMP(3);
    // ---- logits to int8, then the loss's error: one warp per sample, one lane per class
    const int exp_w = *p.exp_w;
    {
        bool z;
        const int shift = shift_for(__ldcg(&umax[0]), CALC_ACT, p.bits, &z);
        const int out_exp = shift + *p.exp_x + (p.dropout ? 1 : 0) + exp_w;
        if (blockIdx.x == 0 && t == 0) *p.exp_out = out_exp;
        if (warp == 0) {
            for (int b = blockIdx.x; b < B; b += G) {
                const bool on = lane < J;
                const unsigned long long elem = (p.sample_offset + b) * static_cast<unsigned long long>(J) + lane;
                int o8 = 0;
                if (on) {
                    const uint32_t rnd = (p.act_mode == ROUND_STOCHASTIC && shift > 0) ? random_word(seed, p.layer_stream, elem) : 0u;
                    o8 = narrow(p.out32[b * J + lane], shift, p.act_mode, rnd);
                    p.out8[b * J + lane] = static_cast<int8_t>(o8);
                }
                float g = 0.0f;
                long long contrib = 0;
                if (out_exp > -7) {
                    float s = -3.0e38f;
                    if (on) {
                        s = __fdiv_rn(static_cast<float>(o8 * 47274), 32768.0f);
                        s = out_exp >= 0 ? __fmul_rn(s, pow2f_int(out_exp)) : __fdiv_rn(s, pow2f_int(-out_exp));
                    }
                    float mx = s;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
                    const float offset = __fsub_rn(mx, 10.0f);
                    if (on) {
                        const float d = fmaxf(__fsub_rn(s, offset), 0.0f);
                        g = __fsub_rn(static_cast<float>(exp2_det(static_cast<double>(d))), 1.0f);
                        contrib = static_cast<long long>(g);
                    }
                } else if (on) {
                    const long long a = 1ll << (1 - 2 * out_exp), bq = 1ll << (1 - out_exp);
                    const long long s = o8;
                    contrib = a + s * bq + s * s;
                    g = __ll2float_rn(contrib);
                }
                const float denom = __ll2float_rn(warp_sum_ll(contrib));
                long long rs = 0;
                if (on) {
                    g = __fdiv_rn(__fmul_rn(g, 2048.0f), denom);
                    rs = static_cast<long long>(g);
                }
                const long long row_sum = warp_sum_ll(rs);
                if (on) {
                    if (lane == static_cast<int>(p.target[b])) g = __fsub_rn(g, __ll2float_rn(row_sum));
                    const int g32 = static_cast<int>(g);  // truncation, like tensor.type(torch.int32)
                    p.err8[b * J + lane] = narrow(g32, 4, ROUND_STOCHASTIC, random_word(seed, p.loss_stream, elem));
                }
            }
        }
    }
    HEAD_STAMP(4);
    if (!bounded_grid_barrier(&p.state[3], 2 * G, p.status, 6, sFlag)) return;
    HEAD_STAMP(5);

    // ---- every block needs every sample's error
    for (int i = t; i < B * J; i += HEAD_THREADS) sErr[i] = __ldcg(reinterpret_cast<const signed char*>(p.err8) + i);
    for (int i = t; i < J * 4 * S; i += HEAD_THREADS) {
        const int j = i / (4 * S), b = i % (4 * S);
        sErrT[i] = b < B ? __ldcg(reinterpret_cast<const signed char*>(p.err8) + b * J + j) : int8_t(0);
    }
    __syncthreads();

    // ---- error-backward GEMM, first pass: max|e32|.  The chunks of the block's FIRST sample (all there is when the
    //      batch is not larger than the grid) stay in registers until the shift is known; the rest is recomputed then.
    constexpr int KEEP_CHUNKS = 2;
    int ekeep[KEEP_CHUNKS][16];
    {
        unsigned m = 0;
        if (static_cast<int>(blockIdx.x) < B) {
#pragma unroll
            for (int k = 0; k < KEEP_CHUNKS; ++k) {
                const int c = t + k * HEAD_THREADS;
                if (c < F16) {
                    dgrad_chunk(sW, sErr + blockIdx.x * J, J, F16, c, ekeep[k]);
#pragma unroll
                    for (int i = 0; i < 16; ++i) m = max(m, iabs32(ekeep[k][i]));
                }
            }
        }
        for (int b = blockIdx.x; b < B; b += G)
            for (int c = t + (b == static_cast<int>(blockIdx.x) ? KEEP_CHUNKS * HEAD_THREADS : 0); c < F16; c += HEAD_THREADS) {
                int e[16];
                dgrad_chunk(sW, sErr + b * J, J, F16, c, e);
#pragma unroll
                for (int k = 0; k < 16; ++k) m = max(m, iabs32(e[k]));
            }
        block_max(&umax[1], m, sRed);
    }
    HEAD_STAMP(6);
    // ---- weight gradient g32[j][f] = sum_b err8[b][j] * drop(x)[b][f].  A block owns 16-feature chunks and takes
    //      four of them (64 features) per pass: thread = (feature, one of 4 batch groups); the loads of a batch of
    //      samples are issued together, the groups meet in shared memory.
    const int fq = t & 63, bq = t >> 6;
    {
        unsigned m = 0;
        for (int c0 = blockIdx.x; c0 < F16; c0 += 4 * G) {
            const int c = c0 + (fq >> 4) * G, fl = fq & 15;
            const bool live = c < F16;
            const int f = c * 16 + fl;
            int acc[HEAD_MAX_CLASSES];
#pragma unroll
            for (int j = 0; j < HEAD_MAX_CLASSES; ++j) acc[j] = 0;
            if (live && ((sMask[c] >> fl) & 1u)) {
                // batch group bq takes samples [bq S, bq S + S): four at a time, packed into one word for __dp4a
                const int8_t* xp = p.x + f;
                const uint32_t* eT = reinterpret_cast<const uint32_t*>(sErrT);
#pragma unroll 1
                for (int b0 = bq * S; b0 < bq * S + S; b0 += 16) {
                    uint32_t xb[16];  // sixteen loads in flight
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const int b = b0 + u;
                        xb[u] = (b < B && b < bq * S + S) ? static_cast<uint32_t>(static_cast<uint8_t>(__ldg(xp + static_cast<size_t>(b) * F))) : 0u;
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int b = b0 + 4 * q;
                        if (b < bq * S + S) {
                            const int x4 = static_cast<int>(xb[4 * q] | (xb[4 * q + 1] << 8) | (xb[4 * q + 2] << 16) | (xb[4 * q + 3] << 24));
#pragma unroll
                            for (int j = 0; j < HEAD_MAX_CLASSES; ++j)
                                if (j < J) acc[j] = __dp4a(x4, static_cast<int>(eT[j * S + (b >> 2)]), acc[j]);
                        }
                    }
                }
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < HEAD_MAX_CLASSES; ++j) sRed[(bq * 16 + j) * 64 + fq] = acc[j];
            __syncthreads();
            if (live)
                for (int j = bq; j < J; j += 4) {  // thread = (feature, classes bq, bq + 4, ...)
                    int v = 0;
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) v += sRed[(gq * 16 + j) * 64 + fq];
                    p.g32[static_cast<size_t>(j) * F + f] = v;
                    m = max(m, iabs32(v));
                }
        }
        block_max(&umax[2], m, sRed);
    }
    HEAD_STAMP(7);
    if (!bounded_grid_barrier(&p.state[3], 3 * G, p.status, 6, sFlag)) return;
    HEAD_STAMP(8);

    // ---- error to the features: recompute, narrow with the tensor-wide shift, apply the dropout bits
    {
        bool z;
        const int shift = shift_for(__ldcg(&umax[1]), CALC_ERR, p.bits, &z);
        if (blockIdx.x == 0 && t == 0) *p.exp_err = shift + exp_w;  // the loss's error has exponent 0
        const bool stochastic = p.err_mode == ROUND_STOCHASTIC && shift > 0;
        // one 16-feature chunk of sample b: narrow, apply the dropout bits, store
        auto emit = [&](int b, int c, const int (&e)[16]) {
            const unsigned long long e0 = (p.sample_offset + b) * static_cast<unsigned long long>(F) + c * 16;
            uint32_t packed[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t rnd[4] = {0, 0, 0, 0};
                if (stochastic) random_block(seed, p.layer_stream + 1, (e0 >> 2) + q, rnd);
                uint32_t wd = 0;
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    wd |= static_cast<uint32_t>(static_cast<uint8_t>(narrow(e[q * 4 + r], shift, p.err_mode, rnd[r]))) << (8 * r);
                packed[q] = wd;
            }
            const unsigned bits = sMask[c];
            uint4 o;
            o.x = packed[0] & expand4(bits); o.y = packed[1] & expand4(bits >> 4);
            o.z = packed[2] & expand4(bits >> 8); o.w = packed[3] & expand4(bits >> 12);
            reinterpret_cast<uint4*>(p.e8)[static_cast<size_t>(b) * F16 + c] = o;
        };
        if (static_cast<int>(blockIdx.x) < B) {
#pragma unroll
            for (int k = 0; k < KEEP_CHUNKS; ++k) {
                const int c = t + k * HEAD_THREADS;
                if (c < F16) emit(blockIdx.x, c, ekeep[k]);
            }
        }
        for (int b = blockIdx.x; b < B; b += G)
            for (int c = t + (b == static_cast<int>(blockIdx.x) ? KEEP_CHUNKS * HEAD_THREADS : 0); c < F16; c += HEAD_THREADS) {
                int e[16];
                dgrad_chunk(sW, sErr + b * J, J, F16, c, e);
                emit(b, c, e);
            }
    }
    HEAD_STAMP(9);
    // ---- the update of the weights this block computed the gradient of
    {
        bool zero_out;
        const unsigned mg = __ldcg(&umax[2]);
        if (blockIdx.x == 0 && t == 0) *p.grad_maxabs = mg;
        if (p.update) {
            const int shift = shift_for(mg, CALC_GRAD, p.mu, &zero_out);
            const int8_t* sWb = reinterpret_cast<const int8_t*>(sW);
            for (int c0 = blockIdx.x; c0 < F16; c0 += 4 * G) {
                const int c = c0 + (fq >> 4) * G;
                if (c >= F16) continue;
                for (int j = bq; j < J; j += 4) {
                    const size_t i = static_cast<size_t>(j) * F + c * 16 + (fq & 15);
                    const uint32_t rnd = (p.grad_mode == ROUND_STOCHASTIC && shift > 0) ? random_word(seed, p.layer_stream + 2, i) : 0u;
                    const int g8 = zero_out ? 0 : narrow(p.g32[i], shift, p.grad_mode, rnd);
                    p.w[i] = static_cast<int8_t>(clamp127(static_cast<int>(sWb[i]) - g8));
                }
            }
        }
    }
    HEAD_STAMP(10);
}

size_t head_smem_bytes(int B, int F, int J) {
    size_t off = static_cast<size_t>(J) * F;
    off = (off + 2 * static_cast<size_t>(F / 16) + 15) & ~static_cast<size_t>(15);
    off = (off + static_cast<size_t>(B) * J + 15) & ~static_cast<size_t>(15);
    off += static_cast<size_t>(J) * 4 * ((((B + 3) >> 2) + 3) & ~3);
    return off + HEAD_RED_INTS * sizeof(int32_t) + 16;
}

}  // namespace
}  // namespace niti

using namespace niti;

extern "C" int niti_fc_head_supported(int B, int F, int J) {
    if (B <= 0 || F <= 0 || J <= 0) return 0;
    return (J <= HEAD_MAX_CLASSES && F % 16 == 0 && head_smem_bytes(B, F, J) <= HEAD_MAX_SMEM) ? 1 : 0;
}

extern "C" size_t niti_fc_head_scratch_bytes(int B, int F, int J) {
    if (B <= 0 || F <= 0 || J <= 0) return 0;
    return (static_cast<size_t>(B) * J + 4) * sizeof(int32_t);
}

extern "C" int niti_fc_head_train_i8(const niti_fc_head_args* a, void* stream) {
    if (a == nullptr) return NITI_ERR_BAD_ARG;
    if (!(a->x && a->exp_x && a->w && a->exp_w && a->target && a->out8 && a->exp_out && a->err8 && a->e8 && a->exp_err &&
          a->g32 && a->grad_maxabs && a->scratch && a->seed && a->B > 0 && a->F > 0 && a->J > 0))
        return NITI_ERR_BAD_ARG;
    if (a->act_round < 0 || a->act_round > 2 || a->err_round < 0 || a->err_round > 2 || a->grad_round < 0 || a->grad_round > 2)
        return NITI_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->w) | reinterpret_cast<uintptr_t>(a->e8)) % 16 != 0)
        return NITI_ERR_BAD_ARG;
    if (!niti_fc_head_supported(a->B, a->F, a->J)) return NITI_ERR_UNSUPPORTED;
    if (a->scratch_bytes < niti_fc_head_scratch_bytes(a->B, a->F, a->J)) return NITI_ERR_SCRATCH;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    HeadParams p;
    p.x = a->x; p.exp_x = a->exp_x; p.w = a->w; p.exp_w = a->exp_w; p.target = reinterpret_cast<const long long*>(a->target);
    p.out8 = a->out8; p.exp_out = a->exp_out; p.err8 = a->err8; p.e8 = a->e8; p.exp_err = a->exp_err; p.g32 = a->g32;
    p.grad_maxabs = a->grad_maxabs;
    p.state = static_cast<int32_t*>(a->scratch);
    p.out32 = p.state + 4;
    p.B = a->B; p.F = a->F; p.J = a->J; p.dropout = a->dropout ? 1 : 0; p.bits = a->bits;
    p.act_mode = a->act_round; p.err_mode = a->err_round; p.grad_mode = a->grad_round; p.mu = a->mu; p.update = a->update ? 1 : 0;
    p.seed = reinterpret_cast<const unsigned long long*>(a->seed);
    p.layer_stream = a->layer_stream; p.dropout_stream = a->dropout_stream; p.loss_stream = a->loss_stream;
    p.sample_offset = a->sample_offset;
    p.status = a->status;

    static int sms[64] = {0};
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_cuda_error(e);
    const size_t smem = head_smem_bytes(p.B, p.F, p.J);
    if (dev < 64 && sms[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms[dev] = n > 0 ? n : 1;
    }
    if (dev >= 64 || !attr_set[dev]) {
        e = cudaFuncSetAttribute(fc_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(HEAD_MAX_SMEM));
        if (e != cudaSuccess) return set_cuda_error(e);
        if (dev < 64) attr_set[dev] = true;
    }
    int grid = dev < 64 ? sms[dev] : 1;
    const int useful = p.B > p.F / 16 ? p.B : p.F / 16;
    if (grid > useful) grid = useful;

    e = cudaMemsetAsync(p.state, 0, 4 * sizeof(int32_t), st);
    if (e != cudaSuccess) return set_cuda_error(e);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(HEAD_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = g_cooperative;  // the grid is at most one block per SM
    cfg.attrs = attr; cfg.numAttrs = 1;
    return set_cuda_error(cudaLaunchKernelEx(&cfg, fc_head_kernel, p));
}
