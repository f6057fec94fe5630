// CUDA-core kernels: the memory-bound layers of the int8 training path (requantisation, max-pool,
// ReLU, dropout, loss, weight update, input quantisation) and the contractions whose shapes cannot
// fill a tensor-core tile (3-channel first convolution, 10-class FC layer).
// All of them are bandwidth- or latency-bound: 16-byte accesses along the channel axis, packed
// byte SIMD (__vmaxs4, __vcmpeq4, __dp4a), warp shuffles for reductions, one atomic per warp.
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/niti_b200.h"
#include "internal.h"
#include "requant.cuh"
#include "loss_math.cuh"
#include "grid_barrier.cuh"

namespace niti {

static inline int blocks_for(long long work_items, int threads, int cap) {
    long long b = (work_items + threads - 1) / threads;
    if (b < 1) b = 1;
    if (b > cap) b = cap;
    return static_cast<int>(b);
}
static int sm_count_simt() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

__device__ __forceinline__ unsigned iabs_u(int x) { return static_cast<unsigned>(x < 0 ? -x : x); }

__device__ __forceinline__ void warp_atomic_max(unsigned* dst, unsigned v) {
    v = __reduce_max_sync(0xFFFFFFFFu, v);
    if ((threadIdx.x & 31) == 0 && v != 0 && dst != nullptr) atomicMax(dst, v);
}

// Same for a whole block (every thread must call it): atomics on one address serialise at the L2, so a
// grid-wide maximum costs one atomic per block, not one per warp.
__device__ __forceinline__ void block_atomic_max(unsigned* dst, unsigned v) {
    __shared__ unsigned warp_part[32];
    v = __reduce_max_sync(0xFFFFFFFFu, v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) warp_part[w] = v;
    __syncthreads();
    if (w == 0) {
        unsigned x = l < static_cast<int>((blockDim.x + 31) >> 5) ? warp_part[l] : 0u;
        x = __reduce_max_sync(0xFFFFFFFFu, x);
        if (l == 0 && x != 0 && dst != nullptr) atomicMax(dst, x);
    }
    __syncthreads();
}

// ------------------------------------------------------------------------------------------------
// requantisation: int32 -> int8 by the tensor-wide shift
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
requant_kernel(const int32_t* __restrict__ acc, int8_t* __restrict__ out, const unsigned* __restrict__ maxabs,
               long long n, int kind, int target_bits, int mode, const unsigned long long* seed_p, unsigned rng_stream,
               unsigned long long rng_offset, int relu, const int32_t* exp_a, const int32_t* exp_b,
               int32_t* exp_out, int32_t* shift_out) {
    bool zero_out;
    const int shift = shift_for(*maxabs, kind, target_bits, &zero_out);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int e = shift + (exp_a ? *exp_a : 0) + (exp_b ? *exp_b : 0);
        if (exp_out) *exp_out = e;
        if (shift_out) *shift_out = shift;
    }
    const long long groups = n >> 4;  // 16 elements per thread-iteration
    const bool stochastic = (mode == ROUND_STOCHASTIC) && shift > 0;
    const unsigned long long seed = stochastic ? *seed_p : 0ull;
    const bool aligned_rng = (rng_offset & 3ull) == 0;
    for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
         g += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int4* src = reinterpret_cast<const int4*>(acc) + g * 4;
        int4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __ldcs(src + i);
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t rnd[4] = {0, 0, 0, 0};
            const unsigned long long e0 = static_cast<unsigned long long>(g) * 16 + i * 4;
            if (stochastic) {
                if (aligned_rng) random_block(seed, rng_stream, (rng_offset + e0) >> 2, rnd);
                else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) rnd[j] = random_word(seed, rng_stream, rng_offset + e0 + j);
                }
            }
            int x[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int8_t r = zero_out ? int8_t(0) : narrow(x[j], shift, mode, rnd[j]);
                if (relu && r < 0) r = 0;
                w |= static_cast<uint32_t>(static_cast<uint8_t>(r)) << (8 * j);
            }
            packed[i] = w;
        }
        reinterpret_cast<uint4*>(out)[g] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    // tail (n not a multiple of 16)
    const long long tail0 = groups << 4;
    for (long long i = tail0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        uint32_t rnd = stochastic ? random_word(seed, rng_stream, rng_offset + i) : 0u;
        int8_t r = zero_out ? int8_t(0) : narrow(acc[i], shift, mode, rnd);
        if (relu && r < 0) r = 0;
        out[i] = r;
    }
}

__global__ void __launch_bounds__(256)
absmax_kernel(const int32_t* __restrict__ acc, long long n, unsigned* maxabs) {
    unsigned m = 0;
    const long long groups = n >> 2;
    for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
         g += static_cast<long long>(gridDim.x) * blockDim.x) {
        int4 v = reinterpret_cast<const int4*>(acc)[g];
        m = max(max(m, iabs_u(v.x)), max(iabs_u(v.y), max(iabs_u(v.z), iabs_u(v.w))));
    }
    for (long long i = (groups << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        m = max(m, iabs_u(acc[i]));
    block_atomic_max(maxabs, m);
}

int absmax_i32(const int32_t* acc, long long n, unsigned* maxabs, cudaStream_t st) {
    absmax_kernel<<<blocks_for(n / 4 + 1, 256, sm_count_simt() * 8), 256, 0, st>>>(acc, n, maxabs);
    return set_cuda_error(cudaGetLastError());
}

// out[i] = sum over splits of partial[s][i]; max|out| reduced into *maxabs.
// Block = 64 int4 columns x 4 split groups: each thread sums every fourth split (loads of different
// splits are independent, so several are in flight), the groups meet in shared memory.
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const int32_t* __restrict__ partial, int splits, long long n, int32_t* __restrict__ out,
                       unsigned* maxabs) {
    __shared__ int4 sm[4][64];
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    unsigned m = 0;
    const long long groups = (n + 3) >> 2;  // n is a multiple of 4 for every caller (asserted on the host)
    for (long long g0 = static_cast<long long>(blockIdx.x) * 64; g0 < groups; g0 += static_cast<long long>(gridDim.x) * 64) {
        const long long g = g0 + tx;
        int4 s = make_int4(0, 0, 0, 0);
        if (g < groups) {
#pragma unroll 4
            for (int k = ty; k < splits; k += 4) {
                const int4 v = __ldcs(reinterpret_cast<const int4*>(partial + static_cast<long long>(k) * n) + g);
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
        }
        sm[ty][tx] = s;
        __syncthreads();
        if (ty == 0 && g < groups) {
#pragma unroll
            for (int j = 1; j < 4; ++j) { const int4 v = sm[j][tx]; s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
            reinterpret_cast<int4*>(out)[g] = s;
            m = max(max(m, iabs_u(s.x)), max(iabs_u(s.y), max(iabs_u(s.z), iabs_u(s.w))));
        }
        __syncthreads();
    }
    if (maxabs) warp_atomic_max(maxabs, m);
}

int reduce_partials(const int32_t* partial, int splits, long long n, int32_t* out, unsigned* maxabs, cudaStream_t st) {
    if (n % 4 != 0) return NITI_ERR_UNSUPPORTED;
    reduce_partials_kernel<<<blocks_for((n / 4 + 63) / 64, 1, sm_count_simt() * 8), 256, 0, st>>>(partial, splits, n, out, maxabs);
    return set_cuda_error(cudaGetLastError());
}

// Same fold for row-padded partials: partial[s][row][cols_in] -> out[row][cols_out] (cols_out <= cols_in = 32).
// One block per row; thread = (column, split group of 8).
__global__ void __launch_bounds__(256)
reduce_rows_kernel(const int32_t* __restrict__ partial, int splits, int rows, int cols_out, int32_t* __restrict__ out,
                   unsigned* maxabs) {
    __shared__ int sm[8][32];
    const int col = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int row = blockIdx.x;
    int s = 0;
    for (int k = grp; k < splits; k += 8) s += __ldcs(partial + (static_cast<long long>(k) * rows + row) * 32 + col);
    sm[grp][col] = s;
    __syncthreads();
    unsigned m = 0;
    if (grp == 0) {
#pragma unroll
        for (int j = 1; j < 8; ++j) s += sm[j][col];
        if (col < cols_out) { out[static_cast<long long>(row) * cols_out + col] = s; m = iabs_u(s); }
    }
    if (maxabs) warp_atomic_max(maxabs, m);
}

int reduce_rows32(const int32_t* partial, int splits, int rows, int cols_out, int32_t* out, unsigned* maxabs, cudaStream_t st) {
    reduce_rows_kernel<<<rows, 256, 0, st>>>(partial, splits, rows, cols_out, out, maxabs);
    return set_cuda_error(cudaGetLastError());
}

// Thin convolutions (R*S*C <= 32, the 3-channel first layer) run as GEMMs over an explicit patch
// matrix: xcol[pixel][32] holds the R*S*C bytes of the pixel's receptive field, zero padded.
// One thread per pixel: walks the receptive field in (r, s, c) order, packs the bytes into eight
// words and writes the 32-byte row with two 16-byte stores.
__global__ void __launch_bounds__(256)
im2col32_kernel(const int8_t* __restrict__ x, uint4* __restrict__ xcol, int Nimg, int H, int W, int C, int R, int S, int pad,
                const int8_t* __restrict__ w, int8_t* __restrict__ wp, int K) {
    const int rsc = R * S * C;
    const long long pixels = static_cast<long long>(Nimg) * H * W;
    // the filters of the same layer, w[K][rsc] -> wp[K][32] zero padded, ride along (wp null: not wanted)
    if (wp != nullptr)
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < K * 32; i += gridDim.x * blockDim.x) {
            const int k = i >> 5, e = i & 31;
            wp[i] = e < rsc ? w[k * rsc + e] : int8_t(0);
        }
    for (long long pix = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; pix < pixels;
         pix += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int wq = static_cast<int>(pix % W);
        const int hq = static_cast<int>((pix / W) % H);
        const long long n = pix / (static_cast<long long>(W) * H);
        uint32_t word[8];
        int c = 0, sx = 0, r = 0;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            uint32_t v = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (t * 4 + j < rsc) {
                    const int hh = hq + r - pad, ww = wq + sx - pad;
                    if (hh >= 0 && hh < H && ww >= 0 && ww < W)
                        v |= static_cast<uint32_t>(static_cast<uint8_t>(__ldg(x + ((n * H + hh) * W + ww) * C + c))) << (8 * j);
                    if (++c == C) { c = 0; if (++sx == S) { sx = 0; ++r; } }
                }
            }
            word[t] = v;
        }
        xcol[pix * 2] = make_uint4(word[0], word[1], word[2], word[3]);
        xcol[pix * 2 + 1] = make_uint4(word[4], word[5], word[6], word[7]);
    }
}
int im2col32(const int8_t* x, int8_t* xcol, int Nimg, int H, int W, int C, int R, int S, int pad, cudaStream_t st,
             const int8_t* w, int8_t* wp, int K) {
    const long long total = static_cast<long long>(Nimg) * H * W;
    im2col32_kernel<<<blocks_for(total, 256, sm_count_simt() * 16), 256, 0, st>>>(x, reinterpret_cast<uint4*>(xcol), Nimg, H, W, C, R, S, pad,
                                                                                 w, wp, K);
    return set_cuda_error(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// max-pool, ReLU, dropout
// ------------------------------------------------------------------------------------------------
// 2x2 stride 2, C % 16 == 0: one thread per 16 channels of one output pixel
__global__ void __launch_bounds__(256)
maxpool2_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int Nimg, int H, int W, int C16, int P, int Q) {
    const long long total = static_cast<long long>(Nimg) * P * Q * C16;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % C16);
        long long t = i / C16;
        const int q = static_cast<int>(t % Q); t /= Q;
        const int p = static_cast<int>(t % P);
        const int n = static_cast<int>(t / P);
        const long long base = ((static_cast<long long>(n) * H + 2 * p) * W + 2 * q) * C16 + c;
        uint4 a = __ldg(x + base), b = __ldg(x + base + C16);
        uint4 d = __ldg(x + base + static_cast<long long>(W) * C16), e = __ldg(x + base + static_cast<long long>(W) * C16 + C16);
        uint4 r;
        r.x = __vmaxs4(__vmaxs4(a.x, b.x), __vmaxs4(d.x, e.x));
        r.y = __vmaxs4(__vmaxs4(a.y, b.y), __vmaxs4(d.y, e.y));
        r.z = __vmaxs4(__vmaxs4(a.z, b.z), __vmaxs4(d.z, e.z));
        r.w = __vmaxs4(__vmaxs4(a.w, b.w), __vmaxs4(d.w, e.w));
        y[i] = r;
    }
}

// relu_mask: the position that receives dy holds the window maximum m, so "x > 0 there" is "m > 0"
__device__ __forceinline__ void route4(unsigned a, unsigned b, unsigned d, unsigned e, unsigned dy, int relu_mask,
                                       unsigned& oa, unsigned& ob, unsigned& od, unsigned& oe) {
    const unsigned m = __vmaxs4(__vmaxs4(a, b), __vmaxs4(d, e));
    if (relu_mask) dy &= __vcmpgts4(m, 0);
    const unsigned ha = __vcmpeq4(a, m);
    const unsigned hb = __vcmpeq4(b, m) & ~ha;
    const unsigned hd = __vcmpeq4(d, m) & ~(ha | hb);
    const unsigned he = ~(ha | hb | hd);  // the maximum is one of the four: what is left is the last
    oa = dy & ha; ob = dy & hb; od = dy & hd; oe = dy & he;
}

__global__ void __launch_bounds__(256)
maxpool2_bwd_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, uint4* __restrict__ dx, int Nimg, int H,
                    int W, int C16, int P, int Q, int relu_mask) {
    const long long total = static_cast<long long>(Nimg) * P * Q * C16;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % C16);
        long long t = i / C16;
        const int q = static_cast<int>(t % Q); t /= Q;
        const int p = static_cast<int>(t % P);
        const int n = static_cast<int>(t / P);
        const long long base = ((static_cast<long long>(n) * H + 2 * p) * W + 2 * q) * C16 + c;
        const long long row = static_cast<long long>(W) * C16;
        uint4 a = __ldg(x + base), b = __ldg(x + base + C16), d = __ldg(x + base + row), e = __ldg(x + base + row + C16);
        uint4 g = __ldg(dy + i);
        uint4 oa, ob, od, oe;
        route4(a.x, b.x, d.x, e.x, g.x, relu_mask, oa.x, ob.x, od.x, oe.x);
        route4(a.y, b.y, d.y, e.y, g.y, relu_mask, oa.y, ob.y, od.y, oe.y);
        route4(a.z, b.z, d.z, e.z, g.z, relu_mask, oa.z, ob.z, od.z, oe.z);
        route4(a.w, b.w, d.w, e.w, g.w, relu_mask, oa.w, ob.w, od.w, oe.w);
        dx[base] = oa; dx[base + C16] = ob; dx[base + row] = od; dx[base + row + C16] = oe;
    }
}

// any k / stride / C (pad 0): one thread per output (forward) or per input element (backward)
__global__ void maxpool_fwd_generic(const int8_t* __restrict__ x, int8_t* __restrict__ y, int Nimg, int H, int W, int C,
                                    int k, int stride, int P, int Q) {
    const long long total = static_cast<long long>(Nimg) * P * Q * C;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % C);
        long long t = i / C;
        const int q = static_cast<int>(t % Q); t /= Q;
        const int p = static_cast<int>(t % P);
        const int n = static_cast<int>(t / P);
        int m = -128;
        for (int a = 0; a < k; ++a)
            for (int b = 0; b < k; ++b)
                m = max(m, static_cast<int>(x[((static_cast<long long>(n) * H + p * stride + a) * W + q * stride + b) * C + c]));
        y[i] = static_cast<int8_t>(m);
    }
}
__global__ void maxpool_bwd_generic(const int8_t* __restrict__ x, const int8_t* __restrict__ dy, int8_t* __restrict__ dx,
                                    int Nimg, int H, int W, int C, int k, int stride, int P, int Q, int relu_mask) {
    const long long total = static_cast<long long>(Nimg) * H * W * C;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % C);
        long long t = i / C;
        const int w = static_cast<int>(t % W); t /= W;
        const int h = static_cast<int>(t % H);
        const int n = static_cast<int>(t / H);
        int sum = 0;
        // windows (p,q) that contain (h,w)
        const int p_lo = max(0, (h - k + stride) / stride), p_hi = min(P - 1, h / stride);
        const int q_lo = max(0, (w - k + stride) / stride), q_hi = min(Q - 1, w / stride);
        for (int p = p_lo; p <= p_hi; ++p)
            for (int q = q_lo; q <= q_hi; ++q) {
                int m = -129, am = 0, bm = 0;
                for (int a = 0; a < k; ++a)
                    for (int b = 0; b < k; ++b) {
                        int v = x[((static_cast<long long>(n) * H + p * stride + a) * W + q * stride + b) * C + c];
                        if (v > m) { m = v; am = a; bm = b; }
                    }
                if (p * stride + am == h && q * stride + bm == w && (!relu_mask || m > 0))
                    sum += dy[((static_cast<long long>(n) * P + p) * Q + q) * C + c];
            }
        dx[i] = static_cast<int8_t>(sum);
    }
}

__global__ void __launch_bounds__(256)
relu_fwd_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, long long n) {
    const long long groups = n >> 4;
    for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
         g += static_cast<long long>(gridDim.x) * blockDim.x) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(x) + g);
        v.x = __vmaxs4(v.x, 0); v.y = __vmaxs4(v.y, 0); v.z = __vmaxs4(v.z, 0); v.w = __vmaxs4(v.w, 0);
        reinterpret_cast<uint4*>(y)[g] = v;
    }
    for (long long i = (groups << 4) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        y[i] = x[i] > 0 ? x[i] : int8_t(0);
}
__global__ void __launch_bounds__(256)
relu_bwd_kernel(const int8_t* __restrict__ act, const int8_t* __restrict__ err, int8_t* __restrict__ out, long long n) {
    const long long groups = n >> 4;
    for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
         g += static_cast<long long>(gridDim.x) * blockDim.x) {
        uint4 a = __ldg(reinterpret_cast<const uint4*>(act) + g);
        uint4 e = __ldg(reinterpret_cast<const uint4*>(err) + g);
        uint4 o;
        o.x = e.x & __vcmpgts4(a.x, 0); o.y = e.y & __vcmpgts4(a.y, 0);
        o.z = e.z & __vcmpgts4(a.z, 0); o.w = e.w & __vcmpgts4(a.w, 0);
        reinterpret_cast<uint4*>(out)[g] = o;
    }
    for (long long i = (groups << 4) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = act[i] > 0 ? err[i] : int8_t(0);
}
__global__ void __launch_bounds__(256)
dropout_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, long long rows, long long features,
               const unsigned long long* seed_p, unsigned rng_stream) {
    const unsigned long long seed = *seed_p;
    const long long total = rows * features;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const unsigned long long f = static_cast<unsigned long long>(i % features);
        y[i] = (random_word(seed, rng_stream, f) & 1u) ? x[i] : int8_t(0);
    }
}
// features % 16 == 0: one thread owns 16 features (four generator blocks, drawn once) and walks a strip of
// rows with 16-byte accesses; the mask depends on the feature only.
constexpr int DROPOUT_ROWS_PER_THREAD = 8;
__global__ void __launch_bounds__(256)
dropout16_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long rows, long long f16,
                 const unsigned long long* seed_p, unsigned rng_stream) {
    const unsigned long long seed = *seed_p;
    const long long strips = (rows + DROPOUT_ROWS_PER_THREAD - 1) / DROPOUT_ROWS_PER_THREAD;
    const long long total = strips * f16;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long fq = i % f16, strip = i / f16;
        uint32_t m[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            uint32_t w[4];
            random_block(seed, rng_stream, static_cast<unsigned long long>(fq) * 4 + b, w);
            m[b] = ((w[0] & 1u) ? 0xFFu : 0u) | ((w[1] & 1u) ? 0xFF00u : 0u) | ((w[2] & 1u) ? 0xFF0000u : 0u) |
                   ((w[3] & 1u) ? 0xFF000000u : 0u);
        }
        const long long r0 = strip * DROPOUT_ROWS_PER_THREAD;
#pragma unroll
        for (int r = 0; r < DROPOUT_ROWS_PER_THREAD; ++r)
            if (r0 + r < rows) {
                uint4 v = __ldg(x + (r0 + r) * f16 + fq);
                v.x &= m[0]; v.y &= m[1]; v.z &= m[2]; v.w &= m[3];
                y[(r0 + r) * f16 + fq] = v;
            }
    }
}

// ------------------------------------------------------------------------------------------------
// loss (ti_loss.py:6-36), one thread per sample.  float32 steps in the reference's order; 2**s by a
// fixed sequence of IEEE double operations so that the result does not depend on a math library.
// ------------------------------------------------------------------------------------------------
constexpr int LOSS_MAX_CLASSES = 32;

__global__ void loss_kernel(const int8_t* __restrict__ out8, const int32_t* __restrict__ out_exp_p,
                            const long long* __restrict__ target, int8_t* __restrict__ err8, int B, int classes,
                            const unsigned long long* seed_p, unsigned rng_stream, unsigned long long sample_offset) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const unsigned long long seed = *seed_p;
    const int out_exp = *out_exp_p;
    float g[LOSS_MAX_CLASSES];
    long long out_sum = 0;
    if (out_exp > -7) {
        float mx = -3.0e38f;
        for (int c = 0; c < classes; ++c) {
            float s = __fdiv_rn(static_cast<float>(static_cast<int>(out8[b * classes + c]) * 47274), 32768.0f);
            s = out_exp >= 0 ? __fmul_rn(s, pow2f_int(out_exp)) : __fdiv_rn(s, pow2f_int(-out_exp));
            g[c] = s;
            mx = fmaxf(mx, s);
        }
        const float offset = __fsub_rn(mx, 10.0f);
        for (int c = 0; c < classes; ++c) {
            float s = fmaxf(__fsub_rn(g[c], offset), 0.0f);
            float v = __fsub_rn(static_cast<float>(exp2_det(static_cast<double>(s))), 1.0f);
            g[c] = v;
            out_sum += static_cast<long long>(v);
        }
    } else {
        const long long a = 1ll << (1 - 2 * out_exp), bq = 1ll << (1 - out_exp);
        for (int c = 0; c < classes; ++c) {
            const long long s = out8[b * classes + c];
            const long long gi = a + s * bq + s * s;
            out_sum += gi;
            g[c] = __ll2float_rn(gi);
        }
    }
    const float denom = __ll2float_rn(out_sum);
    long long row_sum = 0;
    for (int c = 0; c < classes; ++c) {
        g[c] = __fdiv_rn(__fmul_rn(g[c], 2048.0f), denom);
        row_sum += static_cast<long long>(g[c]);
    }
    const int tgt = static_cast<int>(target[b]);
    for (int c = 0; c < classes; ++c) {
        float v = g[c];
        if (c == tgt) v = __fsub_rn(v, __ll2float_rn(row_sum));
        const int g32 = static_cast<int>(v);  // truncation, like tensor.type(torch.int32)
        const unsigned long long idx = (sample_offset + b) * static_cast<unsigned long long>(classes) + c;
        err8[b * classes + c] = narrow(g32, 4, ROUND_STOCHASTIC, random_word(seed, rng_stream, idx));
    }
}

// ------------------------------------------------------------------------------------------------
// weight update and the flipped / transposed filter bank the error-backward convolution reads
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
update_kernel(int8_t* __restrict__ w, const int32_t* __restrict__ g32, const unsigned* __restrict__ maxabs, long long n,
              int mu, int mode, const unsigned long long* seed_p, unsigned rng_stream) {
    bool zero_out;
    const int shift = shift_for(*maxabs, CALC_GRAD, mu, &zero_out);
    const bool stochastic = (mode == ROUND_STOCHASTIC) && shift > 0;
    const unsigned long long seed = stochastic ? *seed_p : 0ull;
    const long long groups = n >> 2;  // four weights per thread-iteration: one int4 of gradients, one word of weights
    for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
         g += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int4 gv = __ldcs(reinterpret_cast<const int4*>(g32) + g);
        const uint32_t wv = reinterpret_cast<const uint32_t*>(w)[g];
        uint32_t rnd[4] = {0, 0, 0, 0};
        if (stochastic) random_block(seed, rng_stream, static_cast<unsigned long long>(g), rnd);
        const int gx[4] = {gv.x, gv.y, gv.z, gv.w};
        uint32_t o = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int g8 = zero_out ? 0 : narrow(gx[j], shift, mode, rnd[j]);
            const int wj = static_cast<int8_t>(wv >> (8 * j));
            o |= static_cast<uint32_t>(static_cast<uint8_t>(clamp127(wj - g8))) << (8 * j);
        }
        reinterpret_cast<uint32_t*>(w)[g] = o;
    }
    for (long long i = (groups << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const uint32_t rnd = stochastic ? random_word(seed, rng_stream, static_cast<unsigned long long>(i)) : 0u;
        const int g8 = zero_out ? 0 : narrow(g32[i], shift, mode, rnd);
        w[i] = static_cast<int8_t>(clamp127(static_cast<int>(w[i]) - g8));
    }
}

// All weighted layers of a step in one cooperative launch: max|g32| of every layer, a grid barrier, then
// every layer's update with its own shift.  The second read of the gradients comes from L2.
constexpr int UPDATE_MULTI_MAX = 16;
struct UpdateItem { int8_t* w; int32_t* g32; unsigned* maxabs; long long n; unsigned rng_stream; };
struct UpdateMultiParams {
    UpdateItem item[UPDATE_MULTI_MAX];
    int first_block[UPDATE_MULTI_MAX + 1];  // layer l is shared by blocks [first_block[l], first_block[l + 1])
    int count, mu, mode, clear;
    const unsigned long long* seed;
    int32_t* state;  // [count] maxima, [UPDATE_MULTI_MAX] barrier arrivals; zero at launch
    int32_t* status;
};
__device__ __forceinline__ unsigned absmax4(const int4 v) {
    return max(max(iabs_u(v.x), iabs_u(v.y)), max(iabs_u(v.z), iabs_u(v.w)));
}
__device__ __forceinline__ uint32_t update_word(const int4 gv, const uint32_t wv, const uint32_t (&rnd)[4], int shift, int mode,
                                                bool zero_out) {
    const int gx[4] = {gv.x, gv.y, gv.z, gv.w};
    uint32_t o = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int g8 = zero_out ? 0 : narrow(gx[j], shift, mode, rnd[j]);
        const int wj = static_cast<int8_t>(wv >> (8 * j));
        o |= static_cast<uint32_t>(static_cast<uint8_t>(clamp127(wj - g8))) << (8 * j);
    }
    return o;
}
// Every block works on ONE layer (blocks are dealt to the layers in proportion to their sizes on the host), so a
// block has one chain of loads -> maximum -> atomic before the barrier and one read of its layer's maximum after it.
__global__ void __launch_bounds__(256)
update_multi_kernel(const UpdateMultiParams p) {
    __shared__ int flag;
    unsigned* umax = reinterpret_cast<unsigned*>(p.state);
    int l = 0;
    while (l + 1 < p.count && static_cast<int>(blockIdx.x) >= p.first_block[l + 1]) ++l;
    const UpdateItem& it = p.item[l];
    const long long nthreads = static_cast<long long>(p.first_block[l + 1] - p.first_block[l]) * blockDim.x;
    const long long tid = static_cast<long long>(static_cast<int>(blockIdx.x) - p.first_block[l]) * blockDim.x + threadIdx.x;
    const long long groups = it.n >> 2;
    const int4* g4 = reinterpret_cast<const int4*>(it.g32);
    uint32_t* w4 = reinterpret_cast<uint32_t*>(it.w);
    // The first KEEP word groups of a thread (all of them, with the grid the host picks for VGG-sized layers) stay in
    // registers from the maximum pass to the update, together with their weights, which do not depend on the maximum:
    // after the barrier there is arithmetic and stores, no second round trip to memory.
    constexpr int KEEP = 4;
    int4 gv[KEEP];
    uint32_t wv[KEEP];
    {   // ---- the layer's maximum: the loads of all kept groups go out together, one global atomic per block
        unsigned m = 0;
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const long long g = tid + k * nthreads;
            if (g < groups) { gv[k] = g4[g]; wv[k] = w4[g]; }
        }
#pragma unroll
        for (int k = 0; k < KEEP; ++k)
            if (tid + k * nthreads < groups) m = max(m, absmax4(gv[k]));
        for (long long g = tid + KEEP * nthreads; g < groups; g += nthreads) m = max(m, absmax4(g4[g]));
        for (long long i = (groups << 2) + tid; i < it.n; i += nthreads) m = max(m, iabs_u(it.g32[i]));
        block_atomic_max(&umax[l], m);
    }
    if (!bounded_grid_barrier(&p.state[UPDATE_MULTI_MAX], static_cast<int>(gridDim.x), p.status, 7, &flag)) return;
    // ---- the update
    const unsigned mx = __ldcg(&umax[l]);
    if (tid == 0 && it.maxabs != nullptr) *it.maxabs = mx;
    bool zero_out;
    const int shift = shift_for(mx, CALC_GRAD, p.mu, &zero_out);
    const bool stochastic = (p.mode == ROUND_STOCHASTIC) && shift > 0;
    const unsigned long long seed = stochastic ? *p.seed : 0ull;
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const long long g = tid + k * nthreads;
        if (g < groups) {
            uint32_t rnd[4] = {0, 0, 0, 0};
            if (stochastic) random_block(seed, it.rng_stream, static_cast<unsigned long long>(g), rnd);
            w4[g] = update_word(gv[k], wv[k], rnd, shift, p.mode, zero_out);
            if (p.clear) reinterpret_cast<int4*>(it.g32)[g] = make_int4(0, 0, 0, 0);
        }
    }
    for (long long g = tid + KEEP * nthreads; g < groups; g += nthreads) {
        uint32_t rnd[4] = {0, 0, 0, 0};
        if (stochastic) random_block(seed, it.rng_stream, static_cast<unsigned long long>(g), rnd);
        w4[g] = update_word(__ldcs(g4 + g), w4[g], rnd, shift, p.mode, zero_out);
        if (p.clear) reinterpret_cast<int4*>(it.g32)[g] = make_int4(0, 0, 0, 0);
    }
    for (long long i = (groups << 2) + tid; i < it.n; i += nthreads) {
        const uint32_t rnd = stochastic ? random_word(seed, it.rng_stream, static_cast<unsigned long long>(i)) : 0u;
        const int g8 = zero_out ? 0 : narrow(it.g32[i], shift, p.mode, rnd);
        it.w[i] = static_cast<int8_t>(clamp127(static_cast<int>(it.w[i]) - g8));
        if (p.clear) it.g32[i] = 0;
    }
}

// ------------------------------------------------------------------------------------------------
// the update of a data-parallel step over peer memory: every rank sums ITS slice of the gradient buckets of all
// ranks, the slices' maxima are exchanged, every rank updates its slice of the weights and stores the new bytes
// into every replica.  Against all-reduce + update this moves the int32 sums once instead of twice (the way back
// carries int8 weights) and needs no second launch.
// ------------------------------------------------------------------------------------------------
constexpr int DP_MAX_RANKS = 8;
constexpr unsigned long long PEER_WAIT_LIMIT_NS = 4000000000ull;  // 4 s
// exchange area of one rank, in 32-bit words
constexpr int DPX_EPOCH = 0, DPX_ARRIVALS = 1, DPX_GO = 2 /* and DPX_GO + 1 = failed; one 8-byte word */,
              DPX_OWN_MAX = 16 /* [UPDATE_MULTI_MAX] */, DPX_FLAGS = 32 /* [DP_MAX_RANKS], written by the peers */,
              DPX_MAXIMA = 64 /* [DP_MAX_RANKS][UPDATE_MULTI_MAX], written by the peers */,
              DPX_WORDS = DPX_MAXIMA + DP_MAX_RANKS * UPDATE_MULTI_MAX;
// staged[r] (all null, or one pointer per rank; the own rank's is unused): where rank r's contribution to THIS rank's
// slice of the layer already lies in THIS rank's memory (pushed there by r during its backward pass), as the address
// word group 0 of the layer would have: the reduce phase then reads local memory instead of r's bucket.
struct DpItem { long long w_off, g_off, n; unsigned rng_stream; const int32_t* staged[DP_MAX_RANKS]; };
struct DpUpdateParams {
    DpItem item[UPDATE_MULTI_MAX];
    int first_block[UPDATE_MULTI_MAX + 1];
    int count, mu, mode, rank, world;
    int8_t* weights[DP_MAX_RANKS];
    int32_t* grads[DP_MAX_RANKS];
    int32_t* exchange[DP_MAX_RANKS];
    const unsigned long long* seed;
    unsigned* maxabs;
    int32_t* status;
};
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_sys(const int32_t* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void st_release_gpu_u64(void* p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// a peer's memory is read with system scope, so that no cache of THIS GPU can answer with an older step's value
__device__ __forceinline__ int4 ld_relaxed_sys_v4(const int4* p) {
    int4 v;
    asm volatile("ld.relaxed.sys.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int4 add4(const int4 a, const int4 b) { return make_int4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// Barrier number `seq` (grows by one per barrier, over all launches) across all blocks of all ranks.  Block 0 collects
// the arrivals of its own grid, tells every rank (thread r talks to rank r) and waits for every rank's word; the other
// blocks wait for block 0's verdict.  send_maxima: the layer maxima of this rank's slices travel with the arrival.
__device__ bool dp_barrier(const DpUpdateParams& p, int seq, int number, bool send_maxima, int* flag) {
    int32_t* L = p.exchange[p.rank];
    __syncthreads();
    if (blockIdx.x == 0) {
        if (threadIdx.x == 0) {
            const unsigned long long t0 = grid_timer_ns();
            bool ok = true;
            for (unsigned spin = 0; ld_acquire_gpu(&L[DPX_ARRIVALS]) < static_cast<int>(gridDim.x) - 1; ++spin)
                if ((spin & 63) == 63 && grid_timer_ns() - t0 > GRID_WAIT_LIMIT_NS) { ok = false; break; }
            L[DPX_ARRIVALS] = 0;  // nobody arrives again before this barrier's verdict, which is stored after this
#ifdef NITI_DP_TIMING
            reinterpret_cast<unsigned long long*>(L + 40)[5 + number] = grid_timer_ns();
#endif
            *flag = ok ? 1 : 0;
        }
        __syncthreads();
        int ok = *flag, waited_for = -1;
        if (ok && static_cast<int>(threadIdx.x) < p.world) {
            const int peer = static_cast<int>(threadIdx.x);
            int32_t* X = p.exchange[peer];
            if (send_maxima) {
                unsigned* dst = reinterpret_cast<unsigned*>(X + DPX_MAXIMA + p.rank * UPDATE_MULTI_MAX);
                for (int l = 0; l < p.count; ++l) st_relaxed_sys(dst + l, static_cast<unsigned>(__ldcg(&L[DPX_OWN_MAX + l])));
            }
            st_release_sys(&X[DPX_FLAGS + p.rank], seq);  // release: everything this grid wrote before is visible to who sees it
            const unsigned long long t0 = grid_timer_ns();
            // relaxed polls (the word is in this GPU's memory), ONE acquire fence once the peer's number is there
            for (unsigned spin = 0; ld_relaxed_sys(&L[DPX_FLAGS + peer]) - seq < 0; ++spin)
                if ((spin & 63) == 63 && grid_timer_ns() - t0 > PEER_WAIT_LIMIT_NS) { ok = 0; waited_for = peer; break; }
            fence_acq_rel_sys();
        }
        const int all_ok = __syncthreads_and(ok);
        if (!ok && p.status != nullptr && atomicCAS(p.status, 0, 9) == 0) { p.status[1] = waited_for; p.status[2] = number; }
        if (threadIdx.x == 0) {
            if (send_maxima) for (int l = 0; l < p.count; ++l) L[DPX_OWN_MAX + l] = 0;  // for the next launch
            const unsigned long long verdict = all_ok ? static_cast<unsigned long long>(static_cast<unsigned>(seq))
                                                      : (static_cast<unsigned long long>(static_cast<unsigned>(seq)) << 32);
            st_release_gpu_u64(&L[DPX_GO], verdict);
            *flag = all_ok;
        }
    } else if (threadIdx.x == 0) {
        red_release_add(&L[DPX_ARRIVALS], 1);
        const unsigned long long t0 = grid_timer_ns();
        int ok = 0;
        for (unsigned spin = 0;; ++spin) {
            const unsigned long long v = ld_acquire_gpu_u64(&L[DPX_GO]);
            if (static_cast<int>(v & 0xFFFFFFFFu) == seq) { ok = 1; break; }
            if (static_cast<int>(v >> 32) == seq) break;
            if ((spin & 63) == 63 && grid_timer_ns() - t0 > PEER_WAIT_LIMIT_NS + 2 * GRID_WAIT_LIMIT_NS) break;
        }
        *flag = ok;
    }
    __syncthreads();
    return *flag != 0;
}

// Sum of word groups [lo, hi) of one layer over all ranks, stored in place in the own bucket; returns max |sum| of
// this thread's groups.  A thread has U groups x (world - 1) peer loads in flight (about eight 16-byte loads): the
// loop is bound by the round trip to the peers, not by bandwidth.  U = 4 serves world <= 2, U = 2 world <= 4.
template <int U>
__device__ __forceinline__ unsigned reduce_slice(const DpUpdateParams& p, const DpItem& it, int4* mine, long long lo, long long hi,
                                                 long long tid, long long nthreads) {
    constexpr int SLOTS = DP_MAX_RANKS / U;  // own + peers
    unsigned m = 0;
    for (long long g0 = lo + tid; g0 < hi; g0 += U * nthreads) {
        int4 v[U][SLOTS];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long g = g0 + u * nthreads;
            if (g < hi) {
                v[u][0] = __ldcg(mine + g);
#pragma unroll
                for (int r = 1; r < SLOTS; ++r) {
                    if (r < p.world) {
                        int pr = p.rank + r;
                        if (pr >= p.world) pr -= p.world;
                        const int32_t* src = it.staged[pr] != nullptr ? it.staged[pr] : p.grads[pr] + it.g_off;
                        v[u][r] = ld_relaxed_sys_v4(reinterpret_cast<const int4*>(src) + g);
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long g = g0 + u * nthreads;
            if (g < hi) {
                int4 s = v[u][0];
#pragma unroll
                for (int r = 1; r < SLOTS; ++r)
                    if (r < p.world) s = add4(s, v[u][r]);
                mine[g] = s;
                m = max(m, absmax4(s));
            }
        }
    }
    return m;
}

// -DNITI_DP_TIMING: block 0 leaves %globaltimer stamps in the unused words 40..63 of the exchange area: 0..5 = start,
// after each barrier and each phase; 6..8 = inside barrier 1..3, when the own grid had arrived
#ifdef NITI_DP_TIMING
#define DP_STAMP(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<unsigned long long*>(L + 40)[i] = grid_timer_ns(); } while (0)
// a block in the middle of the largest layer's range, last thread: stamps 9..11 inside the update phase
#define DP_PROBE(i) do { if (static_cast<int>(blockIdx.x) == (p.first_block[p.count - 2] + p.first_block[p.count - 1]) / 2 && threadIdx.x == blockDim.x - 1) reinterpret_cast<unsigned long long*>(L + 40)[i] = grid_timer_ns(); } while (0)
#else
#define DP_STAMP(i) do { } while (0)
#define DP_PROBE(i) do { } while (0)
#endif
__global__ void __launch_bounds__(256)
dp_update_kernel(const DpUpdateParams p) {
    __shared__ int flag;
    int32_t* L = p.exchange[p.rank];
    int l = 0;
    while (l + 1 < p.count && static_cast<int>(blockIdx.x) >= p.first_block[l + 1]) ++l;
    const DpItem& it = p.item[l];
    const long long nthreads = static_cast<long long>(p.first_block[l + 1] - p.first_block[l]) * blockDim.x;
    const long long tid = static_cast<long long>(static_cast<int>(blockIdx.x) - p.first_block[l]) * blockDim.x + threadIdx.x;
    const long long groups = it.n >> 2;
    const long long lo = groups * p.rank / p.world, hi = groups * (p.rank + 1) / p.world;
    int4* mine = reinterpret_cast<int4*>(p.grads[p.rank] + it.g_off);
    const int seq0 = 3 * __ldcg(&L[DPX_EPOCH]);  // the same in every block: the word changes after the last barrier only

    DP_STAMP(0);
    // ---- 1: every rank's gradients are complete
    if (!dp_barrier(p, seq0 + 1, 1, false, &flag)) return;
    DP_STAMP(1);
    {   // ---- 2: sum this rank's slice over the ranks (in place in the own bucket), its maximum
        const unsigned m = p.world <= 2 ? reduce_slice<4>(p, it, mine, lo, hi, tid, nthreads)
                         : p.world <= 4 ? reduce_slice<2>(p, it, mine, lo, hi, tid, nthreads)
                                        : reduce_slice<1>(p, it, mine, lo, hi, tid, nthreads);
        block_atomic_max(reinterpret_cast<unsigned*>(&L[DPX_OWN_MAX + l]), m);
    }
    DP_STAMP(2);
    // ---- 3: the slices' maxima reach every rank; every rank has finished reading the others' buckets
    if (!dp_barrier(p, seq0 + 2, 2, true, &flag)) return;
    DP_STAMP(3);
    {
        unsigned mx = 0;
        for (int r = 0; r < p.world; ++r) mx = max(mx, static_cast<unsigned>(__ldcg(&L[DPX_MAXIMA + r * UPDATE_MULTI_MAX + l])));
        if (tid == 0 && p.maxabs != nullptr) p.maxabs[l] = mx;
        bool zero_out;
        const int shift = shift_for(mx, CALC_GRAD, p.mu, &zero_out);
        const bool stochastic = (p.mode == ROUND_STOCHASTIC) && shift > 0;
        const unsigned long long seed = stochastic ? *p.seed : 0ull;
        const uint32_t* w_own = reinterpret_cast<const uint32_t*>(p.weights[p.rank] + it.w_off);
        for (long long g0 = lo + tid; g0 < hi; g0 += 4 * nthreads) {  // the own slice: four groups' loads go out together
            int4 sv[4];
            uint32_t wv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long g = g0 + u * nthreads;
                if (g < hi) { sv[u] = __ldcg(mine + g); wv[u] = w_own[g]; }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long g = g0 + u * nthreads;
                if (g < hi) {
                    uint32_t rnd[4] = {0, 0, 0, 0};
                    if (stochastic) random_block(seed, it.rng_stream, static_cast<unsigned long long>(g), rnd);
                    const uint32_t o = update_word(sv[u], wv[u], rnd, shift, p.mode, zero_out);
#pragma unroll
                    for (int r = 0; r < DP_MAX_RANKS; ++r)
                        if (r < p.world) reinterpret_cast<uint32_t*>(p.weights[r] + it.w_off)[g] = o;
                    mine[g] = make_int4(0, 0, 0, 0);
                }
            }
        }
        DP_PROBE(9);
        // the rest of the own bucket: the weight-gradient kernels of the next step add into a zeroed bucket
        for (long long g = tid; g < lo; g += nthreads) mine[g] = make_int4(0, 0, 0, 0);
        for (long long g = hi + tid; g < groups; g += nthreads) mine[g] = make_int4(0, 0, 0, 0);
        DP_PROBE(10);
        __threadfence_system();
        DP_PROBE(11);
    }
    DP_STAMP(4);
    // ---- 4: every rank's weight stores have landed
    if (!dp_barrier(p, seq0 + 3, 3, false, &flag)) return;
    DP_STAMP(5);
    if (blockIdx.x == 0 && threadIdx.x == 0) L[DPX_EPOCH] = L[DPX_EPOCH] + 1;
}

// ------------------------------------------------------------------------------------------------
// input quantisation (ti_torch.py:341-356 + the permute of ti_net.py:19)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) absmax_f32_kernel(const float* __restrict__ x, long long n, unsigned* bits) {
    unsigned m = 0;  // |x| as IEEE bits orders like the value for non-negative floats
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        m = max(m, __float_as_uint(fabsf(x[i])));
    block_atomic_max(bits, m);
}
__global__ void __launch_bounds__(256)
quantize_input_kernel(const float* __restrict__ x, int8_t* __restrict__ x8, int32_t* exp_out, const unsigned* bits,
                      int Nimg, int C, int H, int W) {
    const unsigned mb = *bits;
    // ceil(log2(r)) from the exponent and mantissa fields of r
    const int e = static_cast<int>((mb >> 23) & 0xFF) - 127;
    const int bw = (mb & 0x7FFFFF) ? e + 1 : e;
    if (blockIdx.x == 0 && threadIdx.x == 0) *exp_out = bw - 7;
    const float scale = pow2f_int(7 - bw);
    const long long total = static_cast<long long>(Nimg) * H * W * C;
    for (long long o = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; o < total;
         o += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(o % C);
        long long t = o / C;
        const int w = static_cast<int>(t % W); t /= W;
        const int h = static_cast<int>(t % H);
        const int n = static_cast<int>(t / H);
        const float v = rintf(__fmul_rn(x[((static_cast<long long>(n) * C + c) * H + h) * W + w], scale));
        x8[o] = static_cast<int8_t>(fminf(fmaxf(v, -128.0f), 127.0f));
    }
}

// ------------------------------------------------------------------------------------------------
// CUDA-core contractions: shapes the tensor-core kernels do not take (odd channel counts, other
// paddings) and the 10-class FC layer.
// ------------------------------------------------------------------------------------------------
// Convolution forward, any shape: one thread per output element.
__global__ void conv_fprop_direct_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ w,
                                         int32_t* __restrict__ y32, unsigned* maxabs, int Nimg, int H, int W, int C, int K,
                                         int R, int S, int pad, int P, int Q) {
    const long long total = static_cast<long long>(Nimg) * P * Q * K;
    unsigned m = 0;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int k = static_cast<int>(i % K);
        long long t = i / K;
        const int q = static_cast<int>(t % Q); t /= Q;
        const int p = static_cast<int>(t % P);
        const long long n = t / P;
        int acc = 0;
        for (int r = 0; r < R; ++r) {
            const int hh = p + r - pad;
            if (hh < 0 || hh >= H) continue;
            for (int s = 0; s < S; ++s) {
                const int ww = q + s - pad;
                if (ww < 0 || ww >= W) continue;
                const int8_t* xp = x + ((n * H + hh) * W + ww) * C;
                const int8_t* wp = w + ((static_cast<long long>(k) * R + r) * S + s) * C;
                for (int c = 0; c < C; ++c) acc += static_cast<int>(xp[c]) * static_cast<int>(wp[c]);
            }
        }
        y32[i] = acc;
        m = max(m, iabs_u(acc));
    }
    warp_atomic_max(maxabs, m);
}
// Error-backward, any shape with "same" padding: dX[n,h,w,c] = sum_{r,s,k} err[n,h+pad-r,w+pad-s,k] * w[k,r,s,c].
__global__ void conv_dgrad_direct_kernel(const int8_t* __restrict__ err, const int8_t* __restrict__ w,
                                         int32_t* __restrict__ e32, unsigned* maxabs, int Nimg, int H, int W, int C, int K,
                                         int R, int S, int pad) {
    const long long total = static_cast<long long>(Nimg) * H * W * C;
    unsigned m = 0;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % C);
        long long t = i / C;
        const int wq = static_cast<int>(t % W); t /= W;
        const int hq = static_cast<int>(t % H);
        const long long n = t / H;
        int acc = 0;
        for (int r = 0; r < R; ++r) {
            const int hh = hq + pad - r;
            if (hh < 0 || hh >= H) continue;
            for (int s = 0; s < S; ++s) {
                const int ww = wq + pad - s;
                if (ww < 0 || ww >= W) continue;
                const int8_t* ep = err + ((n * H + hh) * W + ww) * K;
                for (int k = 0; k < K; ++k)
                    acc += static_cast<int>(ep[k]) * static_cast<int>(w[((static_cast<long long>(k) * R + r) * S + s) * C + c]);
            }
        }
        e32[i] = acc;
        m = max(m, iabs_u(acc));
    }
    warp_atomic_max(maxabs, m);
}
int simt_conv_fprop(const int8_t* x, const int8_t* w, int32_t* y32, unsigned* maxabs, int Nimg, int H, int W, int C,
                    int K, int R, int S, int pad, cudaStream_t st) {
    const int P = H + 2 * pad - R + 1, Q = W + 2 * pad - S + 1;
    const long long total = static_cast<long long>(Nimg) * P * Q * K;
    conv_fprop_direct_kernel<<<blocks_for(total, 256, sm_count_simt() * 16), 256, 0, st>>>(x, w, y32, maxabs, Nimg, H, W, C, K,
                                                                                         R, S, pad, P, Q);
    return set_cuda_error(cudaGetLastError());
}
int simt_conv_dgrad(const int8_t* err, const int8_t* w, int32_t* e32, unsigned* maxabs, int Nimg, int H, int W, int C,
                    int K, int R, int S, int pad, cudaStream_t st) {
    const long long total = static_cast<long long>(Nimg) * H * W * C;
    conv_dgrad_direct_kernel<<<blocks_for(total, 256, sm_count_simt() * 16), 256, 0, st>>>(err, w, e32, maxabs, Nimg, H, W, C,
                                                                                         K, R, S, pad);
    return set_cuda_error(cudaGetLastError());
}

// Weight gradient, any shape: one thread per gradient element, summing over all pixels.
__global__ void conv_wgrad_direct_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ err,
                                         int32_t* __restrict__ g32, unsigned* maxabs, int Nimg, int H, int W, int C, int K,
                                         int R, int S, int pad, int P, int Q) {
    const long long total = static_cast<long long>(K) * R * S * C;
    unsigned m = 0;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % C);
        long long t = i / C;
        const int s = static_cast<int>(t % S); t /= S;
        const int r = static_cast<int>(t % R);
        const int k = static_cast<int>(t / R);
        int acc = 0;
        for (long long n = 0; n < Nimg; ++n)
            for (int p = 0; p < P; ++p) {
                const int hh = p + r - pad;
                if (hh < 0 || hh >= H) continue;
                for (int q = 0; q < Q; ++q) {
                    const int ww = q + s - pad;
                    if (ww < 0 || ww >= W) continue;
                    acc += static_cast<int>(err[((n * P + p) * Q + q) * K + k]) * static_cast<int>(x[((n * H + hh) * W + ww) * C + c]);
                }
            }
        g32[i] = acc;
        m = max(m, iabs_u(acc));
    }
    warp_atomic_max(maxabs, m);
}
int simt_conv_wgrad(const int8_t* x, const int8_t* err, int32_t* g32, unsigned* maxabs, int Nimg, int H, int W, int C,
                    int K, int R, int S, int pad, cudaStream_t st) {
    const int P = H + 2 * pad - R + 1, Q = W + 2 * pad - S + 1;
    const long long total = static_cast<long long>(K) * R * S * C;
    conv_wgrad_direct_kernel<<<blocks_for(total, 128, 1 << 20), 128, 0, st>>>(x, err, g32, maxabs, Nimg, H, W, C, K, R, S, pad, P, Q);
    return set_cuda_error(cudaGetLastError());
}

// GEMM, both operands contiguous along the reduction (trans_a = 0, trans_b = 1): one warp per
// output element, 16-byte loads, dp4a, shuffle reduction.  The 10-class FC forward.
__global__ void __launch_bounds__(256)
gemm_kk_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B, int32_t* __restrict__ C32, unsigned* maxabs,
               int M, int N, int K) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    unsigned mx = 0;
    const bool vec = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) % 16 == 0);
    for (long long o = warp; o < static_cast<long long>(M) * N; o += nwarps) {
        const int m = static_cast<int>(o / N), n = static_cast<int>(o % N);
        const int8_t* a = A + static_cast<long long>(m) * K;
        const int8_t* b = B + static_cast<long long>(n) * K;
        int acc = 0;
        if (vec) {
            for (int k = lane * 16; k < K; k += 32 * 16) {
                const int4 av = __ldg(reinterpret_cast<const int4*>(a + k));
                const int4 bv = __ldg(reinterpret_cast<const int4*>(b + k));
                acc = __dp4a(av.x, bv.x, acc); acc = __dp4a(av.y, bv.y, acc);
                acc = __dp4a(av.z, bv.z, acc); acc = __dp4a(av.w, bv.w, acc);
            }
        } else {
            for (int k = lane; k < K; k += 32) acc += static_cast<int>(a[k]) * static_cast<int>(b[k]);
        }
        acc = __reduce_add_sync(0xFFFFFFFFu, acc);
        if (lane == 0) { C32[o] = acc; mx = max(mx, iabs_u(acc)); }
    }
    if (lane == 0 && mx != 0 && maxabs != nullptr) atomicMax(maxabs, mx);
}
// GEMM, any majors: one thread per output element, consecutive threads along N.
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B, int32_t* __restrict__ C32,
                    unsigned* maxabs, int M, int N, int K, int trans_a, int trans_b) {
    unsigned mx = 0;
    const long long sa_m = trans_a ? 1 : K, sa_k = trans_a ? M : 1;
    const long long sb_k = trans_b ? 1 : N, sb_n = trans_b ? K : 1;
    for (long long o = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; o < static_cast<long long>(M) * N;
         o += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long m = o / N, n = o % N;
        int acc = 0;
        for (int k = 0; k < K; ++k) acc += static_cast<int>(A[m * sa_m + k * sa_k]) * static_cast<int>(B[k * sb_k + n * sb_n]);
        C32[o] = acc;
        mx = max(mx, iabs_u(acc));
    }
    warp_atomic_max(maxabs, mx);
}
// GEMM with B stored [K][N], N % 4 == 0: each thread produces four adjacent outputs from 32-bit
// loads of B (FC error e*W and FC gradient e^T*a: short reductions, wide outputs).
__global__ void __launch_bounds__(256)
gemm_bn4_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B, int32_t* __restrict__ C32, unsigned* maxabs,
                int M, int N, int K, int trans_a) {
    unsigned mx = 0;
    const int n4 = N >> 2;
    const long long sa_m = trans_a ? 1 : K, sa_k = trans_a ? M : 1;
    for (long long o = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; o < static_cast<long long>(M) * n4;
         o += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long m = o / n4;
        const int nq = static_cast<int>(o % n4);
        const uint32_t* bp = reinterpret_cast<const uint32_t*>(B) + nq;
        const int8_t* ap = A + m * sa_m;
        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
#pragma unroll 16
        for (int k = 0; k < K; ++k) {
            const int a = ap[k * sa_k];
            const uint32_t b = __ldg(bp + static_cast<long long>(k) * n4);
            a0 += a * static_cast<int8_t>(b); a1 += a * static_cast<int8_t>(b >> 8);
            a2 += a * static_cast<int8_t>(b >> 16); a3 += a * static_cast<int8_t>(b >> 24);
        }
        reinterpret_cast<int4*>(C32)[o] = make_int4(a0, a1, a2, a3);
        mx = max(max(mx, iabs_u(a0)), max(iabs_u(a1), max(iabs_u(a2), iabs_u(a3))));
    }
    warp_atomic_max(maxabs, mx);
}
int simt_gemm(const int8_t* A, const int8_t* B, int32_t* C32, unsigned* maxabs, int M, int N, int K, int trans_a,
              int trans_b, cudaStream_t st) {
    const long long outs = static_cast<long long>(M) * N;
    if (!trans_a && trans_b && K >= 256)
        gemm_kk_kernel<<<blocks_for(outs * 32, 256, sm_count_simt() * 16), 256, 0, st>>>(A, B, C32, maxabs, M, N, K);
    else if (!trans_b && N % 4 == 0 && reinterpret_cast<uintptr_t>(B) % 4 == 0 && reinterpret_cast<uintptr_t>(C32) % 16 == 0)
        gemm_bn4_kernel<<<blocks_for(outs / 4, 128, sm_count_simt() * 32), 128, 0, st>>>(A, B, C32, maxabs, M, N, K, trans_a);
    else
        gemm_generic_kernel<<<blocks_for(outs, 256, sm_count_simt() * 32), 256, 0, st>>>(A, B, C32, maxabs, M, N, K, trans_a, trans_b);
    return set_cuda_error(cudaGetLastError());
}

}  // namespace niti

// ================================================================================================
// C ABI for the CUDA-core kernels
// ================================================================================================
using namespace niti;

#define NITI_REQUIRE(cond) do { if (!(cond)) return NITI_ERR_BAD_ARG; } while (0)

extern "C" int niti_requant_i8(const int32_t* acc, int8_t* out, const uint32_t* maxabs, int64_t n, int kind,
                               int target_bits, int round_mode, const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset,
                               int relu, const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                               void* stream) {
    NITI_REQUIRE(acc && out && maxabs && n >= 0 && kind >= 0 && kind <= 2 && round_mode >= 0 && round_mode <= 2);
    NITI_REQUIRE(seed || round_mode != NITI_ROUND_STOCHASTIC);
    NITI_REQUIRE(reinterpret_cast<uintptr_t>(acc) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0);
    requant_kernel<<<blocks_for(n / 16 + 1, 256, sm_count_simt() * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        acc, out, maxabs, n, kind, target_bits, round_mode, reinterpret_cast<const unsigned long long*>(seed), rng_stream, rng_offset, relu, exp_a, exp_b, exp_out, shift_out);
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_absmax_i32(const int32_t* acc, int64_t n, uint32_t* maxabs, void* stream) {
    NITI_REQUIRE(acc && maxabs && n >= 0 && reinterpret_cast<uintptr_t>(acc) % 16 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = set_cuda_error(cudaMemsetAsync(maxabs, 0, 4, st))) return e;
    absmax_kernel<<<blocks_for(n / 4 + 1, 256, sm_count_simt() * 8), 256, 0, st>>>(acc, n, maxabs);
    return set_cuda_error(cudaGetLastError());
}

// Two signed 4-bit values per byte, element 2i in the low nibble (the packing of CUTLASS' int4b_t arrays), to int8.
__global__ void __launch_bounds__(256) unpack_i4_kernel(const uint8_t* __restrict__ in, int8_t* __restrict__ out, long long nbytes) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nbytes; i += stride) {
        const unsigned b = in[i];
        const int lo = static_cast<int>(b << 28) >> 28, hi = static_cast<int>(b << 24) >> 28;  // sign-extend each nibble
        reinterpret_cast<char2*>(out)[i] = make_char2(static_cast<signed char>(lo), static_cast<signed char>(hi));
    }
}
namespace niti {
int unpack_i4(const uint8_t* in, int8_t* out, long long nbytes, cudaStream_t st) {
    unpack_i4_kernel<<<blocks_for(nbytes, 256, sm_count_simt() * 16), 256, 0, st>>>(in, out, nbytes);
    return set_cuda_error(cudaGetLastError());
}
}  // namespace niti

// Grouped cross-correlation with ONE input channel per group and a batch of one: the only form in which the
// reference calls int8conv_cuda.group_conv (conv2d_weight_int8 folds batch and channels into groups and the error
// maps into filters as large as the image).  out[p][q][g*Kg + k] = sum_{r,s} in[p+r-pad][q+s-pad][g] * wt[g*Kg+k][r][s].
// One warp per output channel: the lanes split the filter window, a shuffle tree adds up, exact int32.
__global__ void __launch_bounds__(256)
group_conv1_kernel(const int8_t* __restrict__ in, const int8_t* __restrict__ wt, int32_t* __restrict__ out, int H, int W,
                   int G, int Kg, int R, int S, int pad, int P, int Q) {
    const int lane = threadIdx.x & 31;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    const long long chans = static_cast<long long>(G) * Kg;
    for (long long oc = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; oc < chans; oc += warps) {
        const int g = static_cast<int>(oc / Kg);
        const int8_t* f = wt + oc * R * S;
        for (int p = 0; p < P; ++p)
            for (int q = 0; q < Q; ++q) {
                int acc = 0;
                for (int i = lane; i < R * S; i += 32) {
                    const int r = i / S, sx = i - r * S;
                    const int hh = p + r - pad, ww = q + sx - pad;
                    if (hh >= 0 && hh < H && ww >= 0 && ww < W)
                        acc += static_cast<int>(in[(static_cast<long long>(hh) * W + ww) * G + g]) * static_cast<int>(f[i]);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
                if (lane == 0) out[(static_cast<long long>(p) * Q + q) * chans + oc] = acc;
            }
    }
}

extern "C" int niti_group_conv1_i8(const int8_t* in, const int8_t* wt, int32_t* out32, int H, int W, int G, int Kg, int R, int S,
                                   int pad, void* stream) {
    NITI_REQUIRE(in && wt && out32 && H > 0 && W > 0 && G > 0 && Kg > 0 && R > 0 && S > 0 && pad >= 0);
    const int P = H + 2 * pad - R + 1, Q = W + 2 * pad - S + 1;
    if (P <= 0 || Q <= 0) return NITI_ERR_BAD_ARG;
    const long long chans = static_cast<long long>(G) * Kg;
    group_conv1_kernel<<<blocks_for(chans * 32, 256, sm_count_simt() * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        in, wt, out32, H, W, G, Kg, R, S, pad, P, Q);
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_maxpool_fwd_i8(const int8_t* x, int8_t* y, int N, int H, int W, int C, int k, int stride, void* stream) {
    NITI_REQUIRE(x && y && N > 0 && H >= k && W >= k && C > 0 && k > 0 && stride > 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int P = (H - k) / stride + 1, Q = (W - k) / stride + 1;
    if (k == 2 && stride == 2 && C % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
        const long long total = static_cast<long long>(N) * P * Q * (C / 16);
        maxpool2_fwd_kernel<<<blocks_for(total, 256, sm_count_simt() * 16), 256, 0, st>>>(
            reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(y), N, H, W, C / 16, P, Q);
    } else {
        const long long total = static_cast<long long>(N) * P * Q * C;
        maxpool_fwd_generic<<<blocks_for(total, 256, sm_count_simt() * 16), 256, 0, st>>>(x, y, N, H, W, C, k, stride, P, Q);
    }
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_maxpool_bwd_i8(const int8_t* x, const int8_t* dy, int8_t* dx, int N, int H, int W, int C, int k,
                                   int stride, int relu_mask, void* stream) {
    NITI_REQUIRE(x && dy && dx && N > 0 && H >= k && W >= k && C > 0 && k > 0 && stride > 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int P = (H - k) / stride + 1, Q = (W - k) / stride + 1;
    const bool al = (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) % 16 == 0;
    if (k == 2 && stride == 2 && C % 16 == 0 && H % 2 == 0 && W % 2 == 0 && al) {
        const long long total = static_cast<long long>(N) * P * Q * (C / 16);
        maxpool2_bwd_kernel<<<blocks_for(total, 256, sm_count_simt() * 16), 256, 0, st>>>(
            reinterpret_cast<const uint4*>(x), reinterpret_cast<const uint4*>(dy), reinterpret_cast<uint4*>(dx), N, H, W, C / 16, P, Q, relu_mask);
    } else {
        const long long total = static_cast<long long>(N) * H * W * C;
        maxpool_bwd_generic<<<blocks_for(total, 256, sm_count_simt() * 16), 256, 0, st>>>(x, dy, dx, N, H, W, C, k, stride, P, Q, relu_mask);
    }
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_relu_fwd_i8(const int8_t* x, int8_t* y, int64_t n, void* stream) {
    NITI_REQUIRE(x && y && n >= 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16 == 0);
    relu_fwd_kernel<<<blocks_for(n / 16 + 1, 256, sm_count_simt() * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n);
    return set_cuda_error(cudaGetLastError());
}
extern "C" int niti_relu_bwd_i8(const int8_t* act, const int8_t* err, int8_t* out, int64_t n, void* stream) {
    NITI_REQUIRE(act && err && out && n >= 0);
    NITI_REQUIRE((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(err) | reinterpret_cast<uintptr_t>(out)) % 16 == 0);
    relu_bwd_kernel<<<blocks_for(n / 16 + 1, 256, sm_count_simt() * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(act, err, out, n);
    return set_cuda_error(cudaGetLastError());
}
extern "C" int niti_dropout_i8(const int8_t* x, int8_t* y, int64_t rows, int64_t features, const uint64_t* seed,
                               uint32_t rng_stream, void* stream) {
    NITI_REQUIRE(x && y && seed && rows >= 0 && features > 0);
    if (features % 16 == 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16 == 0) {
        const long long work = ((rows + DROPOUT_ROWS_PER_THREAD - 1) / DROPOUT_ROWS_PER_THREAD) * (features / 16);
        dropout16_kernel<<<blocks_for(work, 128, sm_count_simt() * 8), 128, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(y), rows, features / 16,
            reinterpret_cast<const unsigned long long*>(seed), rng_stream);
    } else {
        dropout_kernel<<<blocks_for(rows * features, 256, sm_count_simt() * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            x, y, rows, features, reinterpret_cast<const unsigned long long*>(seed), rng_stream);
    }
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_loss_i8(const int8_t* out8, const int32_t* out_exp, const int64_t* target, int8_t* err8, int B,
                            int classes, const uint64_t* seed, uint32_t rng_stream, uint64_t sample_offset, void* stream) {
    NITI_REQUIRE(out8 && out_exp && target && err8 && seed && B > 0 && classes > 0);
    if (classes > LOSS_MAX_CLASSES) return NITI_ERR_UNSUPPORTED;
    loss_kernel<<<(B + 63) / 64, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        out8, out_exp, reinterpret_cast<const long long*>(target), err8, B, classes,
        reinterpret_cast<const unsigned long long*>(seed), rng_stream, sample_offset);
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_update_i8(int8_t* w, const int32_t* g32, const uint32_t* maxabs, int64_t n, int mu, int round_mode,
                              const uint64_t* seed, uint32_t rng_stream, void* stream) {
    NITI_REQUIRE(w && g32 && maxabs && n > 0 && round_mode >= 0 && round_mode <= 2);
    NITI_REQUIRE(seed || round_mode != NITI_ROUND_STOCHASTIC);
    NITI_REQUIRE(reinterpret_cast<uintptr_t>(w) % 4 == 0 && reinterpret_cast<uintptr_t>(g32) % 16 == 0);
    update_kernel<<<blocks_for(n / 4 + 1, 256, sm_count_simt() * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        w, g32, maxabs, n, mu, round_mode, reinterpret_cast<const unsigned long long*>(seed), rng_stream);
    return set_cuda_error(cudaGetLastError());
}

extern "C" size_t niti_update_multi_scratch_bytes(void) { return 2 * UPDATE_MULTI_MAX * sizeof(int32_t); }

extern "C" int niti_update_multi_i8(const niti_update_item* items, int count, int mu, int round_mode, int clear_gradients,
                                    const uint64_t* seed, void* scratch, size_t scratch_bytes, int32_t* status, void* stream) {
    NITI_REQUIRE(items && count > 0 && round_mode >= 0 && round_mode <= 2 && scratch);
    NITI_REQUIRE(seed || round_mode != NITI_ROUND_STOCHASTIC);
    if (scratch_bytes < niti_update_multi_scratch_bytes()) return NITI_ERR_SCRATCH;
    for (int i = 0; i < count; ++i) {
        NITI_REQUIRE(items[i].w && items[i].g32 && items[i].n > 0);
        NITI_REQUIRE(reinterpret_cast<uintptr_t>(items[i].w) % 4 == 0 && reinterpret_cast<uintptr_t>(items[i].g32) % 16 == 0);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static int blocks_per_sm = 0;
    if (blocks_per_sm == 0) {
        int n = 0;
        if (int e = set_cuda_error(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, update_multi_kernel, 256, 0))) return e;
        blocks_per_sm = n < 1 ? 1 : (n > 8 ? 8 : n);
    }
    for (int first = 0; first < count; first += UPDATE_MULTI_MAX) {
        UpdateMultiParams p;
        p.count = count - first < UPDATE_MULTI_MAX ? count - first : UPDATE_MULTI_MAX;
        long long total = 0;
        for (int i = 0; i < p.count; ++i) {
            const niti_update_item& it = items[first + i];
            p.item[i] = UpdateItem{it.w, it.g32, it.maxabs, it.n, it.rng_stream};
            total += it.n;
        }
        p.mu = mu; p.mode = round_mode; p.clear = clear_gradients ? 1 : 0;
        p.seed = reinterpret_cast<const unsigned long long*>(seed);
        p.state = static_cast<int32_t*>(scratch);
        p.status = status;
        if (int e = set_cuda_error(cudaMemsetAsync(scratch, 0, niti_update_multi_scratch_bytes(), st))) return e;
        // deal the blocks of one resident wave to the layers in proportion to their sizes (at least one each)
        const int wave = sm_count_simt() * blocks_per_sm;
        int grid = 0;
        for (int i = 0; i < p.count; ++i) {
            long long share = (static_cast<long long>(wave - p.count) * p.item[i].n) / (total > 0 ? total : 1);
            const long long useful = (p.item[i].n / 4 + 255) / 256;  // a block per 256 word groups is as fine as it gets
            if (share > useful - 1) share = useful - 1;
            if (share < 0) share = 0;
            p.first_block[i] = grid;
            grid += 1 + static_cast<int>(share);
        }
        p.first_block[p.count] = grid;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = g_cooperative;  // the grid fits in one wave
        cfg.attrs = attr; cfg.numAttrs = 1;
        if (int e = set_cuda_error(cudaLaunchKernelEx(&cfg, update_multi_kernel, p))) return e;
    }
    return NITI_OK;
}

extern "C" size_t niti_dp_exchange_bytes(void) { return DPX_WORDS * sizeof(int32_t); }

extern "C" int niti_peer_copy(void* dst, const void* src, size_t bytes, void* stream) {
    NITI_REQUIRE(dst && src && bytes > 0);
    return set_cuda_error(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
}

extern "C" int niti_dp_update_i8(const niti_dp_update_args* a, void* stream) {
    NITI_REQUIRE(a && a->items && a->count > 0 && a->count <= UPDATE_MULTI_MAX);
    NITI_REQUIRE(a->world >= 1 && a->world <= DP_MAX_RANKS && a->rank >= 0 && a->rank < a->world);
    NITI_REQUIRE(a->weights && a->grads && a->exchange && a->round_mode >= 0 && a->round_mode <= 2);
    NITI_REQUIRE(a->seed || a->round_mode != NITI_ROUND_STOCHASTIC);
    DpUpdateParams p;
    long long total = 0;
    for (int i = 0; i < a->count; ++i) {
        const niti_dp_item& it = a->items[i];
        NITI_REQUIRE(it.n > 0 && it.n % 4 == 0 && it.w_offset % 4 == 0 && it.g_offset % 4 == 0);
        p.item[i] = DpItem{it.w_offset, it.g_offset, it.n, it.rng_stream, {}};
        for (int r = 0; r < DP_MAX_RANKS; ++r) {
            p.item[i].staged[r] = (r < a->world && r != a->rank) ? static_cast<const int32_t*>(it.staged[r]) : nullptr;
            NITI_REQUIRE(reinterpret_cast<uintptr_t>(p.item[i].staged[r]) % 16 == 0);
        }
        {   // all peers staged, or none
            int have = 0;
            for (int r = 0; r < a->world; ++r) have += (r != a->rank && p.item[i].staged[r] != nullptr) ? 1 : 0;
            NITI_REQUIRE(have == 0 || have == a->world - 1);
        }
        total += it.n;
    }
    for (int r = 0; r < DP_MAX_RANKS; ++r) {
        const int s = r < a->world ? r : a->rank;  // unused slots repeat the own pointers
        NITI_REQUIRE(a->weights[s] && a->grads[s] && a->exchange[s]);
        NITI_REQUIRE(reinterpret_cast<uintptr_t>(a->weights[s]) % 4 == 0 && reinterpret_cast<uintptr_t>(a->grads[s]) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(a->exchange[s]) % 8 == 0);
        p.weights[r] = static_cast<int8_t*>(a->weights[s]);
        p.grads[r] = static_cast<int32_t*>(a->grads[s]);
        p.exchange[r] = static_cast<int32_t*>(a->exchange[s]);
    }
    p.count = a->count; p.mu = a->mu; p.mode = a->round_mode; p.rank = a->rank; p.world = a->world;
    p.seed = reinterpret_cast<const unsigned long long*>(a->seed);
    p.maxabs = a->maxabs; p.status = a->status;
    static int blocks_per_sm = 0;
    if (blocks_per_sm == 0) {
        int n = 0;
        if (int e = set_cuda_error(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, dp_update_kernel, 256, 0))) return e;
        blocks_per_sm = n < 1 ? 1 : (n > 8 ? 8 : n);
    }
    // one resident wave, dealt to the layers in proportion to their sizes; a block per 256 word groups of the WHOLE
    // layer is as fine as it gets (the clearing pass walks the whole layer, the slice is 1 / world of it)
    const int wave = sm_count_simt() * blocks_per_sm;
    int grid = 0;
    for (int i = 0; i < p.count; ++i) {
        long long share = (static_cast<long long>(wave - p.count) * p.item[i].n) / (total > 0 ? total : 1);
        const long long useful = (p.item[i].n / 4 + 255) / 256;
        if (share > useful - 1) share = useful - 1;
        if (share < 0) share = 0;
        p.first_block[i] = grid;
        grid += 1 + static_cast<int>(share);
    }
    p.first_block[p.count] = grid;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = g_cooperative;  // the grid fits in one wave
    cfg.attrs = attr; cfg.numAttrs = 1;
    return set_cuda_error(cudaLaunchKernelEx(&cfg, dp_update_kernel, p));
}

// Self-test of the bounded grid barrier: ONE block waits at a barrier that expects two.  Nothing else will ever arrive,
// so the wait runs into its 0.5 s limit, the block writes {code 8, block, target} to `status` and the kernel returns.
__global__ void barrier_timeout_selftest_kernel(int32_t* counter, int32_t* status) {
    __shared__ int flag;
    if (bounded_grid_barrier(counter, 2, status, 8, &flag)) status[3] = 1;  // cannot happen: one arrival, target two
}
extern "C" int niti_selftest_barrier_timeout(int32_t* scratch, int32_t* status, void* stream) {
    NITI_REQUIRE(scratch && status);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = set_cuda_error(cudaMemsetAsync(scratch, 0, 4, st))) return e;
    barrier_timeout_selftest_kernel<<<1, 32, 0, st>>>(scratch, status);
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_absmax_f32(const float* x, int64_t n, uint32_t* maxbits, void* stream) {
    NITI_REQUIRE(x && maxbits && n > 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = set_cuda_error(cudaMemsetAsync(maxbits, 0, 4, st))) return e;
    absmax_f32_kernel<<<blocks_for(n, 256, sm_count_simt() * 4), 256, 0, st>>>(x, n, maxbits);
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_quantize_input_with_max_f32(const float* x, int8_t* x8, int32_t* exp_out, const uint32_t* maxbits, int N,
                                                int C, int H, int W, void* stream) {
    NITI_REQUIRE(x && x8 && exp_out && maxbits && N > 0 && C > 0 && H > 0 && W > 0);
    const long long n = static_cast<long long>(N) * C * H * W;
    quantize_input_kernel<<<blocks_for(n, 256, sm_count_simt() * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, x8, exp_out, maxbits, N, C, H, W);
    return set_cuda_error(cudaGetLastError());
}

extern "C" int niti_quantize_input_f32(const float* x, int8_t* x8, int32_t* exp_out, uint32_t* scratch, int N, int C,
                                       int H, int W, void* stream) {
    NITI_REQUIRE(x && x8 && exp_out && scratch && N > 0 && C > 0 && H > 0 && W > 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long n = static_cast<long long>(N) * C * H * W;
    if (int e = set_cuda_error(cudaMemsetAsync(scratch, 0, 4, st))) return e;
    absmax_f32_kernel<<<blocks_for(n, 256, sm_count_simt() * 4), 256, 0, st>>>(x, n, scratch);
    quantize_input_kernel<<<blocks_for(n, 256, sm_count_simt() * 8), 256, 0, st>>>(x, x8, exp_out, scratch, N, C, H, W);
    return set_cuda_error(cudaGetLastError());
}
