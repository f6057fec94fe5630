// NITI's int32 -> int8 requantisation and the counter-based random bits behind its
// stochastic rounding, as device functions shared by every kernel that narrows.
//
// Follows the reference's ti_torch.py: RangeEstimate :366-377 (bit-width from max|x|),
// act_calc/err_calc/grad_calc :103-147 (shift = bit-width - target), RoundShift :23-31,
// StoShift :33-46, PstoShift :48-69, int8_clip :71-72, with `//` truncating toward zero
// as in the torch release the reference was written for.
#pragma once
#include <cstdint>

namespace niti {

enum RoundMode : int { ROUND_NEAREST = 0, ROUND_STOCHASTIC = 1, ROUND_PSEUDO_STOCHASTIC = 2 };
enum CalcKind : int { CALC_ACT = 0, CALC_ERR = 1, CALC_GRAD = 2 };

// ---- Philox4x32-10 (Salmon et al., SC'11), keyed by (seed, stream), counter = element block.
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
// Four words for elements 4*block .. 4*block+3 of `stream`.
__device__ __forceinline__ void random_block(uint64_t seed, uint32_t stream, uint64_t block, uint32_t (&out)[4]) {
    philox4x32_10(static_cast<uint32_t>(block), static_cast<uint32_t>(block >> 32), stream, 0u,
                  static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), out);
}
__device__ __forceinline__ uint32_t random_word(uint64_t seed, uint32_t stream, uint64_t idx) {
    uint32_t w[4];
    random_block(seed, stream, idx >> 2, w);
    return w[idx & 3];
}

// ---- bit-width and shift selection
__host__ __device__ __forceinline__ int bitwidth_of_max(uint32_t m) {
    if (m == 0) return 0;
#ifdef __CUDA_ARCH__
    return 32 - __clz(static_cast<int>(m - 1));
#else
    int b = 0; uint32_t v = m - 1; while (v) { ++b; v >>= 1; } return b;
#endif
}
// shift (>= 0) applied to a tensor whose max|x| is `m`; `zero_out` is grad_calc's all-zero case.
__host__ __device__ __forceinline__ int shift_for(uint32_t m, int kind, int target_bits, bool* zero_out) {
    int b = bitwidth_of_max(m);
    *zero_out = (kind == CALC_GRAD) && (b == 0);
    int s = b - target_bits;
    return s > 0 ? s : 0;
}

__device__ __forceinline__ int clamp127(int v) { return max(-127, min(127, v)); }

// One element: shift == 0 wraps like `.type(torch.int8)`; shift > 0 rounds then clamps to +-127.
__device__ __forceinline__ int8_t narrow(int x, int shift, int mode, uint32_t rnd) {
    if (shift == 0) return static_cast<int8_t>(x);
    uint32_t a = static_cast<uint32_t>(x < 0 ? -x : x);
    uint32_t q = a >> shift;
    uint32_t lo = a & ((1u << shift) - 1u);
    uint32_t up;
    if (mode == ROUND_NEAREST) {
        up = lo >> (shift - 1);
    } else if (mode == ROUND_STOCHASTIC) {
        up = lo > (rnd & ((1u << shift) - 1u));
    } else {
        int h = shift >> 1;
        uint32_t qp = lo >> h;
        uint32_t pr = lo & ((1u << h) - 1u);
        if (shift & 1) pr <<= 1;
        up = qp > pr;
    }
    int v = static_cast<int>(q + up);
    return static_cast<int8_t>(clamp127(x < 0 ? -v : v));
}

}  // namespace niti
