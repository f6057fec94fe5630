// Scalar pieces of the integer cross-entropy error (the reference's ti_loss.py:6-36) shared by the
// stand-alone loss kernel and the fused classifier-head kernel.  2**s is a fixed sequence of IEEE double
// operations, so the result does not depend on a math library.
#pragma once
#include <cstdint>

namespace niti {

__device__ __forceinline__ double exp2_det(double s) {
    const double i = floor(s);
    const double t = __dmul_rn(s - i, 0.6931471805599453);
    // 1/j! for j = 17 .. 0
    const double c[18] = {1.0 / 355687428096000.0, 1.0 / 20922789888000.0, 1.0 / 1307674368000.0, 1.0 / 87178291200.0,
                          1.0 / 6227020800.0, 1.0 / 479001600.0, 1.0 / 39916800.0, 1.0 / 3628800.0, 1.0 / 362880.0,
                          1.0 / 40320.0, 1.0 / 5040.0, 1.0 / 720.0, 1.0 / 120.0, 1.0 / 24.0, 1.0 / 6.0, 1.0 / 2.0, 1.0, 1.0};
    double acc = c[0];
#pragma unroll
    for (int j = 1; j < 18; ++j) acc = __dadd_rn(__dmul_rn(acc, t), c[j]);
    return scalbn(acc, static_cast<int>(i));
}
__device__ __forceinline__ float pow2f_int(int e) {  // 2**e as float, e in [-126, 127]
    return __int_as_float((e + 127) << 23);
}

}  // namespace niti
