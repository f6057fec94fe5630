// C ABI: error reporting and the contraction entry points, which choose between the tensor-core
// (tcgen05) kernels and the CUDA-core kernels by shape.  Declarations: include/niti_b200.h.
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/niti_b200.h"
#include "internal.h"

namespace niti {

static thread_local char g_cuda_error[256] = "";

int set_cuda_error_text(const char* text) {
    std::snprintf(g_cuda_error, sizeof g_cuda_error, "%s", text);
    return NITI_ERR_CUDA;
}
int set_cuda_error(cudaError_t e) {
    if (e == cudaSuccess) return NITI_OK;
    std::snprintf(g_cuda_error, sizeof g_cuda_error, "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
    return NITI_ERR_CUDA;
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace niti

using namespace niti;

#define NITI_REQUIRE(cond) do { if (!(cond)) return NITI_ERR_BAD_ARG; } while (0)

extern "C" int niti_version(void) { return 100; }

extern "C" const char* niti_strerror(int code) {
    switch (code) {
        case NITI_OK: return "ok";
        case NITI_ERR_BAD_ARG: return "bad argument (null or misaligned pointer, non-positive size, unknown mode)";
        case NITI_ERR_UNSUPPORTED: return "shape or option not implemented by the kernels";
        case NITI_ERR_CUDA: return "CUDA call failed (see niti_last_cuda_error)";
        case NITI_ERR_SCRATCH: return "scratch buffer too small";
        default: return "unknown niti error code";
    }
}
extern "C" const char* niti_last_cuda_error(void) { return g_cuda_error; }

static int clear_word(uint32_t* p, cudaStream_t st) { return set_cuda_error(cudaMemsetAsync(p, 0, 4, st)); }

static bool conv_on_tensor_cores(int H, int W, int C, int R, int S, int pad) {
    // 128-byte reduction blocks over channels, "same" output size, at most 3 taps per filter row
    return C % 128 == 0 && R == 2 * pad + 1 && S == 2 * pad + 1 && S <= 3 && R <= 8 && H >= 1 && W >= 1;
}

extern "C" int niti_conv_fprop_i8(const int8_t* x, const int8_t* w, int32_t* y32, uint32_t* maxabs, int N, int H, int W,
                                  int C, int K, int R, int S, int pad, int stride, int32_t* status, void* stream) {
    NITI_REQUIRE(x && w && y32 && maxabs && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    if (stride != 1) return NITI_ERR_UNSUPPORTED;
    if (H + 2 * pad - R + 1 <= 0 || W + 2 * pad - S + 1 <= 0) return NITI_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = clear_word(maxabs, st)) return e;
    if (conv_on_tensor_cores(H, W, C, R, S, pad) && K % 4 == 0 && aligned16(x) && aligned16(w) && aligned16(y32))
        return umma_conv_fprop(x, w, y32, maxabs, N, H, W, C, K, R, S, pad, status, st);
    return simt_conv_fprop(x, w, y32, maxabs, N, H, W, C, K, R, S, pad, st);
}

extern "C" int niti_conv_dgrad_i8(const int8_t* err, const int8_t* wt, int32_t* e32, uint32_t* maxabs, int N, int H,
                                  int W, int C, int K, int R, int S, int pad, int32_t* status, void* stream) {
    // dX = err (x) wt with wt[c][r][s][k] = w[k][R-1-r][S-1-s][c]: a forward convolution whose
    // input channels are K and output channels are C, padded by R-1-pad
    NITI_REQUIRE(pad >= 0 && R - 1 - pad >= 0);
    return niti_conv_fprop_i8(err, wt, e32, maxabs, N, H, W, K, C, R, S, R - 1 - pad, 1, status, stream);
}

extern "C" size_t niti_conv_wgrad_scratch_bytes(int N, int H, int W, int C, int K, int R, int S) {
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || R <= 0 || S <= 0) return 0;
    const int pad = (R - 1) / 2;
    if (conv_on_tensor_cores(H, W, C, R, S, pad) && R == S) return umma_wgrad_scratch_bytes(N, H, W, C, K, R, S);
    return simt_wgrad_scratch_bytes(N, H, W, C, K, R, S);
}

extern "C" int niti_conv_wgrad_i8(const int8_t* x, const int8_t* err, int32_t* g32, uint32_t* maxabs, void* scratch,
                                  size_t scratch_bytes, int N, int H, int W, int C, int K, int R, int S, int pad,
                                  int32_t* status, void* stream) {
    NITI_REQUIRE(x && err && g32 && maxabs && scratch && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(aligned16(scratch) && aligned16(g32));
    if (H + 2 * pad - R + 1 != H || W + 2 * pad - S + 1 != W) {
        // the CUDA-core fallback handles other paddings; the gradient then has P != H
        if (H + 2 * pad - R + 1 <= 0 || W + 2 * pad - S + 1 <= 0) return NITI_ERR_BAD_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = clear_word(maxabs, st)) return e;
    const long long n = static_cast<long long>(K) * R * S * C;
    int splits = 0;
    int rc;
    const bool tc = conv_on_tensor_cores(H, W, C, R, S, pad) && R == S && K % 16 == 0 && aligned16(x) && aligned16(err);
    const size_t need = tc ? umma_wgrad_scratch_bytes(N, H, W, C, K, R, S) : simt_wgrad_scratch_bytes(N, H, W, C, K, R, S);
    if (scratch_bytes < need) return NITI_ERR_SCRATCH;
    if (tc) rc = umma_conv_wgrad_partials(x, err, static_cast<int32_t*>(scratch), &splits, N, H, W, C, K, R, S, pad, status, st);
    else    rc = simt_conv_wgrad_partials(x, err, static_cast<int32_t*>(scratch), &splits, N, H, W, C, K, R, S, pad, st);
    if (rc) return rc;
    return reduce_partials(static_cast<const int32_t*>(scratch), splits, n, g32, maxabs, st);
}

extern "C" int niti_gemm_i8(const int8_t* A, const int8_t* B, int32_t* C32, uint32_t* maxabs, int M, int N, int K,
                            int trans_a, int trans_b, int32_t* status, void* stream) {
    NITI_REQUIRE(A && B && C32 && maxabs && M > 0 && N > 0 && K > 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = clear_word(maxabs, st)) return e;
    const int pitch_a = trans_a ? M : K, pitch_b = trans_b ? K : N;
    const bool tc = pitch_a % 16 == 0 && pitch_b % 16 == 0 && M >= 64 && N >= 64 && K >= 64 && aligned16(A) && aligned16(B) &&
                    aligned16(C32);
    if (tc) return umma_gemm(A, B, C32, maxabs, M, N, K, trans_a, trans_b, status, st);
    return simt_gemm(A, B, C32, maxabs, M, N, K, trans_a, trans_b, st);
}
