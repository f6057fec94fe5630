// C ABI: error reporting and the contraction entry points, which choose between the tensor-core
// (tcgen05) kernels and the CUDA-core kernels by shape.  Declarations: include/niti_b200.h.
#include <cuda_runtime.h>
#include <atomic>
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
        case NITI_ERR_TOO_LARGE: return "problem needs more scratch than the library's built-in buffer holds (use the variant that takes caller scratch)";
        default: return "unknown niti error code";
    }
}
extern "C" const char* niti_last_cuda_error(void) { return g_cuda_error; }

// tuning switches (process-wide): see niti_set_option
static int g_opt_parking = 1;
static int g_opt_wgrad_reduce = 1;

extern "C" int niti_set_option(int option, int value) {
    if (option == NITI_OPT_ACCUMULATOR_PARKING) { const int old = g_opt_parking; g_opt_parking = value ? 1 : 0; return old; }
    if (option == NITI_OPT_CTA_PAIRS) { const int old = g_two_cta; g_two_cta = value & 3; return old; }
    if (option == NITI_OPT_COOPERATIVE_LAUNCH) { const int old = g_cooperative; g_cooperative = value ? 1 : 0; return old; }
    if (option == NITI_OPT_STAGE_CAP) { const int old = g_stage_cap; g_stage_cap = value < 0 ? 0 : value; return old; }
    if (option == NITI_OPT_WGRAD_TMA_REDUCE) { const int old = g_opt_wgrad_reduce; g_opt_wgrad_reduce = value ? 1 : 0; return old; }
    return NITI_ERR_BAD_ARG;
}

// ---- peer-visible arenas (CUDA IPC) for the data-parallel update kernel
static_assert(sizeof(cudaIpcMemHandle_t) <= NITI_PEER_HANDLE_BYTES, "handle size");
extern "C" int niti_peer_arena_create(size_t bytes, void** ptr, void* handle) {
    NITI_REQUIRE(bytes > 0 && ptr && handle);
    void* p = nullptr;
    if (int e = set_cuda_error(cudaMalloc(&p, bytes))) return e;
    if (int e = set_cuda_error(cudaMemset(p, 0, bytes))) { cudaFree(p); return e; }
    if (int e = set_cuda_error(cudaDeviceSynchronize())) { cudaFree(p); return e; }
    cudaIpcMemHandle_t h;
    if (int e = set_cuda_error(cudaIpcGetMemHandle(&h, p))) { cudaFree(p); return e; }
    memset(handle, 0, NITI_PEER_HANDLE_BYTES);
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return NITI_OK;
}
extern "C" int niti_peer_arena_open(const void* handle, void** ptr) {
    NITI_REQUIRE(handle && ptr);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (int e = set_cuda_error(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess))) return e;
    *ptr = p;
    return NITI_OK;
}
extern "C" int niti_peer_arena_close(void* ptr) {
    NITI_REQUIRE(ptr);
    return set_cuda_error(cudaIpcCloseMemHandle(ptr));
}
extern "C" int niti_peer_arena_destroy(void* ptr) {
    NITI_REQUIRE(ptr);
    return set_cuda_error(cudaFree(ptr));
}

static int clear_word(uint32_t* p, cudaStream_t st) { return set_cuda_error(cudaMemsetAsync(p, 0, 4, st)); }

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Which kernel family takes a convolution.  TC: implicit GEMM on the tensor cores (channels in
// 128-byte blocks; channel counts that are multiples of 16 ride on TMA zero fill).  THIN: R*S*C <= 32 (the 3-channel first layer): explicit patch
// matrix + tensor-core GEMM.  Otherwise the CUDA-core kernels.
enum ConvPath { CONV_SIMT = 0, CONV_TC = 1, CONV_THIN = 2 };

static bool same_padding(int R, int S, int pad) { return R == 2 * pad + 1 && S == 2 * pad + 1; }

static ConvPath fprop_path(int C, int K, int R, int S, int pad) {
    if (!same_padding(R, S, pad) || K % 4 != 0) return CONV_SIMT;
    if (R * S * C <= 32) return CONV_THIN;
    if (C % 16 == 0) return CONV_TC;
    return CONV_SIMT;
}
static ConvPath wgrad_path(int C, int K, int R, int S, int pad) {
    if (!same_padding(R, S, pad) || K % 16 != 0) return CONV_SIMT;
    if (R * S * C <= 32) return CONV_THIN;
    if (C % 16 == 0 && S <= 3) return CONV_TC;
    return CONV_SIMT;
}

extern "C" size_t niti_conv_fprop_scratch_bytes(int N, int H, int W, int C, int K, int R, int S) {
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || R <= 0 || S <= 0) return 0;
    if (fprop_path(C, K, R, S, (R - 1) / 2) != CONV_THIN) return 0;
    return align_up(static_cast<size_t>(N) * H * W * 32, 1024) + static_cast<size_t>(K) * 32;
}

extern "C" int niti_conv_fprop_i8(const int8_t* x, const int8_t* w, int32_t* y32, uint32_t* maxabs, void* scratch,
                                  size_t scratch_bytes, int N, int H, int W, int C, int K, int R, int S, int pad, int stride,
                                  int32_t* status, void* stream) {
    NITI_REQUIRE(x && w && y32 && maxabs && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    if (stride != 1) return NITI_ERR_UNSUPPORTED;
    if (H + 2 * pad - R + 1 <= 0 || W + 2 * pad - S + 1 <= 0) return NITI_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = clear_word(maxabs, st)) return e;
    ConvPath path = fprop_path(C, K, R, S, pad);
    if (!(aligned16(x) && aligned16(w) && aligned16(y32))) path = CONV_SIMT;
    if (path == CONV_TC) return umma_conv(x, w, y32, maxabs, N, H, W, C, K, R, S, pad, 0, nullptr, status, st);
    if (path == CONV_THIN) {
        const size_t m = static_cast<size_t>(N) * H * W;
        if (!scratch || !aligned16(scratch) || scratch_bytes < niti_conv_fprop_scratch_bytes(N, H, W, C, K, R, S)) return NITI_ERR_SCRATCH;
        int8_t* xcol = static_cast<int8_t*>(scratch);
        int8_t* wp = xcol + align_up(m * 32, 1024);
        if (int e = im2col32(x, xcol, N, H, W, C, R, S, pad, st, w, wp, K)) return e;
        return umma_gemm(xcol, wp, y32, maxabs, static_cast<int>(m), K, 32, 0, 1, 1, nullptr, status, st);
    }
    return simt_conv_fprop(x, w, y32, maxabs, N, H, W, C, K, R, S, pad, st);
}

// ---------------------------------------------------------------- int4 operands
extern "C" size_t niti_conv_fprop_i4_scratch_bytes(int N, int H, int W, int C2, int K, int R, int S) {
    if (N <= 0 || H <= 0 || W <= 0 || C2 <= 0 || K <= 0 || R <= 0 || S <= 0) return 0;
    const size_t xb = align_up(static_cast<size_t>(N) * H * W * C2 * 2, 1024), wb = align_up(static_cast<size_t>(K) * R * S * C2 * 2, 1024);
    return xb + wb + niti_conv_fprop_scratch_bytes(N, H, W, 2 * C2, K, R, S);
}

extern "C" int niti_conv_fprop_i4(const uint8_t* x4, const uint8_t* w4, int32_t* y32, uint32_t* maxabs, void* scratch,
                                  size_t scratch_bytes, int N, int H, int W, int C2, int K, int R, int S, int pad,
                                  int32_t* status, void* stream) {
    NITI_REQUIRE(x4 && w4 && y32 && maxabs && scratch && N > 0 && H > 0 && W > 0 && C2 > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(aligned16(scratch) && reinterpret_cast<uintptr_t>(x4) % 2 == 0);
    if (scratch_bytes < niti_conv_fprop_i4_scratch_bytes(N, H, W, C2, K, R, S)) return NITI_ERR_SCRATCH;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t xn = static_cast<size_t>(N) * H * W * C2, wn = static_cast<size_t>(K) * R * S * C2;
    int8_t* x8 = static_cast<int8_t*>(scratch);
    int8_t* w8 = x8 + align_up(2 * xn, 1024);
    int8_t* rest = w8 + align_up(2 * wn, 1024);
    if (int e = unpack_i4(x4, x8, static_cast<long long>(xn), st)) return e;
    if (int e = unpack_i4(w4, w8, static_cast<long long>(wn), st)) return e;
    const size_t used = static_cast<size_t>(rest - static_cast<int8_t*>(scratch));
    return niti_conv_fprop_i8(x8, w8, y32, maxabs, rest, scratch_bytes - used, N, H, W, 2 * C2, K, R, S, pad, 1, status, stream);
}

extern "C" int niti_conv_dgrad_i8(const int8_t* err, const int8_t* w, int32_t* e32, uint32_t* maxabs, int N, int H,
                                  int W, int C, int K, int R, int S, int pad, int32_t* status, void* stream) {
    NITI_REQUIRE(err && w && e32 && maxabs && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    if (!same_padding(R, S, pad)) return NITI_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = clear_word(maxabs, st)) return e;
    if (K % 16 == 0 && C % 16 == 0 && aligned16(err) && aligned16(w) && aligned16(e32))
        return umma_conv(err, w, e32, maxabs, N, H, W, C, K, R, S, pad, 1, nullptr, status, st);
    return simt_conv_dgrad(err, w, e32, maxabs, N, H, W, C, K, R, S, pad, st);
}

extern "C" size_t niti_conv_wgrad_scratch_bytes(int N, int H, int W, int C, int K, int R, int S) {
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || R <= 0 || S <= 0) return 0;
    const ConvPath path = wgrad_path(C, K, R, S, (R - 1) / 2);
    if (path == CONV_TC) return g_opt_wgrad_reduce ? 16 : umma_wgrad_scratch_bytes(N, H, W, C, K, R, S);
    if (path == CONV_THIN) {
        const size_t m = static_cast<size_t>(N) * H * W;
        return align_up(m * 32, 1024) + static_cast<size_t>(umma_gemm_splits(K, 32, static_cast<int>(m))) * K * 32 * 4;
    }
    return 16;
}

extern "C" int niti_conv_wgrad_i8(const int8_t* x, const int8_t* err, int32_t* g32, uint32_t* maxabs, void* scratch,
                                  size_t scratch_bytes, int N, int H, int W, int C, int K, int R, int S, int pad,
                                  int32_t* status, void* stream) {
    NITI_REQUIRE(x && err && g32 && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(aligned16(g32));
    if (H + 2 * pad - R + 1 <= 0 || W + 2 * pad - S + 1 <= 0) return NITI_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (maxabs != nullptr)  // null: the caller finds max|g32| later (niti_update_multi_i8 does)
        if (int e = clear_word(maxabs, st)) return e;
    ConvPath path = wgrad_path(C, K, R, S, pad);
    if (!(aligned16(x) && aligned16(err))) path = CONV_SIMT;
    if (path == CONV_SIMT) return simt_conv_wgrad(x, err, g32, maxabs, N, H, W, C, K, R, S, pad, st);
    if (!scratch || !aligned16(scratch) || scratch_bytes < niti_conv_wgrad_scratch_bytes(N, H, W, C, K, R, S)) return NITI_ERR_SCRATCH;
    const long long n = static_cast<long long>(K) * R * S * C;
    if (path == CONV_TC) {
        int splits = 0;
        if (g_opt_wgrad_reduce) {
            // zero the gradient, let every thread block add its tiles into it at the L2 (TMA reductions), then one
            // pass for max|g|: no partial sums in memory, no folding kernel
            if (int e = set_cuda_error(cudaMemsetAsync(g32, 0, static_cast<size_t>(n) * 4, st))) return e;
            if (int rc = umma_conv_wgrad_partials(x, err, g32, &splits, 0, N, H, W, C, K, R, S, pad, status, st, 1)) return rc;
            return maxabs != nullptr ? absmax_i32(g32, n, maxabs, st) : NITI_OK;
        }
        if (int rc = umma_conv_wgrad_partials(x, err, static_cast<int32_t*>(scratch), &splits, 0, N, H, W, C, K, R, S, pad, status, st)) return rc;
        return reduce_partials(static_cast<const int32_t*>(scratch), splits, n, g32, maxabs, st);
    }
    // thin: g[k][0..R*S*C) = sum_pixels err[pixel][k] * xcol[pixel][0..32)  (split-K GEMM, then fold and drop the padding)
    const size_t m = static_cast<size_t>(N) * H * W;
    int8_t* xcol = static_cast<int8_t*>(scratch);
    int32_t* partial = reinterpret_cast<int32_t*>(xcol + align_up(m * 32, 1024));
    const int splits = umma_gemm_splits(K, 32, static_cast<int>(m));
    if (int e = im2col32(x, xcol, N, H, W, C, R, S, pad, st)) return e;
    if (int e = umma_gemm(err, xcol, partial, nullptr, K, 32, static_cast<int>(m), 1, 0, splits, nullptr, status, st)) return e;
    return reduce_rows32(partial, splits, K, R * S * C, g32, maxabs, st);
}

extern "C" size_t niti_conv_wgrad_patches_scratch_bytes(int N, int H, int W, int C, int K, int R, int S) {
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || R <= 0 || S <= 0) return 0;
    if (wgrad_path(C, K, R, S, (R - 1) / 2) != CONV_THIN) return 0;
    return static_cast<size_t>(umma_gemm_splits(K, 32, static_cast<int>(static_cast<size_t>(N) * H * W))) * K * 32 * 4;
}

extern "C" int niti_conv_wgrad_patches_i8(const int8_t* patches, const int8_t* err, int32_t* g32, uint32_t* maxabs, void* scratch,
                                          size_t scratch_bytes, int N, int H, int W, int C, int K, int R, int S,
                                          int32_t* status, void* stream) {
    NITI_REQUIRE(patches && err && g32 && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0);
    NITI_REQUIRE(aligned16(patches) && aligned16(err) && aligned16(g32));
    if (wgrad_path(C, K, R, S, (R - 1) / 2) != CONV_THIN) return NITI_ERR_UNSUPPORTED;
    if (!scratch || !aligned16(scratch) || scratch_bytes < niti_conv_wgrad_patches_scratch_bytes(N, H, W, C, K, R, S)) return NITI_ERR_SCRATCH;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (maxabs != nullptr)
        if (int e = clear_word(maxabs, st)) return e;
    const size_t m = static_cast<size_t>(N) * H * W;
    const int splits = umma_gemm_splits(K, 32, static_cast<int>(m));
    int32_t* partial = static_cast<int32_t*>(scratch);
    if (int e = umma_gemm(err, patches, partial, nullptr, K, 32, static_cast<int>(m), 1, 0, splits, nullptr, status, st)) return e;
    return reduce_rows32(partial, splits, K, R * S * C, g32, maxabs, st);
}

extern "C" int niti_conv_wgrad_accumulate_supported(int C, int K, int R, int S, int pad) {
    return wgrad_path(C, K, R, S, pad) == CONV_TC ? 1 : 0;
}

extern "C" int niti_conv_wgrad_accumulate_i8(const int8_t* x, const int8_t* err, int32_t* g32, int N, int H, int W, int C, int K,
                                             int R, int S, int pad, int32_t* status, void* stream) {
    NITI_REQUIRE(x && err && g32 && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(aligned16(g32) && aligned16(x) && aligned16(err));
    if (H + 2 * pad - R + 1 <= 0 || W + 2 * pad - S + 1 <= 0) return NITI_ERR_BAD_ARG;
    if (wgrad_path(C, K, R, S, pad) != CONV_TC) return NITI_ERR_UNSUPPORTED;
    int splits = 0;
    return umma_conv_wgrad_partials(x, err, g32, &splits, 0, N, H, W, C, K, R, S, pad, status, static_cast<cudaStream_t>(stream), 1);
}

extern "C" int niti_conv_wgrad_accumulate_multi_max(void) { return umma_wgrad_multi_max(); }

extern "C" int niti_conv_wgrad_accumulate_multi_i8(const niti_wgrad_item* items, int count, int32_t* status, void* stream) {
    NITI_REQUIRE(items && count >= 1 && count <= umma_wgrad_multi_max());
    WgradJob jobs[8];
    for (int i = 0; i < count; ++i) {
        const niti_wgrad_item& it = items[i];
        NITI_REQUIRE(it.x && it.err && it.g32 && it.N > 0 && it.H > 0 && it.W > 0 && it.C > 0 && it.K > 0 && it.R > 0 && it.S > 0 && it.pad >= 0);
        NITI_REQUIRE(aligned16(it.g32) && aligned16(it.x) && aligned16(it.err));
        if (it.H + 2 * it.pad - it.R + 1 <= 0 || it.W + 2 * it.pad - it.S + 1 <= 0) return NITI_ERR_BAD_ARG;
        if (wgrad_path(it.C, it.K, it.R, it.S, it.pad) != CONV_TC) return NITI_ERR_UNSUPPORTED;
        jobs[i] = WgradJob{it.x, it.err, it.g32, it.N, it.H, it.W, it.C, it.K, it.R, it.S, it.pad};
    }
    return umma_conv_wgrad_multi(jobs, count, status, static_cast<cudaStream_t>(stream));
}

extern "C" int niti_gemm_i8(const int8_t* A, const int8_t* B, int32_t* C32, uint32_t* maxabs, int M, int N, int K,
                            int trans_a, int trans_b, int32_t* status, void* stream) {
    NITI_REQUIRE(A && B && C32 && maxabs && M > 0 && N > 0 && K > 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int e = clear_word(maxabs, st)) return e;
    const int pitch_a = trans_a ? M : K, pitch_b = trans_b ? K : N;
    const bool tc = pitch_a % 16 == 0 && pitch_b % 16 == 0 && N % 4 == 0 && M >= 64 && N >= 32 && K >= 32 && aligned16(A) &&
                    aligned16(B) && aligned16(C32);
    if (tc) return umma_gemm(A, B, C32, maxabs, M, N, K, trans_a, trans_b, 1, nullptr, status, st);
    return simt_gemm(A, B, C32, maxabs, M, N, K, trans_a, trans_b, st);
}

// ---------------------------------------------------------------- contraction + requantisation in one pass
static int fused_conv(const int8_t* in, const int8_t* w, int8_t* out8, int32_t* state, void* scratch, size_t scratch_bytes,
                      int N, int H, int W, int C, int K, int R, int S, int pad, int flip, int kind, int round_mode,
                      const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset, int relu, const int32_t* exp_a,
                      const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out, int32_t* status, cudaStream_t st,
                      const int8_t* relu_mask = nullptr, int8_t* pool_out = nullptr, void* side = nullptr) {
    FusedArgs f{state, 0, 0, round_mode, relu, reinterpret_cast<const unsigned long long*>(seed), rng_stream, rng_offset,
                kind, 7, exp_a, exp_b, exp_out, shift_out, relu_mask, pool_out, side};
    const bool thin = !flip && fprop_path(C, K, R, S, pad) == CONV_THIN;
    const size_t m = static_cast<size_t>(N) * H * W;
    int8_t* xcol = static_cast<int8_t*>(scratch);
    int8_t* wp = thin ? xcol + align_up(m * 32, 1024) : nullptr;
    if (thin) {
        if (!scratch || !aligned16(scratch) || scratch_bytes < niti_conv_fprop_scratch_bytes(N, H, W, C, K, R, S)) return NITI_ERR_SCRATCH;
        if (int e = im2col32(in, xcol, N, H, W, C, R, S, pad, st, w, wp, K)) return e;
    }
    if (pool_out != nullptr && !(g_opt_parking && !thin && !flip && umma_conv_pool_fusable(N, H, W, K))) return NITI_ERR_UNSUPPORTED;
    // Few enough output tiles for every accumulator to stay in tensor memory: one exact launch.
    if (g_opt_parking && !thin && umma_conv_fits_parked(N, H, W, flip ? C : K, flip)) {
        f.parked = 1;
        return umma_conv(in, w, out8, nullptr, N, H, W, C, K, R, S, pad, flip, &f, status, st);
    }
    // first launch: narrow with the predicted shift, reduce max|acc|, verify; second launch: redo if it was wrong
    for (int pass = 0; pass < 2; ++pass) {
        f.only_if_redo = pass;
        int rc = thin ? umma_gemm(xcol, wp, out8, nullptr, static_cast<int>(m), K, 32, 0, 1, 1, &f, status, st)
                      : umma_conv(in, w, out8, nullptr, N, H, W, C, K, R, S, pad, flip, &f, status, st);
        if (rc) return rc;
    }
    return NITI_OK;
}

extern "C" int niti_conv_fprop_requant_supported(int C, int K, int R, int S, int pad) {
    const ConvPath p = fprop_path(C, K, R, S, pad);
    return (p == CONV_TC || p == CONV_THIN) && K % 16 == 0;
}
extern "C" int niti_conv_dgrad_requant_supported(int C, int K, int R, int S, int pad) {
    return same_padding(R, S, pad) && K % 16 == 0 && C % 16 == 0;
}

extern "C" int niti_conv_fprop_requant_i8(const int8_t* x, const int8_t* w, int8_t* y8, int32_t* state, void* scratch,
                                          size_t scratch_bytes, int N, int H, int W, int C, int K, int R, int S, int pad,
                                          int round_mode, const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset,
                                          int relu, const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out,
                                          int32_t* shift_out, int32_t* status, void* stream) {
    NITI_REQUIRE(x && w && y8 && state && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(round_mode >= 0 && round_mode <= 2 && (seed || round_mode != NITI_ROUND_STOCHASTIC));
    NITI_REQUIRE(aligned16(x) && aligned16(w) && aligned16(y8) && reinterpret_cast<uintptr_t>(state) % 8 == 0);
    if (!niti_conv_fprop_requant_supported(C, K, R, S, pad)) return NITI_ERR_UNSUPPORTED;
    return fused_conv(x, w, y8, state, scratch, scratch_bytes, N, H, W, C, K, R, S, pad, 0, NITI_CALC_ACT, round_mode, seed,
                      rng_stream, rng_offset, relu, exp_a, exp_b, exp_out, shift_out, status, static_cast<cudaStream_t>(stream));
}

extern "C" int niti_conv_fprop_requant_pool_supported(int N, int H, int W, int C, int K, int R, int S, int pad) {
    if (N <= 0 || H <= 0 || W <= 0 || !niti_conv_fprop_requant_supported(C, K, R, S, pad)) return 0;
    return g_opt_parking && fprop_path(C, K, R, S, pad) == CONV_TC && umma_conv_pool_fusable(N, H, W, K) ? 1 : 0;
}

extern "C" int niti_conv_fprop_requant_pool_i8(const int8_t* x, const int8_t* w, int8_t* y8, int8_t* y8_pooled, int32_t* state, int N,
                                               int H, int W, int C, int K, int R, int S, int pad, int round_mode,
                                               const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset, int relu,
                                               const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                                               int32_t* status, void* stream) {
    NITI_REQUIRE(x && w && y8 && y8_pooled && state && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(round_mode >= 0 && round_mode <= 2 && (seed || round_mode != NITI_ROUND_STOCHASTIC));
    NITI_REQUIRE(aligned16(x) && aligned16(w) && aligned16(y8) && aligned16(y8_pooled) && reinterpret_cast<uintptr_t>(state) % 8 == 0);
    if (!niti_conv_fprop_requant_pool_supported(N, H, W, C, K, R, S, pad)) return NITI_ERR_UNSUPPORTED;
    return fused_conv(x, w, y8, state, nullptr, 0, N, H, W, C, K, R, S, pad, 0, NITI_CALC_ACT, round_mode, seed, rng_stream,
                      rng_offset, relu, exp_a, exp_b, exp_out, shift_out, status, static_cast<cudaStream_t>(stream), nullptr, y8_pooled);
}

extern "C" int niti_conv_dgrad_requant_i8(const int8_t* err, const int8_t* w, int8_t* e8, int32_t* state, int N, int H, int W,
                                          int C, int K, int R, int S, int pad, int round_mode, const uint64_t* seed,
                                          uint32_t rng_stream, uint64_t rng_offset, const int32_t* exp_a, const int32_t* exp_b,
                                          int32_t* exp_out, int32_t* shift_out, const int8_t* relu_mask, int32_t* status,
                                          void* stream) {
    NITI_REQUIRE(err && w && e8 && state && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(round_mode >= 0 && round_mode <= 2 && (seed || round_mode != NITI_ROUND_STOCHASTIC));
    NITI_REQUIRE(aligned16(err) && aligned16(w) && aligned16(e8) && aligned16(relu_mask) && reinterpret_cast<uintptr_t>(state) % 8 == 0);
    if (!niti_conv_dgrad_requant_supported(C, K, R, S, pad)) return NITI_ERR_UNSUPPORTED;
    return fused_conv(err, w, e8, state, nullptr, 0, N, H, W, C, K, R, S, pad, 1, NITI_CALC_ERR, round_mode, seed, rng_stream,
                      rng_offset, 0, exp_a, exp_b, exp_out, shift_out, status, static_cast<cudaStream_t>(stream), relu_mask);
}

extern "C" size_t niti_conv_dgrad_requant_side_bytes(int N, int H, int W, int C, int K, int R, int S, int pad) {
    if (N <= 0 || H <= 0 || W <= 0 || !niti_conv_dgrad_requant_supported(C, K, R, S, pad)) return 0;
    if (g_opt_parking && umma_conv_fits_parked(N, H, W, C, 1)) return 0;  // exact in one launch: nothing to predict
    return static_cast<size_t>(N) * H * W * C / 4;
}

extern "C" int niti_conv_dgrad_requant_side_i8(const int8_t* err, const int8_t* w, int8_t* e8, int32_t* state, void* side,
                                               size_t side_bytes, int N, int H, int W, int C, int K, int R, int S, int pad,
                                               int round_mode, const uint64_t* seed, uint32_t rng_stream, uint64_t rng_offset,
                                               const int32_t* exp_a, const int32_t* exp_b, int32_t* exp_out, int32_t* shift_out,
                                               const int8_t* relu_mask, int32_t* status, void* stream) {
    NITI_REQUIRE(err && w && e8 && state && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(round_mode >= 0 && round_mode <= 2 && (seed || round_mode != NITI_ROUND_STOCHASTIC));
    NITI_REQUIRE(aligned16(err) && aligned16(w) && aligned16(e8) && aligned16(relu_mask) && reinterpret_cast<uintptr_t>(state) % 8 == 0);
    if (!niti_conv_dgrad_requant_supported(C, K, R, S, pad)) return NITI_ERR_UNSUPPORTED;
    if (side != nullptr && (!aligned16(side) || side_bytes < static_cast<size_t>(N) * H * W * C / 4)) return NITI_ERR_SCRATCH;
    return fused_conv(err, w, e8, state, nullptr, 0, N, H, W, C, K, R, S, pad, 1, NITI_CALC_ERR, round_mode, seed, rng_stream,
                      rng_offset, 0, exp_a, exp_b, exp_out, shift_out, status, static_cast<cudaStream_t>(stream), relu_mask,
                      nullptr, side);
}

// ---------------------------------------------------------------- weight gradient without caller scratch
// Scratch for callers that have no way to allocate device memory: a fixed buffer inside the library
// image.  Every GPU context that loads the library carries these bytes until it is torn down.
static __device__ __align__(256) unsigned char g_builtin_scratch[NITI_BUILTIN_SCRATCH_BYTES];

// `g_builtin_scratch` names the buffer only in device code.  Host code must ask the runtime for the
// device address (per device: each device has its own copy of the array); it is looked up the first
// time a device uses the entry point, with that device current, and remembered.  The table is keyed by
// the CURRENT device (the stream passed in must belong to it); its slots are atomics because two host
// threads may make their first call on a device at the same time (both would store the same address).
// After cudaDeviceReset the remembered address is stale: a process that resets a device must not call
// the entry point on it again.
static std::atomic<void*> g_builtin_scratch_addr[64];

static int builtin_scratch(void** out) {
    int dev = -1;
    if (int e = set_cuda_error(cudaGetDevice(&dev))) return e;
    if (dev < 0 || dev >= 64) return set_cuda_error_text("device ordinal outside the range the built-in scratch table covers");
    void* p = g_builtin_scratch_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        if (int e = set_cuda_error(cudaGetSymbolAddress(&p, g_builtin_scratch))) return e;
        g_builtin_scratch_addr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return NITI_OK;
}

extern "C" int niti_conv_wgrad_builtin_scratch_i8(const int8_t* x, const int8_t* err, int32_t* g32, uint32_t* maxabs, int N,
                                                  int H, int W, int C, int K, int R, int S, int pad, int32_t* status,
                                                  void* stream) {
    NITI_REQUIRE(x && err && g32 && N > 0 && H > 0 && W > 0 && C > 0 && K > 0 && R > 0 && S > 0 && pad >= 0);
    NITI_REQUIRE(aligned16(g32));
    if (H + 2 * pad - R + 1 <= 0 || W + 2 * pad - S + 1 <= 0) return NITI_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ConvPath path = wgrad_path(C, K, R, S, pad);
    if (!(aligned16(x) && aligned16(err))) path = CONV_SIMT;
    const size_t cap = NITI_BUILTIN_SCRATCH_BYTES;
    const long long n = static_cast<long long>(K) * R * S * C;
    // size check first: nothing is launched for a problem that does not fit
    int max_splits = 0;
    const size_t m = static_cast<size_t>(N) * H * W;
    if (path == CONV_TC) {
        const size_t per_split = static_cast<size_t>(n) * 4;
        if (per_split > cap) return NITI_ERR_TOO_LARGE;
        max_splits = static_cast<int>(cap / per_split);
    } else if (path == CONV_THIN) {
        const size_t fixed = align_up(m * 32, 1024), per_split = static_cast<size_t>(K) * 32 * 4;
        if (fixed + per_split > cap) return NITI_ERR_TOO_LARGE;
        max_splits = static_cast<int>((cap - fixed) / per_split);
    }
    if (maxabs != nullptr)  // null, as in niti_conv_wgrad_i8: the caller finds max|g32| later
        if (int e = clear_word(maxabs, st)) return e;
    if (path == CONV_SIMT) return simt_conv_wgrad(x, err, g32, maxabs, N, H, W, C, K, R, S, pad, st);
    void* scratch = nullptr;
    if (int e = builtin_scratch(&scratch)) return e;
    // Nothing in the buffer has to start at zero: every partial sum that is read back below is first
    // written by this call (the kernels cover [splits][K][R][S][C], resp. the patch matrix, completely).
    if (path == CONV_TC) {
        int splits = 0;
        if (int rc = umma_conv_wgrad_partials(x, err, static_cast<int32_t*>(scratch), &splits, max_splits, N, H, W, C, K, R, S,
                                              pad, status, st)) return rc;
        return reduce_partials(static_cast<const int32_t*>(scratch), splits, n, g32, maxabs, st);
    }
    int8_t* xcol = static_cast<int8_t*>(scratch);
    int32_t* partial = reinterpret_cast<int32_t*>(xcol + align_up(m * 32, 1024));
    int splits = umma_gemm_splits(K, 32, static_cast<int>(m));
    if (splits > max_splits) splits = max_splits;
    if (int e = im2col32(x, xcol, N, H, W, C, R, S, pad, st)) return e;
    if (int e = umma_gemm(err, xcol, partial, nullptr, K, 32, static_cast<int>(m), 1, 0, splits, nullptr, status, st)) return e;
    return reduce_rows32(partial, splits, K, R * S * C, g32, maxabs, st);
}
