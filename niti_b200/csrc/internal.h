// Launchers shared between the translation units of the library (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace niti {

// error plumbing: both return NITI_ERR_CUDA (or 0 for cudaSuccess) and remember the text
int set_cuda_error(cudaError_t e);
int set_cuda_error_text(const char* text);

// Requantisation fused into a contraction's epilogue: the kernel narrows with the shift it finds in
// state[0] and its last CTA verifies that shift; `only_if_redo` launches are no-ops unless state[2] is set.
struct FusedArgs {
    int32_t* state;        // {shift, max|acc|, redo flag, redo count, exit ticket, barrier arrivals, -, -}
    int only_if_redo;
    int parked;            // 1: accumulator-parking kernel (exact in one launch; needs umma_conv_fits_parked)
    int mode, relu;
    const unsigned long long* seed;
    unsigned rng_stream;
    unsigned long long rng_offset;
    int kind, target_bits;
    const int32_t* exp_a; const int32_t* exp_b; int32_t* exp_out; int32_t* shift_out;
    const int8_t* relu_mask;  // optional, same shape as the output: zero the output where this tensor is <= 0
    int8_t* pool_out;         // optional (forward, parked kernel): 2x2 / stride-2 max-pooled copy of the output
    void* side;               // optional (streaming kernel, round-to-nearest, no ReLU): outputs / 4 bytes of side codes
};

extern int g_two_cta;    // CTA pairs (cta_group::2) where the shape allows: bit 0 for GEMMs, bit 1 for convolutions
extern int g_cooperative;  // 1: cooperative launches for the kernels with a grid barrier (see umma_kernels.cu)
extern int g_stage_cap;  // experiments: cap on the shared-memory stages the GEMM / conv kernels use (0 = all)

// tensor-core (tcgen05) paths, umma_kernels.cu; `out` is int32 (fused == null) or int8
int umma_gemm_splits(int M, int N, int K);
int umma_gemm(const int8_t* A, const int8_t* B, void* out, unsigned* maxabs, int M, int N, int K, int trans_a,
              int trans_b, int splits, const FusedArgs* fused, int32_t* status, cudaStream_t st);
int umma_conv(const int8_t* x, const int8_t* w, void* out, unsigned* maxabs, int Nimg, int H, int W, int C, int K,
              int R, int S, int pad, int flip, const FusedArgs* fused, int32_t* status, cudaStream_t st);
bool umma_conv_fits_parked(int Nimg, int H, int W, int outc, int flip);
bool umma_conv_pool_fusable(int Nimg, int H, int W, int outc);  // the fused forward kernel can also emit the 2x2-pooled output
size_t umma_wgrad_scratch_bytes(int Nimg, int H, int W, int C, int K, int R, int S);
// max_splits > 0 caps the number of pixel-range splits (and with it the size of `partial`)
// direct == 1: `partial` is the zeroed gradient and the CTAs add into it (TMA reduction) instead of storing partials
int umma_conv_wgrad_partials(const int8_t* x, const int8_t* err, int32_t* partial, int* splits_out, int max_splits,
                             int Nimg, int H, int W, int C, int K, int R, int S, int pad, int32_t* status, cudaStream_t st,
                             int direct = 0);
// several layers' weight gradients, each ADDED into its g32, in one launch (umma_kernels.cu)
struct WgradJob { const int8_t* x; const int8_t* err; int32_t* g32; int N, H, W, C, K, R, S, pad; };
int umma_wgrad_multi_max();
int umma_conv_wgrad_multi(const WgradJob* jobs, int count, int32_t* status, cudaStream_t st);
int absmax_i32(const int32_t* acc, long long n, unsigned* maxabs, cudaStream_t st);  // reduces into *maxabs (not cleared)

// CUDA-core paths, simt_kernels.cu
int simt_conv_fprop(const int8_t* x, const int8_t* w, int32_t* y32, unsigned* maxabs, int Nimg, int H, int W, int C,
                    int K, int R, int S, int pad, cudaStream_t st);
int simt_conv_dgrad(const int8_t* err, const int8_t* w, int32_t* e32, unsigned* maxabs, int Nimg, int H, int W, int C,
                    int K, int R, int S, int pad, cudaStream_t st);
int simt_conv_wgrad(const int8_t* x, const int8_t* err, int32_t* g32, unsigned* maxabs, int Nimg, int H, int W, int C,
                    int K, int R, int S, int pad, cudaStream_t st);
int simt_gemm(const int8_t* A, const int8_t* B, int32_t* C32, unsigned* maxabs, int M, int N, int K, int trans_a,
              int trans_b, cudaStream_t st);
int reduce_partials(const int32_t* partial, int splits, long long n, int32_t* out, unsigned* maxabs, cudaStream_t st);
int reduce_rows32(const int32_t* partial, int splits, int rows, int cols_out, int32_t* out, unsigned* maxabs, cudaStream_t st);
// w / wp / K: optionally the layer's filters w[K][R*S*C] are padded to wp[K][32] by the same launch
int im2col32(const int8_t* x, int8_t* xcol, int Nimg, int H, int W, int C, int R, int S, int pad, cudaStream_t st,
             const int8_t* w = nullptr, int8_t* wp = nullptr, int K = 0);
int unpack_i4(const uint8_t* in, int8_t* out, long long nbytes, cudaStream_t st);  // two int4 per byte (low nibble first) -> int8

}  // namespace niti
