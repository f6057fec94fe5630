// int8 x int8 -> int32 contractions on the 5th-generation tensor cores (sm_100a):
// GEMM, implicit-GEMM convolution forward / error-backward, and convolution weight gradient.
//
// Common structure (one CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor into 128-byte-swizzled shared-memory stages
//   warp 1      allocates tensor memory, issues tcgen05.mma.kind::i8 (one lane), frees TMEM
//   warps 2..5  epilogue: tcgen05.ld the int32 accumulators, reduce max|acc|, store
// Stages hand over through mbarriers (TMA complete_tx -> MMA, tcgen05.commit -> producer);
// accumulators are double-buffered in TMEM so the epilogue of one tile overlaps the main loop
// of the next.  All waits are bounded (ptx.cuh).
//
// Operand layouts in shared memory.  Every operand tile is rows of 128 bytes, 8-row groups of
// 1024 bytes, 128-byte swizzle -- exactly what a TMA box with a 128-byte inner extent writes.
//   K-major  (reduction index contiguous in memory): row = M/N index, 128 bytes = 128 reduction
//            elements; one MMA (K = 32) advances the descriptor by 32 bytes.
//   MN-major (M/N index contiguous, e.g. [pixels][channels] read as channels x pixels): row =
//            reduction index, 128 bytes = 128 M/N elements; one MMA advances by 32 rows = 4096 B;
//            a second 128-wide panel sits `rows * 128` bytes further (leading byte offset).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/niti_b200.h"
#include "internal.h"
#include "ptx.cuh"
#include "requant.cuh"
#include "grid_barrier.cuh"

namespace niti {
#ifdef NITI_PARKED_TIMING
__device__ unsigned long long g_dbg_stamps[32];
#define PARK_STAMP(i) do { if (blockIdx.x == 0) g_dbg_stamps[i] = global_timer_ns(); } while (0)
#define DBG_CLK(v) const long long v = clock64()
#define DBG_DECL long long dbg_acc[4] = {0, 0, 0, 0}
#define DBG_ACC(i, d) dbg_acc[(i) & 3] += (d)
#define DBG_OUT(base) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) for (int q_ = 0; q_ < 4; ++q_) g_dbg_stamps[(base) + q_] = dbg_acc[q_]; } while (0)
#else
#define DBG_CLK(v) do { } while (0)
#define DBG_DECL do { } while (0)
#define DBG_ACC(i, d) do { } while (0)
#define DBG_OUT(base) do { } while (0)
#define PARK_STAMP(i) do { } while (0)
#endif

// Pin a value in a register: kernel parameters live in the constant bank, and under register pressure the compiler
// re-reads them at every use; in the producer / MMA loops each such load sits on one warp's serial critical path.
__device__ __forceinline__ int keep_reg(int v) { asm volatile("" : "+r"(v)); return v; }

constexpr int BLOCK_M = 128;
constexpr int ROW_BYTES = 128;               // bytes per shared-memory row of an operand tile
constexpr int PANEL_BYTES = 128 * ROW_BYTES; // one 128-row operand panel
constexpr int UMMA_THREADS = 192;
constexpr uint32_t SWIZZLE_128B_CODE = 2;
constexpr int EPI_CHUNK_BYTES = 128 * 32 * 4;  // 128 rows x 32 int32 columns, one TMA store box
constexpr int EPI_BARRIER = 1;                 // named barrier of the 128 epilogue threads

// Epilogue staging: each thread owns one accumulator row of 32 int32 (128 bytes) and writes it as
// eight 16-byte chunks at the 128-byte-swizzled position the TMA store expects (chunk ^ row%8);
// that placement is also free of shared-memory bank conflicts.
__device__ __forceinline__ void stage_row(uint32_t buf, int row, const uint32_t (&v)[32]) {
    const uint32_t base = buf + static_cast<uint32_t>(row) * 128u;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        st_shared_v4(base + (static_cast<uint32_t>(j ^ (row & 7)) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
}

// ------------------------------------------------------------------------------------------------
// GEMM / convolution forward / error-backward
// ------------------------------------------------------------------------------------------------
// Division of a non-negative int by a divisor fixed at launch: q = (umulhi(mul, n) + n) >> shift with
// shift = ceil(log2 d) and mul = floor(2^32 (2^shift - d) / d) + 1, exact for 0 <= n < 2^31.  The tile loops turn a
// tile number into coordinates once per tile; eight hardware-less 32-bit divisions there were a quarter of an epilogue.
struct FastDiv { unsigned mul, shift; int d; };
static FastDiv make_fastdiv(int d) {
    FastDiv f{1u, 0u, d < 1 ? 1 : d};
    while ((1ull << f.shift) < static_cast<unsigned long long>(f.d)) ++f.shift;
    f.mul = static_cast<unsigned>(((1ull << 32) * ((1ull << f.shift) - static_cast<unsigned long long>(f.d))) / static_cast<unsigned long long>(f.d) + 1ull);
    return f;
}
__device__ __forceinline__ int fdiv(int n, const FastDiv& f) {
    return static_cast<int>((__umulhi(f.mul, static_cast<unsigned>(n)) + static_cast<unsigned>(n)) >> f.shift);
}

struct GemmParams {
    int conv;              // 0: plain GEMM, 1: implicit-GEMM convolution (A tile = 4-D box of pixels)
    int M, N;              // output rows (GEMM rows or pixels) and columns
    int num_kb;            // reduction blocks of the whole problem
    int splits;            // split-K: each output tile is produced `splits` times over disjoint reduction ranges
    int m_tiles, n_tiles;
    int a_mn, b_mn;        // operand majors (0 = K-major, 1 = MN-major)
    int a_bytes;           // bytes one A stage receives from TMA
    // convolution geometry
    int H, W, S, pad, Nimg;
    int flip;              // 1: error-backward, taps are read mirrored (offset pad - r instead of r - pad)
    int tapstride;         // elements between consecutive taps in a filter row
    int BW, BH, BI;        // pixels of one tile along w, h and images; BW*BH*BI <= 128
    int tiles_w, tiles_h;
    FastDiv fd_mn, fd_n, fd_tw, fd_th;  // by m_tiles * n_tiles, n_tiles, tiles_w, tiles_h (set by finish_params)
    int cblocks;           // 128-byte blocks per tap: ceil(reduction channels / 128)
    int red;               // reduction channels per tap (conv) -- the last block of a tap may be partial
    unsigned* maxabs;      // max|acc| is reduced into this word; may be null (split-K partials)
    int32_t* status;
    int group_m;           // GEMM tile order: row tiles per group (0 / 1: plain row-major)
    int nstages;           // stages of the ring actually used (<= the compiled maximum; tuning / experiments)
    int split_cols;        // 1: both epilogue warpgroups share every tile (alternate 128-column groups); 0: they alternate tiles
    // fused requantisation (FUSED kernels): int8 output narrowed by the shift in state[0].
    // state = {shift, max|acc|, redo flag, redo count, finished-CTA ticket}; the last CTA of a first
    // launch derives the true shift from max|acc|, publishes it with the exponent / shift outputs and
    // raises the redo flag when the applied shift was wrong.
    int32_t* state;
    int only_if_redo;      // 1: this launch does nothing unless state[2] != 0, and verifies nothing
    int kind, target_bits;
    const int32_t* exp_a; const int32_t* exp_b; int32_t* exp_out; int32_t* shift_out;
    int mode, relu;
    int8_t* out8;          // fused kernels: the int8 output as a plain pointer (rows = row_lin, pitch N bytes)
    const int8_t* mask;    // fused kernels: optional ReLU-backward mask, same shape as the output (zero where mask <= 0)
    int8_t* pool_out;      // parked kernel, forward convolutions: optional 2x2 / stride-2 max-pooled copy of the output [N][H/2][W/2][K]
    uint32_t* side;        // streaming fused kernel, round-to-nearest without ReLU: two more bits per output (16 per word, rows of
                           // N / 4 bytes) from which the output for the next LOWER shift follows exactly (requant_step_down)
    const unsigned long long* seed;
    unsigned rng_stream;
    unsigned long long rng_offset;
};

constexpr int GEMM_THREADS = 320;  // producer warp, MMA warp, two epilogue warpgroups of 4 warps
constexpr unsigned STEP_DOWN_RUN = 12;  // step-downs in a row after which the predicted shift is lowered (< 16)

template <int BN, bool FUSED, bool TWO = false>
struct GemmCfg {
    static constexpr int B_STAGE_BYTES = (TWO ? BN / 2 : BN) * ROW_BYTES;  // a CTA of a pair holds half of the B columns
    static constexpr int STAGE_BYTES = PANEL_BYTES + B_STAGE_BYTES;
    // staging per epilogue warpgroup: one 128 x 128 int8 tile (fused) or two 128 x 32 int32 tiles
    static constexpr int EPI_GROUP_BYTES = FUSED ? EPI_CHUNK_BYTES : 2 * EPI_CHUNK_BYTES;
    static constexpr int EPI_BYTES = 2 * EPI_GROUP_BYTES;
    static constexpr int STAGES = (224 * 1024 - EPI_BYTES) / STAGE_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;  // two accumulators; 256 or 512 columns
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void report_abort(int32_t* status, int code, int role) {
    if (status != nullptr && atomicCAS(status, 0, code) == 0) {
        status[1] = static_cast<int32_t>(blockIdx.x + blockIdx.y * gridDim.x);
        status[2] = role;
    }
}

// Four accumulators of one row -> four int8 packed in a word (NITI's shift, see requant.cuh).
// Round-to-nearest (the default of activations and errors) gets a short branch-free form, below.
// Two int32 -> two saturated bytes in the low half of the result, `upper` moved into the high half
// (cvt.pack: d = upper << 16 | sat(hi) << 8 | sat(lo)).
__device__ __forceinline__ uint32_t pack2_sat_s8(int hi, int lo, uint32_t upper) {
    uint32_t d;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
    return d;
}
__device__ __forceinline__ uint32_t pack2_sat_u8(int hi, int lo, uint32_t upper) {
    uint32_t d;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
    return d;
}
// Round half away from zero is (x + half + (x >> 31)) >> shift with an arithmetic shift (for x < 0 that is
// -((|x| + half) >> shift)); the saturating pack clamps to a byte and one packed min / max finishes the clamp to
// +-127 (ReLU: the unsigned pack turns negatives into 0).  About 3 instructions per value.
template <bool RELU>
__device__ __forceinline__ uint32_t narrow4_nearest(const uint32_t* v, int shift, int half) {
    int y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int x = static_cast<int>(v[j]);
        y[j] = RELU ? (x + half) >> shift : (x + half + (x >> 31)) >> shift;
    }
    if (RELU) return __vminu4(pack2_sat_u8(y[1], y[0], pack2_sat_u8(y[3], y[2], 0u)), 0x7F7F7F7Fu);
    return __vmaxs4(pack2_sat_s8(y[1], y[0], pack2_sat_s8(y[3], y[2], 0u)), 0x81818181u);
}
__device__ __forceinline__ uint32_t narrow4(const uint32_t* v, int shift, int mode, int relu, const uint32_t* rnd) {
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int y = narrow(static_cast<int>(v[j]), shift, mode, rnd[j]);
        if (relu && y < 0) y = 0;
        w |= static_cast<uint32_t>(static_cast<uint8_t>(y)) << (8 * j);
    }
    return w;
}

// Round-to-nearest narrowing of 16 values (one 16-byte piece of an output row) with shift S >= 2 that also keeps bits
// S-1 and S-2 of the rounded-up sum: with u = x + 2^(S-1) - (x < 0), T = u >> (S-2) = 4 * (u >> S) + code, and the value
// for shift S - 1, sign(x) * ((|x| + 2^(S-2)) >> (S-1)), is 2 * (u >> S) + (code == 3) - (code == 0) for either sign.
// The code of byte j of word q sits at bit 8 j + 2 q of the piece's code word.
__device__ __forceinline__ uint32_t narrow16_nearest_codes(const uint32_t* v, int shift2, int half, uint32_t* packed) {
    uint32_t codes = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        int y[4], t[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int x = static_cast<int>(v[4 * q + j]);
            t[j] = (x + half + (x >> 31)) >> shift2;
            y[j] = t[j] >> 2;
        }
        packed[q] = __vmaxs4(pack2_sat_s8(y[1], y[0], pack2_sat_s8(y[3], y[2], 0u)), 0x81818181u);
        // the low bytes of the four t side by side, their two low bits moved to this word's place in every byte
        const uint32_t low = __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410);
        codes |= (low & 0x03030303u) << (2 * q);
    }
    return codes;
}
// Four outputs narrowed with shift S (one word) and their codes (bits 0-1 of each byte of e) -> the four outputs for
// shift S - 1, clamped to +-127.  Two 16-bit lanes per register, biased by 128 so that plain 32-bit arithmetic cannot
// borrow between lanes; the lane-wise add + min / max are single instructions.
__device__ __forceinline__ uint32_t step_down4(uint32_t y4, uint32_t e) {
    const uint32_t e1 = e >> 1;
    const uint32_t eq3 = e & e1;                       // bit 0 of a byte: code == 3
    const uint32_t eq0 = ~(e | e1) & 0x01010101u;      // code == 0
    const uint32_t dd = eq3 + 0x01010101u - eq0;       // d + 1 in {0, 1, 2} per byte
    const uint32_t yb = y4 ^ 0x80808080u;              // y + 128 per byte
    uint32_t la = (yb & 0x00FF00FFu) * 2u + (dd & 0x00FF00FFu);                // bytes 0, 2: 2 y + d + 257
    uint32_t lb = ((yb >> 8) & 0x00FF00FFu) * 2u + ((dd >> 8) & 0x00FF00FFu);  // bytes 1, 3
    la = __viaddmax_s16x2(__viaddmin_s16x2(la, 0xFFFFFFFFu, 0x017F017Fu), 0u, 0x00810081u);  // clamp(2 y + d, +-127) + 256
    lb = __viaddmax_s16x2(__viaddmin_s16x2(lb, 0xFFFFFFFFu, 0x017F017Fu), 0u, 0x00810081u);
    return __byte_perm(la, lb, 0x6240);                // the low byte of a lane is the value modulo 256
}
// The whole int8 output, narrowed with shift S by the launch before, rewritten for shift S - 1 from the side codes
// (every thread of the grid takes 16-byte pieces; the ReLU-backward mask is applied again, the codes ignore it).
__device__ void requant_step_down(int8_t* out8, const uint32_t* side, const int8_t* mask, long long pieces) {
    constexpr int U = 8;
    uint4* o = reinterpret_cast<uint4*>(out8);
    const uint4* m = reinterpret_cast<const uint4*>(mask);
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < pieces; i0 += U * step) {
        uint4 y[U], k[U];
        uint32_t c[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long i = i0 + u * step;
            if (i < pieces) {
                y[u] = __ldcg(o + i);
                c[u] = __ldcg(side + i);
                if (mask != nullptr) k[u] = __ldg(m + i);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long i = i0 + u * step;
            if (i < pieces) {
                uint4 r;
                r.x = step_down4(y[u].x, c[u] & 0x03030303u); r.y = step_down4(y[u].y, (c[u] >> 2) & 0x03030303u);
                r.z = step_down4(y[u].z, (c[u] >> 4) & 0x03030303u); r.w = step_down4(y[u].w, (c[u] >> 6) & 0x03030303u);
                if (mask != nullptr) {
                    r.x &= __vcmpgts4(k[u].x, 0); r.y &= __vcmpgts4(k[u].y, 0);
                    r.z &= __vcmpgts4(k[u].z, 0); r.w &= __vcmpgts4(k[u].w, 0);
                }
                o[i] = r;
            }
        }
    }
}

// Output tile (row tile, column tile) of the mn-th tile in launch order.  Convolutions: row-major (the few column
// tiles of a row tile run together and share its activation tile).  GEMMs: row tiles in groups of 8, column-major
// inside a group, so the ~148 tiles in flight at any time cover a compact block of the output (8 x ~18 tiles) instead
// of 2-3 whole rows: a wave then re-reads ~36 MB of operands instead of all of B.  Only when the operands do not fit
// in L2 anyway (group_m is set on the host): 8192^3 406 -> 376 us, 16384^3 3679 -> 2977 us, 4096^3 unchanged.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int mn, int* m_pair, int* n_t) {
    if (p.group_m <= 1) { *m_pair = fdiv(mn, p.fd_n); *n_t = mn - *m_pair * p.n_tiles; return; }
    const int GM = p.group_m;
    const int per_group = GM * p.n_tiles;
    const int group = mn / per_group, in_group = mn % per_group;
    const int first = group * GM;
    const int rows = min(GM, p.m_tiles - first);
    *m_pair = first + in_group % rows;
    *n_t = in_group / rows;
}

// ---- warp roles shared by the streaming kernel and the accumulator-parking kernel -------------
// TMA producer: fills the stage ring for every tile of this CTA, in tile order.  The WHOLE warp runs the loop and
// an elected lane issues.  TMA and MMA instructions take their operands from uniform registers, and the compiler keeps
// addresses, coordinates and descriptors there only while every branch around them is provably warp-uniform: waits
// therefore spin INSIDE one asm statement and hand back a voted verdict (mbar_wait_uniform), values read from shared
// memory or special registers pass through a shuffle, and the issuing lane comes from elect.sync.  Measured on B200
// (clock64 around the instructions): 50 cycles per tcgen05.mma and ~20 per TMA instruction this way; 85-90 and ~50 when
// a loop-carried value depends on a per-lane asm result or the issuer is chosen by `lane == 0`; a loop entered by a
// single lane sits in between.  Per-tile integer divisions are skipped when the reduction is not split.
// TWO: this CTA is half of a CTA pair (cluster ranks 0/1).  Tiles are 256 rows high: rank r owns rows
// [128 r, 128 r + 128) of the pair's tile (m tile 2*pair_m + r) and columns [r BN/2, (r+1) BN/2) of the B
// operand; all byte counts are reported to rank 0's "full" barrier, which its MMA thread waits on.
template <int BN, int STAGES, int STAGE_BYTES, bool TWO>
__device__ __forceinline__ void producer_role(uint8_t* smem, uint64_t* full_bar, uint64_t* empty_bar, const CUtensorMap* tmA,
                                              const CUtensorMap* tmB, const GemmParams& p, volatile int* abort_flag) {
    const int mn_tiles = p.m_tiles * p.n_tiles;
    const int total_tiles = mn_tiles * p.splits;
    const uint32_t rank = TWO ? __shfl_sync(0xFFFFFFFFu, cluster_ctarank(), 0) : 0u;  // a special register: make it provably uniform
    const int first = TWO ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int step = TWO ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    constexpr int BNH = TWO ? BN / 2 : BN;  // B columns this CTA loads
    const int nst = (p.nstages > 0 && p.nstages < STAGES) ? p.nstages : STAGES;
    const uint32_t abort_addr = smem_u32(const_cast<int*>(abort_flag));
    const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    const int conv = keep_reg(p.conv), flip = keep_reg(p.flip), pad = keep_reg(p.pad), S = keep_reg(p.S), cblocks = keep_reg(p.cblocks);
    const int tapstride = keep_reg(p.tapstride), b_mn = keep_reg(p.b_mn), a_mn = keep_reg(p.a_mn);
    const uint32_t tx_bytes = static_cast<uint32_t>(keep_reg(TWO ? 2 * (p.a_bytes + BNH * ROW_BYTES) : p.a_bytes + BN * ROW_BYTES));
    int s = 0; uint32_t ph = 0;
    uint32_t sa = smem0, fb_cur = full0, eb_cur = empty0;  // running stage pointers, wrapping with the ring
    DBG_DECL;
    DBG_CLK(c_begin);
    for (int tile = first; tile < total_tiles; tile += step) {
        int mn = tile, kb_lo = 0, kb_hi = p.num_kb;
        if (p.splits > 1) {
            const int split = fdiv(tile, p.fd_mn);
            mn = tile - split * mn_tiles;
            kb_lo = static_cast<int>(static_cast<long long>(split) * p.num_kb / p.splits);
            kb_hi = static_cast<int>(static_cast<long long>(split + 1) * p.num_kb / p.splits);
        }
        int m_pair, n_t;
        tile_coords(p, mn, &m_pair, &n_t);
        const int m_t = TWO ? 2 * m_pair + static_cast<int>(rank) : m_pair;
        int tw = 0, th = 0, tn = 0;
        if (conv) { const int q1 = fdiv(m_t, p.fd_tw); tw = m_t - q1 * p.tiles_w; tn = fdiv(q1, p.fd_th); th = q1 - tn * p.tiles_h; }
        const int ncol = n_t * BN + static_cast<int>(rank) * BNH;  // first B column of this CTA
        const int px = tw * p.BW, py = th * p.BH, pn = tn * p.BI;
        // This loop is one warp's serial instruction stream and sets the pace of the whole pipeline: the tap
        // (r, sx) and channel block cb of a reduction block are kept as running counters (four integer divisions per
        // block cost more than the block's MMAs), waits return nothing to branch on, pointers advance by addition.
        int cb = 0, sx = 0, r = 0;
        if (conv && kb_lo != 0) { const int tap0 = kb_lo / cblocks; cb = kb_lo % cblocks; r = tap0 / S; sx = tap0 % S; }
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
            mbar_wait_quiet(eb_cur, ph ^ 1u, abort_addr);
            DBG_ACC(22, 1);
            const uint32_t sb = sa + PANEL_BYTES;
            uint32_t fb = fb_cur;
            if (elect_one()) {
                if (TWO) {
                    if (rank == 0) mbar_arrive_expect_tx(fb, tx_bytes);
                    fb = mapa_u32(fb, 0);
                } else {
                    mbar_arrive_expect_tx(fb, tx_bytes);
                }
                if (conv) {
                    const int tap = r * S + sx;
                    const int dx = flip ? pad - sx : sx - pad, dy = flip ? pad - r : r - pad;
                    if (TWO) tma_load_4d_pair(sa, tmA, fb, cb * ROW_BYTES, px + dx, py + dy, pn);
                    else     tma_load_4d(sa, tmA, fb, cb * ROW_BYTES, px + dx, py + dy, pn);
                    if (b_mn) {
#pragma unroll
                        for (int q = 0; q < BNH / 128; ++q) {
                            if (TWO) tma_load_2d_pair(sb + q * PANEL_BYTES, tmB, fb, tap * tapstride + ncol + q * 128, cb * 128);
                            else     tma_load_2d(sb + q * PANEL_BYTES, tmB, fb, tap * tapstride + ncol + q * 128, cb * 128);
                        }
                    } else {
                        if (TWO) tma_load_2d_pair(sb, tmB, fb, tap * tapstride + cb * ROW_BYTES, ncol);
                        else     tma_load_2d(sb, tmB, fb, tap * tapstride + cb * ROW_BYTES, ncol);
                    }
                } else {
                    if (TWO) {
                        if (a_mn) tma_load_2d_pair(sa, tmA, fb, m_t * BLOCK_M, kb * 128);
                        else      tma_load_2d_pair(sa, tmA, fb, kb * ROW_BYTES, m_t * BLOCK_M);
                    } else {
                        if (a_mn) tma_load_2d(sa, tmA, fb, m_t * BLOCK_M, kb * 128);
                        else      tma_load_2d(sa, tmA, fb, kb * ROW_BYTES, m_t * BLOCK_M);
                    }
                    if (b_mn) {
#pragma unroll
                        for (int q = 0; q < BNH / 128; ++q) {
                            if (TWO) tma_load_2d_pair(sb + q * PANEL_BYTES, tmB, fb, ncol + q * 128, kb * 128);
                            else     tma_load_2d(sb + q * PANEL_BYTES, tmB, fb, ncol + q * 128, kb * 128);
                        }
                    } else {
                        if (TWO) tma_load_2d_pair(sb, tmB, fb, kb * ROW_BYTES, ncol);
                        else     tma_load_2d(sb, tmB, fb, kb * ROW_BYTES, ncol);
                    }
                }
            }
            if (conv && ++cb == cblocks) { cb = 0; if (++sx == S) { sx = 0; ++r; } }
            sa += STAGE_BYTES; fb_cur += 8u; eb_cur += 8u;
            if (++s == nst) { s = 0; ph ^= 1u; sa = smem0; fb_cur = full0; eb_cur = empty0; }
        }
    }
    if (*abort_flag) report_abort(p.status, 1, 0);  // a quiet wait of this role (or another role) gave up
    DBG_CLK(c_end); DBG_ACC(20, c_end - c_begin);
    DBG_OUT(20);
}

// MMA issuer: the whole warp runs the loop with warp-uniform control flow (see the producer), one elected lane issues
// the MMAs and the commits.  Streaming: two accumulators used alternately, each handed back by the
// epilogue (tempty).  PARKED: tile i of this CTA accumulates into TMEM columns [i*BN, (i+1)*BN) and
// stays there until the kernel ends, so no accumulator is ever waited for.
// TWO: run by rank 0 of a CTA pair only; M = 256 MMAs over both CTAs' shared and tensor memory, and every
// completion (stage free, accumulator full) is signalled to both CTAs.
template <bool TWO>
__device__ __forceinline__ void umma_issue(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    if (TWO) umma_i8_pair(d_tmem, a, b, idesc, accumulate); else umma_i8(d_tmem, a, b, idesc, accumulate);
}
template <int BN, int STAGES, int STAGE_BYTES, bool PARKED, bool TWO>
__device__ __forceinline__ void mma_role(uint8_t* smem, uint64_t* full_bar, uint64_t* empty_bar, uint64_t* tfull_bar,
                                         uint64_t* tempty_bar, uint32_t tmem_base_in, const GemmParams& p, volatile int* abort_flag) {
    const int mn_tiles = p.m_tiles * p.n_tiles;
    const int total_tiles = mn_tiles * p.splits;
    const uint32_t idesc = make_idesc_i8(TWO ? 2 * BLOCK_M : BLOCK_M, BN, p.a_mn, p.b_mn);
    const int nst = (p.nstages > 0 && p.nstages < STAGES) ? p.nstages : STAGES;
    const int first = TWO ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int step = TWO ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, tmem_base_in, 0);  // read from shared memory: make it provably uniform
    const uint32_t abort_addr = smem_u32(const_cast<int*>(abort_flag));
    const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    // operand descriptors of stage 0 (a stage's are these advanced by the stage offset) and the K = 32 steps
    const uint32_t s0 = smem_u32(smem);
    const uint64_t a_base = p.a_mn ? make_smem_desc(s0, PANEL_BYTES, 1024, SWIZZLE_128B_CODE) : make_smem_desc(s0, 16, 1024, SWIZZLE_128B_CODE);
    const uint64_t b_base = p.b_mn ? make_smem_desc(s0 + PANEL_BYTES, PANEL_BYTES, 1024, SWIZZLE_128B_CODE)
                                   : make_smem_desc(s0 + PANEL_BYTES, 16, 1024, SWIZZLE_128B_CODE);
    const uint32_t a_step = static_cast<uint32_t>(keep_reg((p.a_mn ? 32 * ROW_BYTES : 32) >> 4));  // in descriptor units of 16 bytes
    const uint32_t b_step = static_cast<uint32_t>(keep_reg((p.b_mn ? 32 * ROW_BYTES : 32) >> 4));
    const int conv = keep_reg(p.conv), red = keep_reg(p.red), cblocks = keep_reg(p.cblocks), num_kb = keep_reg(p.num_kb), splits = keep_reg(p.splits);
    int s = 0; uint32_t ph = 0; bool ok = true; int it = 0;
    // every reduction block has four MMAs unless a conv tap's channel count ends in a partial 128-byte block
    const bool all4 = !conv || (red & 127) == 0;
    // running stage pointers: descriptors and barrier addresses advance by one stage per block and wrap with the ring
    const uint64_t stage_step = STAGE_BYTES >> 4;
    uint64_t a_cur = a_base, b_cur = b_base;
    uint32_t full_cur = full0, empty_cur = empty0;
    DBG_DECL;
#ifdef NITI_PARKED_TIMING
    long long c_first = 0;
#endif
    for (int tile = first; ok && tile < total_tiles; tile += step, ++it) {
        const int acc = PARKED ? it : (it & 1);
        if (!PARKED) {
            const uint32_t aph = (it >> 1) & 1u;
            ok = mbar_wait_uniform(smem_u32(&tempty_bar[acc]), aph ^ 1u, abort_addr);
            if (!ok) { *abort_flag = 1; report_abort(p.status, 2, 1); break; }
            tc_fence_after();
        }
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        int kb_lo = 0, kb_hi = num_kb;
        if (splits > 1) {
            const int split = tile / mn_tiles;
            kb_lo = static_cast<int>(static_cast<long long>(split) * num_kb / splits);
            kb_hi = static_cast<int>(static_cast<long long>(split + 1) * num_kb / splits);
        }
        int cb = (conv && kb_lo != 0) ? kb_lo % cblocks : 0;  // channel block within the tap: a running counter, no division per block
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
            DBG_ACC(19, 1);
#ifdef NITI_PARKED_TIMING
            if (it == 0 && kb == kb_lo) { c_first = clock64(); if (PARKED) PARK_STAMP(2); }
#endif
            if (all4) {
                // wait for the stage, four MMAs, commit: one asm statement, nothing for the loop to branch on
                umma_block4_wait<TWO>(d_tmem, a_cur, b_cur, a_step, b_step, idesc, static_cast<uint32_t>(kb != kb_lo), empty_cur,
                                      full_cur, ph, abort_addr);
            } else {
                // a partial block: issue only the MMAs (K = 32 each) that cover real channels (the rest is TMA zero fill)
                const int left = red - cb * 128;
                const int nmma = left >= 128 ? 4 : (left + 31) >> 5;
                if (++cb == cblocks) cb = 0;
                mbar_wait_quiet(full_cur, ph, abort_addr);
                if (elect_one()) {
                    for (int k = 0; k < nmma; ++k)
                        umma_issue<TWO>(d_tmem, a_cur + k * a_step, b_cur + k * b_step, idesc, static_cast<uint32_t>(kb != kb_lo || k != 0));
                    if (TWO) umma_commit_pair(empty_cur); else umma_commit(empty_cur);
                }
            }
            a_cur += stage_step; b_cur += stage_step; full_cur += 8u; empty_cur += 8u;
            if (++s == nst) { s = 0; ph ^= 1u; a_cur = a_base; b_cur = b_base; full_cur = full0; empty_cur = empty0; }
        }
        if (ok && elect_one()) { if (TWO) umma_commit_pair(smem_u32(&tfull_bar[acc])); else umma_commit(smem_u32(&tfull_bar[acc])); }
    }
    if (*abort_flag) report_abort(p.status, 3, 1);  // a quiet wait of this role (or another role) gave up
    if (PARKED) PARK_STAMP(3);
#ifdef NITI_PARKED_TIMING
    DBG_ACC(16, clock64() - c_first);
#endif
    DBG_OUT(16);
}

// Output row of an epilogue thread: validity, TMA store coordinates of its tile, linear row index.
struct RowInfo { bool valid; int cy, cz, cw; long long row_lin; long long pool_row; };
__device__ __forceinline__ RowInfo row_info(const GemmParams& p, int m_t, int split, int row_in_tile) {
    RowInfo r;
    if (p.conv) {
        const int tw = m_t % p.tiles_w, th = (m_t / p.tiles_w) % p.tiles_h, tn = m_t / (p.tiles_w * p.tiles_h);
        const int w = tw * p.BW + row_in_tile % p.BW;
        const int h = th * p.BH + (row_in_tile / p.BW) % p.BH;
        const int n = tn * p.BI + row_in_tile / (p.BW * p.BH);
        r.valid = row_in_tile < p.BW * p.BH * p.BI && w < p.W && h < p.H && n < p.Nimg;
        r.cy = tw * p.BW; r.cz = th * p.BH; r.cw = tn * p.BI;
        r.row_lin = (static_cast<long long>(n) * p.H + h) * p.W + w;
        // row of the 2x2-pooled tensor this pixel's window goes to; only the window's top-left pixel writes it
        r.pool_row = ((w | h) & 1) == 0 ? (static_cast<long long>(n) * (p.H >> 1) + (h >> 1)) * (p.W >> 1) + (w >> 1) : -1;
    } else {
        r.row_lin = static_cast<long long>(m_t) * BLOCK_M + row_in_tile;
        r.valid = r.row_lin < p.M;
        r.cy = m_t * BLOCK_M; r.cz = split; r.cw = 0;
        r.pool_row = -1;
    }
    return r;
}
// max|x| = max(max x, -min x) over the first `lim` of 128 accumulators: short chains of 3-input min/max
__device__ __forceinline__ void track_minmax(const uint32_t (&v)[4][32], int lim, int (&vmax)[4], int (&vmin)[4]) {
    if (lim >= 128) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                vmax[j] = __vimax3_s32(vmax[j], static_cast<int>(v[j][i]), static_cast<int>(v[j][i + 1]));
                vmin[j] = __vimin3_s32(vmin[j], static_cast<int>(v[j][i]), static_cast<int>(v[j][i + 1]));
            }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (j * 32 + i < lim) {
                    vmax[0] = max(vmax[0], static_cast<int>(v[j][i]));
                    vmin[0] = min(vmin[0], static_cast<int>(v[j][i]));
                }
    }
}
__device__ __forceinline__ unsigned fold_minmax(const int (&vmax)[4], const int (&vmin)[4]) {
    const int hi = max(max(vmax[0], vmax[1]), max(vmax[2], vmax[3]));
    const int lo = min(min(vmin[0], vmin[1]), min(vmin[2], vmin[3]));
    return max(static_cast<unsigned>(hi), static_cast<unsigned>(-static_cast<long long>(lo)));
}
// The same two steps on 32 accumulators at a time, for epilogues that run once or twice per launch: there
// every instruction is fetched cold, so a rolled loop over four 32-column chunks (a quarter of the code, the
// last three trips from the instruction cache) beats the straight-line 128-column form.
__device__ __forceinline__ void minmax32(const uint32_t (&v)[32], int lim, int (&vmax)[4], int (&vmin)[4]) {
    if (lim >= 32) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            vmax[0] = __vimax3_s32(vmax[0], static_cast<int>(v[i]), static_cast<int>(v[i + 1]));
            vmin[0] = __vimin3_s32(vmin[0], static_cast<int>(v[i]), static_cast<int>(v[i + 1]));
            vmax[1] = __vimax3_s32(vmax[1], static_cast<int>(v[i + 2]), static_cast<int>(v[i + 3]));
            vmin[1] = __vimin3_s32(vmin[1], static_cast<int>(v[i + 2]), static_cast<int>(v[i + 3]));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < lim) {
                vmax[0] = max(vmax[0], static_cast<int>(v[i]));
                vmin[0] = min(vmin[0], static_cast<int>(v[i]));
            }
    }
}
__device__ __forceinline__ void narrow32(const uint32_t (&v)[32], uint32_t (&packed)[8], int shift, int mode, int relu,
                                         unsigned long long seed, unsigned rng_stream, unsigned long long e0) {
    if (mode == ROUND_NEAREST && shift > 0) {
        const int half = 1 << (shift - 1);
        if (relu) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) packed[i >> 2] = narrow4_nearest<true>(&v[i], shift, half);
        } else {
#pragma unroll
            for (int i = 0; i < 32; i += 4) packed[i >> 2] = narrow4_nearest<false>(&v[i], shift, half);
        }
    } else {
        const bool stochastic = mode == ROUND_STOCHASTIC && shift > 0;
#pragma unroll 1
        for (int i = 0; i < 32; i += 4) {
            uint32_t rnd[4] = {0, 0, 0, 0};
            if (stochastic) {
                const unsigned long long e = e0 + i;
                if ((e & 3ull) == 0) random_block(seed, rng_stream, e >> 2, rnd);
                else {
#pragma unroll
                    for (int t = 0; t < 4; ++t) rnd[t] = random_word(seed, rng_stream, e + t);
                }
            }
            uint32_t x[4];
            // select without dynamic register indexing
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                x[t] = v[t];
#pragma unroll
                for (int k = 4; k < 32; k += 4) x[t] = (i == k) ? v[k + t] : x[t];
            }
            const uint32_t w = narrow4(x, shift, mode, relu, rnd);
#pragma unroll
            for (int k = 0; k < 8; ++k) if (i == 4 * k) packed[k] = w;
        }
    }
}
// ReLU backward folded into an error-backward epilogue: zero the packed int8 outputs where the layer's forward input
// (the ReLU's output) was not positive.  `m` points at this row's mask bytes for the same columns; `cols` of them exist.
template <int WORDS>
__device__ __forceinline__ void apply_relu_mask(uint32_t (&packed)[WORDS], const int8_t* m, int cols) {
#pragma unroll
    for (int q = 0; q < WORDS / 4; ++q)
        if (16 * q + 16 <= cols) {
            const uint4 x = __ldg(reinterpret_cast<const uint4*>(m) + q);
            packed[4 * q + 0] &= __vcmpgts4(x.x, 0); packed[4 * q + 1] &= __vcmpgts4(x.y, 0);
            packed[4 * q + 2] &= __vcmpgts4(x.z, 0); packed[4 * q + 3] &= __vcmpgts4(x.w, 0);
        }
}
// The same in two steps, so that the loads can be issued long before the bytes they gate exist: PIECES 16-byte pieces
// of the mask row into registers, then the AND.  m null: nothing to do.
template <int PIECES>
__device__ __forceinline__ void mask_load(const int8_t* m, int cols, uint4 (&mk)[PIECES]) {
#pragma unroll
    for (int q = 0; q < PIECES; ++q)
        if (m != nullptr && 16 * q + 16 <= cols) mk[q] = __ldg(reinterpret_cast<const uint4*>(m) + q);
}
template <int PIECES>
__device__ __forceinline__ void mask_apply(uint32_t* packed, const int8_t* m, int cols, const uint4 (&mk)[PIECES]) {
#pragma unroll
    for (int q = 0; q < PIECES; ++q)
        if (m != nullptr && 16 * q + 16 <= cols) {
            packed[4 * q + 0] &= __vcmpgts4(mk[q].x, 0); packed[4 * q + 1] &= __vcmpgts4(mk[q].y, 0);
            packed[4 * q + 2] &= __vcmpgts4(mk[q].z, 0); packed[4 * q + 3] &= __vcmpgts4(mk[q].w, 0);
        }
}
// Byte-wise maximum over a 2x2 pixel window whose four pixels are the rows of lanes l, l^1, l^bw, l^bw^1 of this warp
// (all 32 lanes call it): afterwards every lane of a window holds the window's maxima.
__device__ __forceinline__ void pool_window(uint32_t (&w)[8], int bw) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t m = __vmaxs4(w[i], __shfl_xor_sync(0xFFFFFFFFu, w[i], 1));
        w[i] = __vmaxs4(m, __shfl_xor_sync(0xFFFFFFFFu, m, bw));
    }
}
// 32 packed int8 of one output row to global memory, as two 16-byte stores; `row` is null for rows outside the tensor,
// `off` the byte offset within the unit's columns of which `cols` exist (a multiple of 16)
__device__ __forceinline__ void store_piece(int8_t* row, int off, int cols, const uint32_t (&w)[8]) {
    if (row == nullptr) return;
    if (off + 16 <= cols) *reinterpret_cast<uint4*>(row + off) = make_uint4(w[0], w[1], w[2], w[3]);
    if (off + 32 <= cols) *reinterpret_cast<uint4*>(row + off + 16) = make_uint4(w[4], w[5], w[6], w[7]);
}
// a 32-byte piece (chunk j of the row's 128 bytes) at its 128-byte-swizzled place in the staging tile
__device__ __forceinline__ void stage_piece(uint32_t buf, int row, int j, const uint32_t (&w)[8]) {
    const uint32_t base = buf + static_cast<uint32_t>(row) * 128u;
    st_shared_v4(base + (static_cast<uint32_t>((2 * j) ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
    st_shared_v4(base + (static_cast<uint32_t>((2 * j + 1) ^ (row & 7)) << 4), w[4], w[5], w[6], w[7]);
}
// 128 accumulators of one row -> 32 words of packed int8
__device__ __forceinline__ void narrow_row(const uint32_t (&v)[4][32], uint32_t (&packed)[32], int shift, int mode, int relu,
                                           unsigned long long seed, unsigned rng_stream, unsigned long long e0) {
    if (mode == ROUND_NEAREST && shift > 0) {
        const int half = 1 << (shift - 1);
        if (relu) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 32; i += 4) packed[j * 8 + (i >> 2)] = narrow4_nearest<true>(&v[j][i], shift, half);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 32; i += 4) packed[j * 8 + (i >> 2)] = narrow4_nearest<false>(&v[j][i], shift, half);
        }
    } else {
        const bool stochastic = mode == ROUND_STOCHASTIC && shift > 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                uint32_t rnd[4] = {0, 0, 0, 0};
                if (stochastic) {
                    const unsigned long long e = e0 + j * 32 + i;
                    if ((e & 3ull) == 0) random_block(seed, rng_stream, e >> 2, rnd);
                    else {
#pragma unroll
                        for (int t = 0; t < 4; ++t) rnd[t] = random_word(seed, rng_stream, e + t);
                    }
                }
                packed[j * 8 + (i >> 2)] = narrow4(&v[j][i], shift, mode, relu, rnd);
            }
    }
}

template <int BN, bool FUSED, bool TWO>
__global__ void __launch_bounds__(GEMM_THREADS, 1)  // 10 warps: 3 on one scheduler -> at most 168 registers per thread
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
    using Cfg = GemmCfg<BN, FUSED, TWO>;
    constexpr int STAGES = Cfg::STAGES;
    if (FUSED && p.only_if_redo) {
        const int verdict = p.state[2] & 3;
        if (verdict == 0) return;  // the prediction was right: nothing to redo
        if (verdict == 2) {        // one bit too many was shifted out and the side codes hold what is missing
            requant_step_down(p.out8, p.side, p.mask, static_cast<long long>(p.M) * p.N / 16);
            return;
        }
    }

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* epi_smem = smem + STAGES * Cfg::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::EPI_BYTES);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + STAGES;
    uint64_t* tfull_bar = bars + 2 * STAGES;
    uint64_t* tempty_bar = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile unsigned* warp_max = reinterpret_cast<volatile unsigned*>(tmem_slot + 4);  // one word per epilogue warp

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = TWO ? cluster_ctarank() : 0u;  // rank 0 of a pair issues the MMAs and owns the barriers the MMA thread waits on

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(smem_u32(&full_bar[i]), 1); mbar_init(smem_u32(&empty_bar[i]), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&tfull_bar[i]), 1); mbar_init(smem_u32(&tempty_bar[i]), (p.split_cols ? 8 : 4) * (TWO ? 2 : 1)); }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        tma_prefetch_desc(&tmC);
    }
    if (warp == 1) {
        if (TWO) { tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS); tmem_relinquish_pair(); }
        else     { tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if (TWO) cluster_sync_all();  // the partner's barriers exist before anything is signalled across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int mn_tiles = p.m_tiles * p.n_tiles;  // TWO: m_tiles counts 256-row tiles of the pair
    const int total_tiles = mn_tiles * p.splits;
    const int cta_first = TWO ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int cta_step = TWO ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    // Only one lane of warps 0 and 1 works; the others wait at __syncwarp so that each warp reaches the
    // block-wide barrier of the teardown converged (an aligned barrier executed by a diverged warp is undefined).
    if (warp == 0) {
        producer_role<BN, STAGES, Cfg::STAGE_BYTES, TWO>(smem, full_bar, empty_bar, &tmA, &tmB, p, abort_flag);
        __syncwarp();
    } else if (warp == 1) {
        if (rank == 0)
            mma_role<BN, STAGES, Cfg::STAGE_BYTES, false, TWO>(smem, full_bar, empty_bar, tfull_bar, tempty_bar, tmem_base, p, abort_flag);
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (2 x 4 warps)
        // Two warpgroups.  With several tiles per CTA they alternate tiles (warpgroup g owns
        // accumulator g), so the epilogues of consecutive tiles overlap each other and the main
        // loop; with one or two wide tiles per CTA (split_cols) they share every tile, each taking
        // alternate 128-column groups, which halves the serial tail.  Per group of 128 columns:
        // four tcgen05.ld and ONE wait, the accumulator is handed back as soon as the warpgroup's
        // last columns sit in registers, max|acc| is tracked in registers, rows go to swizzled
        // staging tiles and leave through TMA stores (which clip rows/columns outside the tensor).
        //   plain kernels: int32 out, two rounds of two 128 x 32 staging tiles per column group;
        //   FUSED kernels: int8 out, narrowed with the shift in state[0], one 128 x 128-byte tile.
        const int grp = (warp - 2) >> 2;  // epilogue warpgroup 0 / 1
        const int q = warp & 3;           // TMEM lanes [32q, 32q+32) are the ones this warp may read
        const int row_in_tile = q * 32 + lane;
        const int bar_id = EPI_BARRIER + grp;
        const bool leader = (threadIdx.x == 64 + grp * 128);
        const uint32_t buf = smem_u32(epi_smem) + grp * Cfg::EPI_GROUP_BYTES;
        int shift = 0;
        unsigned long long seed = 0;
        if (FUSED) {
            shift = p.state[0];
            if (p.mode == ROUND_STOCHASTIC && shift > 0) seed = *p.seed;
        }
        const bool fast = FUSED && p.mode == ROUND_NEAREST && shift > 0;
        // a first launch also keeps what the next lower shift would need (see narrow16_nearest_codes)
        const bool with_codes = fast && shift >= 2 && !p.relu && p.side != nullptr && !p.only_if_redo;
        const int half = shift > 0 ? 1 << (shift - 1) : 0;
        int vmax[4] = {0, 0, 0, 0}, vmin[4] = {0, 0, 0, 0};
        const int tile_step = p.split_cols ? cta_step : 2 * cta_step;
        int it = p.split_cols ? 0 : grp;
        // this thread's row inside a tile never changes: pixel offsets within the tile's box
        int row_w = 0, row_h = 0, row_n = 0;
        bool row_in_box = true;
        if (p.conv) {
            const int t_ = row_in_tile / p.BW;
            row_w = row_in_tile - t_ * p.BW; row_n = t_ / p.BH; row_h = t_ - row_n * p.BH;
            row_in_box = row_in_tile < p.BW * p.BH * p.BI;
        }
        for (int tile = cta_first + (p.split_cols ? 0 : grp * cta_step); tile < total_tiles; tile += tile_step, it += (p.split_cols ? 1 : 2)) {
            const int acc = it & 1; const uint32_t aph = (it >> 1) & 1u;
            // where the tile lies, before waiting for its accumulator: the arithmetic and the first touch of the mask hide in the wait
            int split = 0, mn = tile;
            if (p.splits > 1) { split = fdiv(tile, p.fd_mn); mn = tile - split * mn_tiles; }
            int m_pair, n_t;
            tile_coords(p, mn, &m_pair, &n_t);
            const int m_t = TWO ? 2 * m_pair + static_cast<int>(rank) : m_pair;
            bool valid; int cy, cz, cw; long long row_lin;
            if (p.conv) {
                const int q1 = fdiv(m_t, p.fd_tw), tw = m_t - q1 * p.tiles_w, tn = fdiv(q1, p.fd_th), th = q1 - tn * p.tiles_h;
                cy = tw * p.BW; cz = th * p.BH; cw = tn * p.BI;
                const int w = cy + row_w, h = cz + row_h, n = cw + row_n;
                valid = row_in_box && w < p.W && h < p.H && n < p.Nimg;
                row_lin = (static_cast<long long>(n) * p.H + h) * p.W + w;
            } else {
                row_lin = static_cast<long long>(m_t) * BLOCK_M + row_in_tile;
                valid = row_lin < p.M;
                cy = m_t * BLOCK_M; cz = split; cw = 0;
            }
            if (FUSED && p.mask != nullptr && valid) prefetch_l2(p.mask + row_lin * p.N + n_t * BN);
            const uint32_t failed = mbar_wait(smem_u32(&tfull_bar[acc]), aph, abort_flag) ? 0u : 1u;
            if (barrier_or(bar_id, 128, failed)) {  // same verdict in all 128 threads of the warpgroup
                if (failed) report_abort(p.status, 4, 2);
                break;
            }
            tc_fence_after();
            const int col0 = n_t * BN;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
            // column groups of this warpgroup: all of them, or every other one when the tile is shared
            const int g_first = p.split_cols ? grp * 128 : 0, g_step = p.split_cols ? 256 : 128;
            bool released = false;
#pragma unroll 1
            for (int g0 = g_first; g0 < BN && col0 + g0 < p.N; g0 += g_step) {
                uint32_t v[4][32];
#pragma unroll
                for (int j = 0; j < 4; ++j) tmem_ld_32x32(taddr + g0 + j * 32, v[j]);
                tmem_ld_wait();
                if (g0 + g_step >= BN || col0 + g0 + g_step >= p.N) {  // this warpgroup's last group of the tile
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (TWO) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
                        else     mbar_arrive(smem_u32(&tempty_bar[acc]));
                    }
                    released = true;
                }
                const int lim = p.N - (col0 + g0);
                if (valid) {
                    // max|x| = max(max x, -min x): short chains of 3-input min/max
                    if (lim >= 128) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                vmax[j] = __vimax3_s32(vmax[j], static_cast<int>(v[j][i]), static_cast<int>(v[j][i + 1]));
                                vmin[j] = __vimin3_s32(vmin[j], static_cast<int>(v[j][i]), static_cast<int>(v[j][i + 1]));
                            }
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (j * 32 + i < lim) {
                                    vmax[0] = max(vmax[0], static_cast<int>(v[j][i]));
                                    vmin[0] = min(vmin[0], static_cast<int>(v[j][i]));
                                }
                    }
                }
                if constexpr (FUSED) {
                    uint32_t packed[32];
                    if (with_codes) {
                        uint32_t codes[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int i = 0; i < 32; i += 16)
                                codes[j * 2 + (i >> 4)] = narrow16_nearest_codes(&v[j][i], shift - 2, half, &packed[j * 8 + (i >> 2)]);
                        if (valid) {  // a row's codes are 32 consecutive bytes, the rows of a tile mostly consecutive: plain stores
                            uint32_t* srow = p.side + ((row_lin * p.N + col0 + g0) >> 4);
                            if (lim >= 128 && (p.N & 63) == 0) {  // rows of N / 4 bytes: 16-byte aligned when N is a multiple of 64
                                reinterpret_cast<uint4*>(srow)[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                                reinterpret_cast<uint4*>(srow)[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                            } else {
#pragma unroll
                                for (int k = 0; k < 8; ++k)
                                    if (16 * k + 16 <= lim) srow[k] = codes[k];
                            }
                        }
                    } else if (fast) {
                        if (p.relu) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int i = 0; i < 32; i += 4) packed[j * 8 + (i >> 2)] = narrow4_nearest<true>(&v[j][i], shift, half);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
#pragma unroll
                                for (int i = 0; i < 32; i += 4) packed[j * 8 + (i >> 2)] = narrow4_nearest<false>(&v[j][i], shift, half);
                        }
                    } else {
                        const unsigned long long e0 = p.rng_offset + static_cast<unsigned long long>(row_lin) * p.N + (col0 + g0);
                        const bool stochastic = p.mode == ROUND_STOCHASTIC && shift > 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                uint32_t rnd[4] = {0, 0, 0, 0};
                                if (stochastic) {
                                    const unsigned long long e = e0 + j * 32 + i;
                                    if ((e & 3ull) == 0) random_block(seed, p.rng_stream, e >> 2, rnd);
                                    else {
#pragma unroll
                                        for (int t = 0; t < 4; ++t) rnd[t] = random_word(seed, p.rng_stream, e + t);
                                    }
                                }
                                packed[j * 8 + (i >> 2)] = narrow4(&v[j][i], shift, p.mode, p.relu, rnd);
                            }
                    }
                    // (fetching the mask ahead of the narrowing, as the parked kernel does, costs this kernel registers it
                    // does not have: 32.2 / 36.0 us per 128x32x32 call against 29.5 / 33.4 with the loads here)
                    if (p.mask != nullptr && valid) apply_relu_mask<32>(packed, p.mask + row_lin * p.N + col0 + g0, lim);
                    if (leader) bulk_wait_read<0>();  // the previous store has read the staging tile
                    named_barrier(bar_id, 128);
                    stage_row(buf, row_in_tile, packed);
                    fence_proxy_async();
                    named_barrier(bar_id, 128);
                    if (leader) { tma_store_4d(&tmC, buf, col0 + g0, cy, cz, cw); bulk_commit(); }

                } else {
#pragma unroll
                    for (int half_i = 0; half_i < 2; ++half_i) {
                        if (col0 + g0 + half_i * 64 >= p.N) break;
                        if (leader) bulk_wait_read<0>();  // the stores of the pass before have read the staging tiles
                        named_barrier(bar_id, 128);
                        stage_row(buf, row_in_tile, v[2 * half_i]);
                        stage_row(buf + EPI_CHUNK_BYTES, row_in_tile, v[2 * half_i + 1]);
                        fence_proxy_async();
                        named_barrier(bar_id, 128);
                        if (leader) {
                            tma_store_4d(&tmC, buf, col0 + g0 + half_i * 64, cy, cz, cw);
                            if (col0 + g0 + half_i * 64 + 32 < p.N) tma_store_4d(&tmC, buf + EPI_CHUNK_BYTES, col0 + g0 + half_i * 64 + 32, cy, cz, cw);
                            bulk_commit();
                        }
                    }
                }
            }
            if (!released) {  // a shared tile none of whose column groups fell to this warpgroup
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                        if (TWO) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
                        else     mbar_arrive(smem_u32(&tempty_bar[acc]));
                    }
            }
        }
        if (leader) bulk_wait_read<0>();  // shared memory may go once the stores have read it; the writes land by the end of the grid
        const int hi = max(max(vmax[0], vmax[1]), max(vmax[2], vmax[3]));
        const int lo = min(min(vmin[0], vmin[1]), min(vmin[2], vmin[3]));
        unsigned local_max = max(static_cast<unsigned>(hi), static_cast<unsigned>(-static_cast<long long>(lo)));
        local_max = __reduce_max_sync(0xFFFFFFFFu, local_max);
        // one atomic per CTA: atomics on one address serialise at the L2, and there are 8 warps x 148 CTAs
        if (lane == 0) warp_max[warp - 2] = local_max;
        named_barrier(EPI_BARRIER + 2, 256);
        if (threadIdx.x == 64) {
            unsigned m = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) m = max(m, warp_max[i]);
            if (m != 0 && p.maxabs != nullptr) atomicMax(p.maxabs, m);
        }
        if (FUSED && !p.only_if_redo) {
            // the CTA that finishes last turns max|acc| into the true shift and checks the prediction
            if (threadIdx.x == 64) {
                __threadfence();
                int32_t* st = p.state;
                if (atomicAdd(&st[4], 1) == static_cast<int>(gridDim.x) - 1) {
                    __threadfence();
                    bool zero_out;
                    const unsigned m = static_cast<unsigned>(atomicMax(reinterpret_cast<unsigned*>(&st[1]), 0u));
                    const int true_shift = shift_for(m, p.kind, p.target_bits, &zero_out);
                    // st[2] = verdict (0 right, 1 launch again, 2 step the output down one shift from the side codes)
                    //         | run of step-downs << 4 | step-downs so far << 8
                    const int pred = st[0];
                    const unsigned old = static_cast<unsigned>(st[2]);
                    unsigned run = (old >> 4) & 15u, downs = old >> 8;
                    int verdict = 0;
                    if (true_shift == pred) {
                        run = 0;
                    } else if (p.side != nullptr && p.mode == ROUND_NEAREST && !p.relu && pred >= 2 && true_shift == pred - 1) {
                        // the prediction stays: a layer whose maximum hovers around a power of two keeps the upper
                        // shift as its guess and pays the cheap pass when the lower one applies; after
                        // STEP_DOWN_RUN lower ones in a row the guess follows
                        verdict = 2;
                        ++downs;
                        if (++run >= STEP_DOWN_RUN) { run = 0; st[0] = true_shift; }
                    } else {
                        verdict = 1;
                        run = 0;
                        st[3] += 1;
                        st[0] = true_shift;
                    }
                    st[2] = static_cast<int>(static_cast<unsigned>(verdict) | (run << 4) | (downs << 8));
                    st[1] = 0;  // ready for the next call
                    st[4] = 0;
                    if (p.exp_out) *p.exp_out = true_shift + (p.exp_a ? *p.exp_a : 0) + (p.exp_b ? *p.exp_b : 0);
                    if (p.shift_out) *p.shift_out = true_shift;
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (TWO) cluster_sync_all();  // the partner may still signal this CTA's barriers / have MMAs reading its memory
    if (warp == 1) {
        if (*abort_flag) __nanosleep(200000);  // let copies and MMAs already in flight land
        tc_fence_after();
        __syncwarp();
        if (TWO) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS); else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// Exact single-pass requantisation for problems whose accumulators all fit in tensor memory:
// every CTA owns at most 512 / BN output tiles and PARKS their int32 accumulators in TMEM.  After
// its main loops a CTA reduces max|acc| of its tiles into the global word, all CTAs meet at a grid
// barrier (cooperative launch: all resident; bounded spin), read the now final max, derive the true
// shift and only then narrow their parked accumulators to int8.  No prediction, no second launch,
// no int32 in memory.  state = {shift out, max|acc|, redo flag (cleared), redo count, exit ticket,
// -, max|acc| and barrier arrivals (adjacent: read with one 64-bit load)}; words 1, 4, 5, 6 and 7 are zero between calls.
// ------------------------------------------------------------------------------------------------
template <int BN, bool TWO = false>
struct ParkedCfg {
    static constexpr int STAGE_BYTES = PANEL_BYTES + (TWO ? BN / 2 : BN) * ROW_BYTES;
    static constexpr int EPI_GROUP_BYTES = EPI_CHUNK_BYTES;  // one 128 x 128 int8 staging tile per warpgroup
    static constexpr int EPI_BYTES = 2 * EPI_GROUP_BYTES;
    static constexpr int STAGES = (224 * 1024 - EPI_BYTES) / STAGE_BYTES;
    static constexpr int MAX_TILES = 512 / BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
};

constexpr unsigned long long GRID_BARRIER_LIMIT_NS = 500000000ull;  // 0.5 s

template <int BN, bool TWO>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
umma_parked_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
    using Cfg = ParkedCfg<BN, TWO>;
    constexpr int STAGES = Cfg::STAGES;
    if (threadIdx.x == 0) PARK_STAMP(0);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* epi_smem = smem + STAGES * Cfg::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::EPI_BYTES);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + STAGES;
    uint64_t* tfull_bar = bars + 2 * STAGES;  // one per parked tile (up to 4)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* shift_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
    volatile unsigned* warp_max = reinterpret_cast<volatile unsigned*>(tmem_slot + 4);  // one word per epilogue warp

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = TWO ? cluster_ctarank() : 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(smem_u32(&full_bar[i]), 1); mbar_init(smem_u32(&empty_bar[i]), 1); }
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&tfull_bar[i]), 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        tma_prefetch_desc(&tmC);
    }
    if (warp == 1) {
        if (TWO) { tmem_alloc_pair(smem_u32(tmem_slot), 512); tmem_relinquish_pair(); }
        else     { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if (TWO) cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) PARK_STAMP(1);

    const int mn_tiles = p.m_tiles * p.n_tiles;  // TWO: m_tiles counts 256-row tiles of the pair
    const int total_tiles = mn_tiles * p.splits;
    const int cta_first = TWO ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int cta_step = TWO ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (warp == 0) {
        producer_role<BN, STAGES, Cfg::STAGE_BYTES, TWO>(smem, full_bar, empty_bar, &tmA, &tmB, p, abort_flag);
        __syncwarp();  // reach the teardown's block-wide barrier as a converged warp
    } else if (warp == 1) {
        if (rank == 0)
            mma_role<BN, STAGES, Cfg::STAGE_BYTES, true, TWO>(smem, full_bar, empty_bar, tfull_bar, nullptr, tmem_base, p, abort_flag);
        __syncwarp();
    } else {
        // Work units of the epilogue: (tile of this CTA, 128-column group); the two warpgroups take
        // alternate units, the same ones in both passes.
        const int grp = (warp - 2) >> 2;
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        const int bar_id = EPI_BARRIER + grp;
        constexpr int CG = BN / 128;
        int my_tiles = 0;
        for (int tile = cta_first; tile < total_tiles; tile += cta_step) ++my_tiles;
        const int units = my_tiles * CG;

        // Everything about this warpgroup's (at most two) units that does not depend on the accumulators is worked out
        // now, while the main loop runs: tile coordinates, the row this thread owns, tensor-memory address.
        constexpr int MAX_UNITS = 2;  // tiles per CTA <= 512 / BN, 128-column groups per tile = BN / 128, two warpgroups
        RowInfo u_ri[MAX_UNITS]; int u_col[MAX_UNITS], u_it[MAX_UNITS]; uint32_t u_taddr[MAX_UNITS]; bool u_live[MAX_UNITS];
#pragma unroll
        for (int k = 0; k < MAX_UNITS; ++k) {
            const int u = grp + 2 * k;
            u_live[k] = u < units;
            u_it[k] = 0; u_col[k] = 0; u_taddr[k] = 0; u_ri[k] = RowInfo{false, 0, 0, 0, 0, -1};
            if (u_live[k]) {
                const int it = u / CG, g0 = (u % CG) * 128;
                const int tile = cta_first + it * cta_step;
                const int mn = tile % mn_tiles, n_t = mn % p.n_tiles;
                const int m_t = TWO ? 2 * (mn / p.n_tiles) + static_cast<int>(rank) : mn / p.n_tiles;
                u_ri[k] = row_info(p, m_t, tile / mn_tiles, row_in_tile);
                u_it[k] = it;
                u_col[k] = n_t * BN + g0;
                // the ReLU mask this row will be gated with after the main loop: start moving it towards the L2 now
                if (p.mask != nullptr && u_ri[k].valid && u_col[k] < p.N) prefetch_l2(p.mask + u_ri[k].row_lin * p.N + u_col[k]);
                u_taddr[k] = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + it * BN + g0;
            }
        }

        // ---- pass 1: max|acc| of this CTA's tiles (the load of the next 32-column chunk is in flight while this one is reduced)
        int vmax[4] = {0, 0, 0, 0}, vmin[4] = {0, 0, 0, 0};
        bool ok = true;
#pragma unroll
        for (int k = 0; k < MAX_UNITS; ++k) {
            if (!u_live[k] || !ok) continue;
            const uint32_t failed = mbar_wait(smem_u32(&tfull_bar[u_it[k]]), 0, abort_flag) ? 0u : 1u;
            if (barrier_or(bar_id, 128, failed)) { if (failed) report_abort(p.status, 4, 2); ok = false; continue; }
            if (threadIdx.x == 64 && k == 0) PARK_STAMP(4);
            tc_fence_after();
            const int cols = p.N - u_col[k];
            if (cols <= 0) continue;
            const int nch = cols >= 128 ? 4 : (cols + 31) >> 5;
            uint32_t va[32], vb[32];
            tmem_ld_32x32(u_taddr[k], va);
#pragma unroll 1
            for (int j = 0; j < nch; j += 2) {
                tmem_ld_wait();
                if (j + 1 < nch) tmem_ld_32x32(u_taddr[k] + (j + 1) * 32, vb);
                if (u_ri[k].valid) minmax32(va, cols - 32 * j, vmax, vmin);
                tmem_ld_wait();
                if (j + 2 < nch) tmem_ld_32x32(u_taddr[k] + (j + 2) * 32, va);
                if (j + 1 < nch && u_ri[k].valid) minmax32(vb, cols - 32 * (j + 1), vmax, vmin);
            }
        }
        unsigned local_max = __reduce_max_sync(0xFFFFFFFFu, fold_minmax(vmax, vmin));
        int32_t* st = p.state;
        if (lane == 0) warp_max[warp - 2] = local_max;
        if (threadIdx.x == 64) PARK_STAMP(5);

        // ---- grid barrier: every CTA has contributed its maximum (one atomic each: atomics on one address
        //      serialise at the L2; the waiters poll with plain acquire loads for the same reason)
        named_barrier(EPI_BARRIER + 2, 256);
        if (threadIdx.x == 64) {
            unsigned cta_max = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) cta_max = max(cta_max, warp_max[i]);
            // The maximum and the arrival count sit side by side (st[6], st[7]): two fire-and-forget reductions on the
            // way in (the count's release orders the maximum before it), ONE 64-bit acquire load per poll that returns
            // both -- a fence + atomicAdd + atomicMax read-back would add three round trips to the L2.
            if (cta_max != 0) red_relaxed_max(reinterpret_cast<unsigned*>(&st[6]), cta_max);
            red_release_add(&st[7], 1);
            const unsigned long long t0 = global_timer_ns();
            bool arrived = false;
            unsigned m = 0;
            for (unsigned spin = 0;; ++spin) {
                const unsigned long long both = ld_acquire_gpu_u64(&st[6]);
                if (static_cast<int>(both >> 32) >= static_cast<int>(gridDim.x)) { arrived = true; m = static_cast<unsigned>(both); break; }
                if ((spin & 63) == 63) {
                    if (*abort_flag || global_timer_ns() - t0 > GRID_BARRIER_LIMIT_NS) break;
                }
            }
            bool zero_out;
            *shift_slot = arrived ? shift_for(m, p.kind, p.target_bits, &zero_out) : -1;
            if (!arrived) { *abort_flag = 1; report_abort(p.status, 5, 2); }
        }
        named_barrier(EPI_BARRIER + 2, 256);
        const int shift = *shift_slot;
        if (threadIdx.x == 64) PARK_STAMP(6);

        // ---- pass 2: narrow the parked accumulators with the true shift
        if (ok && shift >= 0) {
            unsigned long long seed = 0;
            if (p.mode == ROUND_STOCHASTIC && shift > 0) seed = *p.seed;
#pragma unroll
            for (int k = 0; k < MAX_UNITS; ++k) {
                const int cols = p.N - u_col[k];
                if (!u_live[k] || cols <= 0) continue;
                const RowInfo ri = u_ri[k];
                const int col = u_col[k];
                const uint32_t taddr = u_taddr[k];
                const int nch = cols >= 128 ? 4 : (cols + 31) >> 5;  // the store clips the columns beyond
                const unsigned long long e0 = p.rng_offset + static_cast<unsigned long long>(ri.row_lin) * p.N + col;
                const int8_t* mrow = (p.mask != nullptr && ri.valid) ? p.mask + ri.row_lin * p.N + col : nullptr;
                // Each thread writes its own row straight from registers (32-byte pieces = whole L2 sectors): with one
                // or two units per warpgroup there is nothing for a staged TMA store to overlap with, and its fence,
                // barriers and the wait for the store engine at the end of the kernel cost more than the stores.
                int8_t* orow = ri.valid ? p.out8 + ri.row_lin * p.N + col : nullptr;
                // Max pooling in the same pass (TiMaxpool2d.forward): a warp's 32 rows are whole image rows of the tile
                // (BW is a power of two <= 16, BH even), so the 2x2 window of lane l is lanes l, l^1, l^BW, l^BW^1:
                // two shuffles and two byte-wise maxima per word, and the window's top-left lane stores the pooled piece.
                const bool pooling = p.pool_out != nullptr;  // the same for the whole grid
                int8_t* prow = (pooling && ri.valid && ri.pool_row >= 0) ? p.pool_out + ri.pool_row * p.N + col : nullptr;
                uint32_t va[32], vb[32], packed[8];
                uint4 ma[2], mb[2];  // the mask pieces of the chunk in va / vb, fetched one chunk ahead of their use
                tmem_ld_32x32(taddr, va);
                mask_load<2>(mrow, cols, ma);
#pragma unroll 1
                for (int j = 0; j < nch; j += 2) {
                    tmem_ld_wait();
                    if (j + 1 < nch) { tmem_ld_32x32(taddr + (j + 1) * 32, vb); mask_load<2>(mrow == nullptr ? nullptr : mrow + 32 * (j + 1), cols - 32 * (j + 1), mb); }
                    narrow32(va, packed, shift, p.mode, p.relu, seed, p.rng_stream, e0 + 32 * j);
                    mask_apply<2>(packed, mrow, cols - 32 * j, ma);
                    store_piece(orow, 32 * j, cols, packed);
                    if (pooling) { pool_window(packed, p.BW); store_piece(prow, 32 * j, cols, packed); }
                    tmem_ld_wait();
                    if (j + 2 < nch) { tmem_ld_32x32(taddr + (j + 2) * 32, va); mask_load<2>(mrow == nullptr ? nullptr : mrow + 32 * (j + 2), cols - 32 * (j + 2), ma); }
                    if (j + 1 < nch) {
                        narrow32(vb, packed, shift, p.mode, p.relu, seed, p.rng_stream, e0 + 32 * (j + 1));
                        mask_apply<2>(packed, mrow, cols - 32 * (j + 1), mb);
                        store_piece(orow, 32 * (j + 1), cols, packed);
                        if (pooling) { pool_window(packed, p.BW); store_piece(prow, 32 * (j + 1), cols, packed); }
                    }
                }
            }
        }
        if (threadIdx.x == 64) PARK_STAMP(7);
        // ---- the CTA that leaves last publishes the shift and clears the words for the next call
        named_barrier(EPI_BARRIER + 2, 256);
        if (threadIdx.x == 64) {
            if (atomicAdd(&st[4], 1) == static_cast<int>(gridDim.x) - 1) {
                __threadfence();
                const int s_out = shift < 0 ? 0 : shift;
                st[0] = s_out; st[2] = 0; st[1] = 0; st[5] = 0; st[4] = 0; st[6] = 0; st[7] = 0;
                if (p.exp_out) *p.exp_out = s_out + (p.exp_a ? *p.exp_a : 0) + (p.exp_b ? *p.exp_b : 0);
                if (p.shift_out) *p.shift_out = s_out;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) PARK_STAMP(8);
    if (TWO) cluster_sync_all();
    if (warp == 1) {
        if (*abort_flag) __nanosleep(200000);
        tc_fence_after();
        __syncwarp();
        if (TWO) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
    }
}
#ifdef NITI_PARKED_TIMING
}  // namespace niti
extern "C" __attribute__((visibility("default"))) int niti_debug_stamps(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, niti::g_dbg_stamps, sizeof(niti::g_dbg_stamps)) == cudaSuccess ? 0 : -3;
}
namespace niti {
#endif

// ------------------------------------------------------------------------------------------------
// Convolution weight gradient: g[k][r][s][c] = sum_pixels err[pixel][k] * x[pixel + (r,s) - pad][c]
// A = err tile (MN-major: 128 k-channels x <=128 pixels), B = shifted x tile (MN-major:
// 128 c-channels x the same pixels).  One CTA owns (128 k) x (128 c) x (one filter row r, all S
// taps) and a contiguous range of pixel chunks; its S accumulators live in TMEM side by side.
// Partial sums are written to scratch[split] and folded by wgrad_reduce_kernel.
// ------------------------------------------------------------------------------------------------
struct WgradParams {
    int H, W, C, K, R, S, pad, Nimg;
    int BW, BH, BI;
    int tiles_w, tiles_h, tiles_n;
    int chunks, splits;
    int k_tiles, c_tiles;
    int box_bytes;         // bytes of one TMA box (BW*BH*BI rows of 128 bytes)
    int mma_per_chunk;     // ceil(rows / 32)
    int32_t* partial;      // [splits][K*R*S*C]
    int32_t* status;
    int reduce_direct;     // 1: every CTA adds its tiles straight into the (zeroed) gradient with TMA reductions
};

constexpr int WG_MAX_S = 3;
constexpr int WG_STAGE_BYTES = (1 + WG_MAX_S) * PANEL_BYTES;  // 64 KB
constexpr int WG_STAGES = 3;
constexpr int WG_SMEM_BYTES = WG_STAGES * WG_STAGE_BYTES + 1024 + 256;
constexpr int WG_TMEM_COLS = 512;

// One CTA's share of one layer's weight gradient: work item `item` (filter row, k tile, c tile) over the pixel chunks of
// split `split`.  The tensor maps live in kernel parameter space (grid constants of the calling kernel).
__device__ __forceinline__ void wgrad_body(const CUtensorMap& tmErr, const CUtensorMap& tmX, const CUtensorMap& tmP,
                                           const WgradParams& p, const int split, const int item, const bool probe_cta) {
    if (threadIdx.x == 0 && probe_cta) PARK_STAMP(10);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WG_STAGES * WG_STAGE_BYTES);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + WG_STAGES;
    uint64_t* tfull_bar = bars + 2 * WG_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * WG_STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // Rows past the box (when a tile holds fewer than 128 pixels) are read by the MMA as part of
    // the reduction: they must be zero.  TMA only ever writes the first box_bytes of a panel.
    if ((p.box_bytes / ROW_BYTES) % 32 != 0) {  // full 32-row slabs leave nothing unwritten for the MMAs to read
        int4* z = reinterpret_cast<int4*>(smem);
        for (int i = threadIdx.x; i < WG_STAGES * WG_STAGE_BYTES / 16; i += UMMA_THREADS) z[i] = make_int4(0, 0, 0, 0);
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < WG_STAGES; ++i) { mbar_init(smem_u32(&full_bar[i]), 1); mbar_init(smem_u32(&empty_bar[i]), 1); }
        mbar_init(smem_u32(&tfull_bar[0]), 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmErr);
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmP);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), WG_TMEM_COLS); tmem_relinquish(); }
    fence_proxy_async();  // zero fill (generic proxy) before TMA writes (async proxy)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0 && probe_cta) PARK_STAMP(11);

    const int r = item % p.R;
    const int kt = (item / p.R) % p.k_tiles;
    const int ct = item / (p.R * p.k_tiles);
    const int chunk_lo = static_cast<int>(static_cast<long long>(split) * p.chunks / p.splits);
    const int chunk_hi = static_cast<int>(static_cast<long long>(split + 1) * p.chunks / p.splits);

    // Warps 0 and 1 run their loops whole, with warp-uniform control flow (see producer_role); an elected lane issues.
    const uint32_t abort_addr = smem_u32(const_cast<int*>(abort_flag));
    const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    const int S = keep_reg(p.S);
    if (warp == 0) {
        {
            const int pad = keep_reg(p.pad), BW = keep_reg(p.BW), BH = keep_reg(p.BH), BI = keep_reg(p.BI);
            const int tiles_w = keep_reg(p.tiles_w), tiles_h = keep_reg(p.tiles_h);
            const uint32_t tx_bytes = static_cast<uint32_t>(keep_reg((1 + p.S) * p.box_bytes));
            int s = 0; uint32_t ph = 0;
            // tile coordinates as running counters: this instruction stream paces the pipeline
            int tw = chunk_lo % p.tiles_w, th = (chunk_lo / p.tiles_w) % p.tiles_h, tn = chunk_lo / (p.tiles_w * p.tiles_h);
            for (int ch = chunk_lo; ch < chunk_hi; ++ch) {
                if (!mbar_wait_uniform(empty0 + 8u * s, ph ^ 1u, abort_addr)) { *abort_flag = 1; report_abort(p.status, 11, 0); break; }
                const uint32_t fb = full0 + 8u * s;
                const uint32_t sa = smem0 + static_cast<uint32_t>(s) * WG_STAGE_BYTES;
                if (elect_one()) {
                    mbar_arrive_expect_tx(fb, tx_bytes);
                    tma_load_4d(sa, &tmErr, fb, kt * 128, tw * BW, th * BH, tn * BI);
                    for (int sx = 0; sx < S; ++sx)
                        tma_load_4d(sa + (1 + sx) * PANEL_BYTES, &tmX, fb, ct * 128, tw * BW + sx - pad, th * BH + r - pad, tn * BI);
                }
                if (++s == WG_STAGES) { s = 0; ph ^= 1u; }
                if (++tw == tiles_w) { tw = 0; if (++th == tiles_h) { th = 0; ++tn; } }
            }
        }
        __syncwarp();  // reach the teardown's block-wide barrier as a converged warp
    } else if (warp == 1) {
        {
            const uint32_t idesc = make_idesc_i8(BLOCK_M, 128, 1, 1);
            const uint32_t idesc2 = make_idesc_i8(BLOCK_M, 256, 1, 1);
            const uint32_t tm = __shfl_sync(0xFFFFFFFFu, tmem_base, 0);
            const int nmma = keep_reg(p.mma_per_chunk);
            const uint64_t kstep = (32u * ROW_BYTES) >> 4;  // 32 reduction rows per MMA, in descriptor units
            const uint64_t d0 = make_smem_desc(smem0, PANEL_BYTES, 1024, SWIZZLE_128B_CODE);
            int s = 0; uint32_t ph = 0; bool ok = true;
            bool ready = false;  // the stage's "full" phase was seen complete by the previous chunk's probe
            for (int ch = chunk_lo; ch < chunk_hi; ++ch) {
                if (!ready && !mbar_wait_uniform(full0 + 8u * s, ph, abort_addr)) { ok = false; *abort_flag = 1; report_abort(p.status, 13, 1); break; }
                if (ch == chunk_lo && probe_cta) PARK_STAMP(12);
                const uint64_t a0 = d0 + ((static_cast<uint32_t>(s) * WG_STAGE_BYTES) >> 4);
                const uint32_t first = static_cast<uint32_t>(ch != chunk_lo);
                const int sn = (s + 1 == WG_STAGES) ? 0 : s + 1;
                const uint32_t phn = (sn == 0) ? ph ^ 1u : ph;
                const uint32_t eb = empty0 + 8u * s;
                // The taps' x tiles lie one panel apart, which is exactly the layout of an MN-major B operand of
                // two 128-column panels: two taps go through ONE 256-column MMA (half as many instructions to issue),
                // accumulating into the adjacent TMEM column blocks of the two taps.
                uint32_t probe;
                if (nmma == 4 && S == 3) {
                    umma_seq4(tm, a0, a0 + (PANEL_BYTES >> 4), kstep, kstep, idesc2, first);
                    probe = umma_block4<false>(tm + 256, a0, a0 + ((3 * PANEL_BYTES) >> 4), kstep, kstep, idesc, first, eb, full0 + 8u * sn, phn);
                } else {
                    if (elect_one()) {
                        int sx = 0;
                        for (; sx + 1 < S; sx += 2)
                            for (int k = 0; k < nmma; ++k)
                                umma_i8(tm + sx * 128, a0 + k * kstep, a0 + (((1 + sx) * PANEL_BYTES) >> 4) + k * kstep, idesc2,
                                        static_cast<uint32_t>(ch != chunk_lo || k != 0));
                        for (; sx < S; ++sx)
                            for (int k = 0; k < nmma; ++k)
                                umma_i8(tm + sx * 128, a0 + k * kstep, a0 + (((1 + sx) * PANEL_BYTES) >> 4) + k * kstep, idesc,
                                        static_cast<uint32_t>(ch != chunk_lo || k != 0));
                        umma_commit(eb);
                    }
                    probe = mbar_test_wait(full0 + 8u * sn, phn);
                }
                ready = __all_sync(0xFFFFFFFFu, probe != 0);
                s = sn; ph = phn;
            }
            if (ok && elect_one()) umma_commit(smem_u32(&tfull_bar[0]));
            if (probe_cta) PARK_STAMP(13);
        }
        __syncwarp();
    } else {
        // partial[split][k][r][s][c] viewed as a rank-4 tensor (c, r*S+s, k, split): per tap, four TMA
        // stores of 128 k-rows x 32 channels.  Once the last MMA has completed the operand stages
        // are dead, so stage `sx` serves as the staging area of tap `sx` (64 KB = 4 tiles each) and
        // no store ever waits for another.
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        const bool leader = threadIdx.x == 64;
        const uint32_t failed = mbar_wait(smem_u32(&tfull_bar[0]), 0, abort_flag) ? 0u : 1u;
        if (barrier_or(EPI_BARRIER, 128, failed)) {
            if (failed) report_abort(p.status, 14, 2);
        } else {
            tc_fence_after();
            if (leader && probe_cta) PARK_STAMP(14);
            for (int sx = 0; sx < p.S; ++sx) {
                const uint32_t buf = smem_u32(smem + sx * WG_STAGE_BYTES);
                uint32_t v[4][32];
#pragma unroll
                for (int j = 0; j < 4; ++j) tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + sx * 128 + j * 32, v[j]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) stage_row(buf + j * EPI_CHUNK_BYTES, row_in_tile, v[j]);
                fence_proxy_async();
                named_barrier(EPI_BARRIER, 128);
                if (leader) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (ct * 128 + j * 32 < p.C) {
                            if (p.reduce_direct) tma_reduce_add_4d(&tmP, buf + j * EPI_CHUNK_BYTES, ct * 128 + j * 32, r * p.S + sx, kt * 128, 0);
                            else tma_store_4d(&tmP, buf + j * EPI_CHUNK_BYTES, ct * 128 + j * 32, r * p.S + sx, kt * 128, split);
                        }
                    bulk_commit();
                }
            }
            if (leader && probe_cta) PARK_STAMP(15);
            if (leader) bulk_wait_read<0>();
            if (leader && probe_cta) PARK_STAMP(16);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*abort_flag) __nanosleep(200000);
        tc_fence_after();
        __syncwarp();
        tmem_dealloc(tmem_base, WG_TMEM_COLS);
    }
}

__global__ void __launch_bounds__(UMMA_THREADS, 1)
umma_wgrad_kernel(const __grid_constant__ CUtensorMap tmErr, const __grid_constant__ CUtensorMap tmX,
                  const __grid_constant__ CUtensorMap tmP, const __grid_constant__ WgradParams p) {
    wgrad_body(tmErr, tmX, tmP, p, blockIdx.x, blockIdx.y, blockIdx.y == 0);
}

// Several layers' weight gradients in ONE launch: CTAs [first_cta[l], first_cta[l + 1]) belong to layer l, split-major
// inside.  The host picks the splits so that every CTA of the launch walks about the same number of pixel chunks: a
// step's layers come in pairs of equal work (256->512 and 512->512 at 8x8, ...), which then fill one wave exactly and
// pay the launch, the prologue and the accumulator flush once instead of twice.
constexpr int WG_MULTI_MAX = 4;
struct WgradMultiMaps { CUtensorMap err[WG_MULTI_MAX], x[WG_MULTI_MAX], g[WG_MULTI_MAX]; };
struct WgradMultiParams { WgradParams layer[WG_MULTI_MAX]; int first_cta[WG_MULTI_MAX + 1]; int count; };
__global__ void __launch_bounds__(UMMA_THREADS, 1)
umma_wgrad_multi_kernel(const __grid_constant__ WgradMultiMaps maps, const __grid_constant__ WgradMultiParams mp) {
    int l = 0;
    while (l + 1 < mp.count && static_cast<int>(blockIdx.x) >= mp.first_cta[l + 1]) ++l;
    const int local = static_cast<int>(blockIdx.x) - mp.first_cta[l];
    const WgradParams& p = mp.layer[l];
    wgrad_body(maps.err[l], maps.x[l], maps.g[l], p, local % p.splits, local / p.splits, blockIdx.x == 0);
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// Tensor map with 128-byte swizzle over uint8 (operands) or int32 (outputs) elements; dims/box
// innermost first, in elements; strides of dims 1.. in bytes.
static int encode_map(CUtensorMap* map, const void* ptr, bool int32_elems, int rank, const uint64_t* dims,
                      const uint64_t* strides, const uint32_t* box) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return set_cuda_error_text("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t gdim[4]; cuuint64_t gstr[3]; cuuint32_t bx[4]; cuuint32_t es[4];
    for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides[i];
    CUresult r = enc(map, int32_elems ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8, rank,
                     const_cast<void*>(ptr), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[160];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d)", static_cast<int>(r), rank);
        return set_cuda_error_text(buf);
    }
    return 0;
}

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <int BN, bool FUSED>
static int launch_gemm_inst(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const GemmParams& p,
                            cudaStream_t st) {
    using Cfg = GemmCfg<BN, FUSED, false>;
    cudaError_t e = cudaFuncSetAttribute(umma_gemm_kernel<BN, FUSED, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return set_cuda_error(e);
    int grid = p.m_tiles * p.n_tiles * p.splits;
    if (grid > sm_count()) grid = sm_count();
    umma_gemm_kernel<BN, FUSED, false><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(a, b, c, p);
    return set_cuda_error(cudaGetLastError());
}
// CTA pairs: clusters of two CTAs, p.m_tiles counts 256-row tiles
template <int BN, bool FUSED>
static int launch_gemm_pair_inst(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const GemmParams& p,
                                 cudaStream_t st) {
    using Cfg = GemmCfg<BN, FUSED, true>;
    cudaError_t e = cudaFuncSetAttribute(umma_gemm_kernel<BN, FUSED, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return set_cuda_error(e);
    int pairs = p.m_tiles * p.n_tiles * p.splits;
    if (pairs > sm_count() / 2) pairs = sm_count() / 2;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(GEMM_THREADS); cfg.dynamicSmemBytes = Cfg::SMEM_BYTES; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return set_cuda_error(cudaLaunchKernelEx(&cfg, umma_gemm_kernel<BN, FUSED, true>, a, b, c, p));
}
static int launch_gemm(int bn, bool fused, bool pair, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c,
                       const GemmParams& p, cudaStream_t st) {
    if (pair) {
        if (fused) return bn == 256 ? launch_gemm_pair_inst<256, true>(a, b, c, p, st) : launch_gemm_pair_inst<128, true>(a, b, c, p, st);
        return bn == 256 ? launch_gemm_pair_inst<256, false>(a, b, c, p, st) : launch_gemm_pair_inst<128, false>(a, b, c, p, st);
    }
    if (fused) return bn == 256 ? launch_gemm_inst<256, true>(a, b, c, p, st) : launch_gemm_inst<128, true>(a, b, c, p, st);
    return bn == 256 ? launch_gemm_inst<256, false>(a, b, c, p, st) : launch_gemm_inst<128, false>(a, b, c, p, st);
}
// CTA pairs (M = 256 MMAs, B operand split between the two CTAs): bit 0 enables them for GEMMs, bit 1 for
// convolutions.  Measured on B200: +20 % on large GEMMs (2.2 -> 2.7 POP/s at 8192^3), nothing on the
// convolutions (their A tiles are re-read per filter tap and dominate), hence the default.
int g_two_cta = 1;
// a pair needs two 128-row tiles to share a B tile; an MN-major B splits only at 128-column panels
static bool pair_ok(int m_tiles, int bn, int b_mn, int conv) {
    return (g_two_cta & (conv ? 2 : 1)) && m_tiles >= 2 && (!b_mn || bn == 256);
}
template <int BN, bool TWO>
static int launch_parked_inst(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const GemmParams& p,
                              cudaStream_t st) {
    using Cfg = ParkedCfg<BN, TWO>;
    cudaError_t e = cudaFuncSetAttribute(umma_parked_kernel<BN, TWO>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return set_cuda_error(e);
    int grid = p.m_tiles * p.n_tiles * p.splits;  // TWO: pairs
    if (TWO) { if (grid > sm_count() / 2) grid = sm_count() / 2; grid *= 2; }
    else if (grid > sm_count()) grid = sm_count();
    // cooperative launch: the grid barrier inside needs every CTA resident at the same time
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GEMM_THREADS); cfg.dynamicSmemBytes = Cfg::SMEM_BYTES; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = g_cooperative;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = TWO ? 2 : 1;
    return set_cuda_error(cudaLaunchKernelEx(&cfg, umma_parked_kernel<BN, TWO>, a, b, c, p));
}
// all accumulators of the problem fit in the tensor memory of one wave of CTAs (units: 128-row tiles,
// or 256-row pair tiles on sm/2 pairs)
static bool fits_parked(int bn, int tiles, bool pair) { return tiles <= (pair ? sm_count() / 2 : sm_count()) * (512 / bn); }

// Output tile width: 256 columns halve the A-operand traffic, but when that leaves fewer tiles than
// half the SMs, 128-column tiles put twice as many SMs to work.
static int pick_bn(int m_tiles, int n_cols) {
    if (n_cols <= 128) return 128;
    const int tiles256 = m_tiles * ((n_cols + 255) / 256);
    return tiles256 * 2 <= sm_count() ? 128 : 256;
}

int g_stage_cap = 0;  // 0: use every compiled stage
// 1: kernels with a grid barrier are launched cooperatively (the driver guarantees that all their blocks are
// resident together).  0: plain launches of grids that fit the device in one wave; co-residency then rests on
// nothing else occupying the SMs, and a barrier that is not met ends in the bounded wait's error status.
int g_cooperative = 1;

static void finish_params(GemmParams* p) {
    p->fd_mn = make_fastdiv(p->m_tiles * p->n_tiles); p->fd_n = make_fastdiv(p->n_tiles);
    p->fd_tw = make_fastdiv(p->tiles_w); p->fd_th = make_fastdiv(p->tiles_h);
}

static void set_fused(GemmParams* p, const FusedArgs* f) {
    p->nstages = g_stage_cap;
    if (!f) return;
    p->state = f->state; p->only_if_redo = f->only_if_redo; p->mode = f->mode; p->relu = f->relu;
    p->seed = f->seed; p->rng_stream = f->rng_stream; p->rng_offset = f->rng_offset;
    p->kind = f->kind; p->target_bits = f->target_bits;
    p->exp_a = f->exp_a; p->exp_b = f->exp_b; p->exp_out = f->exp_out; p->shift_out = f->shift_out;
    p->mask = f->relu_mask;
    p->pool_out = nullptr;
    p->out8 = nullptr;
    p->side = static_cast<uint32_t*>(f->side);
    // max|acc| lives in state[1]; a redo launch must leave it alone (the last CTA of the first launch zeroed it)
    p->maxabs = f->only_if_redo ? nullptr : reinterpret_cast<unsigned*>(f->state + 1);
}

// Pixels of one 128-row tile: as much of a row as fits, then rows, then images.
static void pick_pixel_box(int Nimg, int H, int W, int* BW, int* BH, int* BI) {
    *BW = W < 128 ? W : 128;
    int bh = 128 / *BW; if (bh > H) bh = H; if (bh < 1) bh = 1;
    *BH = bh;
    int bi = 128 / (*BW * *BH); if (bi > Nimg) bi = Nimg; if (bi < 1) bi = 1;
    *BI = bi;
}

static bool pool_box_ok(int H, int W, int bw, int bh);

int umma_gemm_splits(int M, int N, int K) {
    const int bn = (N > 128) ? 256 : 128;
    const int tiles = ((M + 127) / 128) * ((N + bn - 1) / bn);
    const int kb = (K + 127) / 128;
    if (tiles * 2 > sm_count() || kb < 8) return 1;
    int splits = sm_count() / tiles;
    if (splits > kb / 2) splits = kb / 2;
    return splits < 1 ? 1 : splits;
}

// out[splits][M][N] (splits == 1: the result itself) = op(A) * op(B) over disjoint reduction ranges.
// `fused` == null: int32 out; otherwise int8 out narrowed by the shift in fused->state[0] (splits must be 1).
int umma_gemm(const int8_t* A, const int8_t* B, void* out, unsigned* maxabs, int M, int N, int K, int trans_a,
              int trans_b, int splits, const FusedArgs* fused, int32_t* status, cudaStream_t st) {
    CUtensorMap ma, mb, mc;
    const int a_mn = trans_a ? 1 : 0, b_mn = trans_b ? 0 : 1;
    const int bn = (N > 128) ? 256 : 128;
    const bool pair = pair_ok((M + 127) / 128, bn, b_mn, 0);
    {
        uint64_t dims[2], str[1]; uint32_t box[2] = {128, 128};
        if (a_mn) { dims[0] = M; dims[1] = K; str[0] = M; } else { dims[0] = K; dims[1] = M; str[0] = K; }
        if (int e = encode_map(&ma, A, false, 2, dims, str, box)) return e;
        if (b_mn) { dims[0] = N; dims[1] = K; str[0] = N; box[1] = 128; } else { dims[0] = K; dims[1] = N; str[0] = K; box[1] = pair ? bn / 2 : bn; }
        if (int e = encode_map(&mb, B, false, 2, dims, str, box)) return e;
        const uint64_t es = fused ? 1 : 4;
        uint64_t dc[4] = {(uint64_t)N, (uint64_t)M, (uint64_t)splits, 1};
        uint64_t sc[3] = {(uint64_t)N * es, (uint64_t)M * N * es, (uint64_t)splits * M * N * es};
        uint32_t bc[4] = {fused ? 128u : 32u, 128, 1, 1};
        if (int e = encode_map(&mc, out, !fused, 4, dc, sc, bc)) return e;
    }
    GemmParams p{};
    p.conv = 0; p.M = M; p.N = N; p.num_kb = (K + 127) / 128; p.splits = splits;
    p.m_tiles = (M + 127) / 128; p.n_tiles = (N + bn - 1) / bn;
    if (pair) p.m_tiles = (p.m_tiles + 1) / 2;
    p.a_mn = a_mn; p.b_mn = b_mn; p.a_bytes = PANEL_BYTES;
    p.maxabs = splits > 1 ? nullptr : maxabs; p.status = status;
    p.split_cols = (bn == 256 && p.m_tiles * p.n_tiles * splits <= 2 * (pair ? sm_count() / 2 : sm_count())) ? 1 : 0;
    // operands beyond ~half of the 126 MB L2: order the tiles in compact groups
    p.group_m = (static_cast<long long>(M) + N) * K > (48ll << 20) ? 8 : 0;
    set_fused(&p, fused);
    finish_params(&p);
    return launch_gemm(bn, fused != nullptr, pair, ma, mb, mc, p, st);
}

// Forward convolution (flip == 0: x [N,H,W,C] with w [K,R,S,C] -> [N,H,W,K]) or error-backward
// (flip == 1: err [N,H,W,K] with the same w -> [N,H,W,C]); "same" padding, stride 1.
// Forward reads w rows as the N operand (K-major); backward reads the very same tensor as the
// reduction operand (MN-major: 128 k rows of 128 c bytes per tap), so no transposed copy exists.
int umma_conv(const int8_t* x, const int8_t* w, void* out, unsigned* maxabs, int Nimg, int H, int W, int C, int K,
              int R, int S, int pad, int flip, const FusedArgs* fused, int32_t* status, cudaStream_t st) {
    CUtensorMap ma, mb, mc;
    const int red = flip ? K : C;   // reduction channels per tap
    const int outc = flip ? C : K;  // output channels
    GemmParams p{};
    pick_pixel_box(Nimg, H, W, &p.BW, &p.BH, &p.BI);
    const int all_m_tiles = ((W + p.BW - 1) / p.BW) * ((H + p.BH - 1) / p.BH) * ((Nimg + p.BI - 1) / p.BI);
    const int bn = pick_bn(all_m_tiles, outc);
    const bool parked = fused && fused->parked;
    const bool pair = pair_ok(all_m_tiles, bn, flip ? 1 : 0, 1);
    {
        uint64_t dims[4] = {(uint64_t)red, (uint64_t)W, (uint64_t)H, (uint64_t)Nimg};
        uint64_t str[3] = {(uint64_t)red, (uint64_t)W * red, (uint64_t)H * W * red};
        uint32_t box[4] = {128, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
        if (int e = encode_map(&ma, x, false, 4, dims, str, box)) return e;
        uint64_t d2[2] = {(uint64_t)R * S * C, (uint64_t)K};
        uint64_t s2[1] = {(uint64_t)R * S * C};
        uint32_t b2[2] = {128, flip ? 128u : (uint32_t)(pair ? bn / 2 : bn)};
        if (int e = encode_map(&mb, w, false, 2, d2, s2, b2)) return e;
        const uint64_t es = fused ? 1 : 4;
        uint64_t dc[4] = {(uint64_t)outc, (uint64_t)W, (uint64_t)H, (uint64_t)Nimg};
        uint64_t sc[3] = {(uint64_t)outc * es, (uint64_t)W * outc * es, (uint64_t)H * W * outc * es};
        uint32_t bc[4] = {fused ? 128u : 32u, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
        if (int e = encode_map(&mc, out, !fused, 4, dc, sc, bc)) return e;
    }
    p.conv = 1; p.flip = flip; p.splits = 1;
    p.H = H; p.W = W; p.S = S; p.pad = pad; p.Nimg = Nimg; p.tapstride = C;
    p.tiles_w = (W + p.BW - 1) / p.BW; p.tiles_h = (H + p.BH - 1) / p.BH;
    const int tiles_n = (Nimg + p.BI - 1) / p.BI;
    p.cblocks = (red + 127) / 128; p.red = red;
    p.M = Nimg * H * W; p.N = outc; p.num_kb = R * S * p.cblocks;
    p.m_tiles = p.tiles_w * p.tiles_h * tiles_n; p.n_tiles = (outc + bn - 1) / bn;
    if (pair) p.m_tiles = (p.m_tiles + 1) / 2;
    p.a_mn = 0; p.b_mn = flip ? 1 : 0; p.a_bytes = p.BW * p.BH * p.BI * ROW_BYTES;
    p.maxabs = maxabs; p.status = status;
    p.split_cols = (bn == 256 && p.m_tiles * p.n_tiles <= 2 * (pair ? sm_count() / 2 : sm_count())) ? 1 : 0;
    set_fused(&p, fused);
    finish_params(&p);
    if (fused) p.out8 = static_cast<int8_t*>(out);
    if (fused && fused->pool_out != nullptr) {
        if (!parked || flip || !pool_box_ok(H, W, p.BW, p.BH)) return NITI_ERR_UNSUPPORTED;
        p.pool_out = fused->pool_out;
    }
    if (parked) {
        if (!fits_parked(bn, p.m_tiles * p.n_tiles, pair)) return NITI_ERR_UNSUPPORTED;
        if (pair) return bn == 256 ? launch_parked_inst<256, true>(ma, mb, mc, p, st) : launch_parked_inst<128, true>(ma, mb, mc, p, st);
        return bn == 256 ? launch_parked_inst<256, false>(ma, mb, mc, p, st) : launch_parked_inst<128, false>(ma, mb, mc, p, st);
    }
    return launch_gemm(bn, fused != nullptr, pair, ma, mb, mc, p, st);
}

// the parked kernel can pool 2x2 / stride 2 in its epilogue when every window lies inside one warp's 32 rows of a tile
static bool pool_box_ok(int H, int W, int bw, int bh) {
    return H % 2 == 0 && W % 2 == 0 && bh % 2 == 0 && (bw == 2 || bw == 4 || bw == 8 || bw == 16);
}
bool umma_conv_pool_fusable(int Nimg, int H, int W, int outc) {
    int bw, bh, bi;
    pick_pixel_box(Nimg, H, W, &bw, &bh, &bi);
    return pool_box_ok(H, W, bw, bh) && umma_conv_fits_parked(Nimg, H, W, outc, 0);
}

bool umma_conv_fits_parked(int Nimg, int H, int W, int outc, int flip) {
    int bw, bh, bi;
    pick_pixel_box(Nimg, H, W, &bw, &bh, &bi);
    const int m_tiles = ((W + bw - 1) / bw) * ((H + bh - 1) / bh) * ((Nimg + bi - 1) / bi);
    const int bn = pick_bn(m_tiles, outc);
    const bool pair = pair_ok(m_tiles, bn, flip, 1);
    return fits_parked(bn, (pair ? (m_tiles + 1) / 2 : m_tiles) * ((outc + bn - 1) / bn), pair);
}

static void wgrad_plan(int Nimg, int H, int W, int C, int K, int R, int max_splits, WgradParams* p) {
    pick_pixel_box(Nimg, H, W, &p->BW, &p->BH, &p->BI);
    p->tiles_w = (W + p->BW - 1) / p->BW; p->tiles_h = (H + p->BH - 1) / p->BH; p->tiles_n = (Nimg + p->BI - 1) / p->BI;
    p->chunks = p->tiles_w * p->tiles_h * p->tiles_n;
    p->k_tiles = (K + 127) / 128; p->c_tiles = (C + 127) / 128;
    const int items = R * p->k_tiles * p->c_tiles;
    int splits = sm_count() / items;  // never more CTAs than SMs: a second wave of a few CTAs would double the time
    if (splits < 1) splits = 1;
    if (splits > p->chunks) splits = p->chunks;
    if (max_splits > 0 && splits > max_splits) splits = max_splits;
    p->splits = splits;
}

size_t umma_wgrad_scratch_bytes(int Nimg, int H, int W, int C, int K, int R, int S) {
    WgradParams p{};
    wgrad_plan(Nimg, H, W, C, K, R, 0, &p);
    return static_cast<size_t>(p.splits) * K * R * S * C * sizeof(int32_t);
}

// Tensor maps and kernel parameters of one layer; p->splits (and the rest of the plan) must already be set.
static int wgrad_setup(const int8_t* x, const int8_t* err, int32_t* out, int direct, int Nimg, int H, int W, int C, int K, int R,
                       int S, int pad, int32_t* status, WgradParams* p, CUtensorMap* me, CUtensorMap* mx, CUtensorMap* mp) {
    p->reduce_direct = direct;
    uint32_t box[4] = {128, (uint32_t)p->BW, (uint32_t)p->BH, (uint32_t)p->BI};
    uint64_t de[4] = {(uint64_t)K, (uint64_t)W, (uint64_t)H, (uint64_t)Nimg};
    uint64_t se[3] = {(uint64_t)K, (uint64_t)W * K, (uint64_t)H * W * K};
    if (int e = encode_map(me, err, false, 4, de, se, box)) return e;
    uint64_t dx[4] = {(uint64_t)C, (uint64_t)W, (uint64_t)H, (uint64_t)Nimg};
    uint64_t sx[3] = {(uint64_t)C, (uint64_t)W * C, (uint64_t)H * W * C};
    if (int e = encode_map(mx, x, false, 4, dx, sx, box)) return e;
    uint64_t dp[4] = {(uint64_t)C, (uint64_t)R * S, (uint64_t)K, (uint64_t)(direct ? 1 : p->splits)};
    uint64_t sp[3] = {(uint64_t)C * 4, (uint64_t)R * S * C * 4, (uint64_t)K * R * S * C * 4};
    uint32_t bp[4] = {32, 1, 128, 1};
    if (int e = encode_map(mp, out, true, 4, dp, sp, bp)) return e;
    p->H = H; p->W = W; p->C = C; p->K = K; p->R = R; p->S = S; p->pad = pad; p->Nimg = Nimg;
    const int rows = p->BW * p->BH * p->BI;
    p->box_bytes = rows * ROW_BYTES;
    p->mma_per_chunk = (rows + 31) / 32;
    p->partial = out; p->status = status;
    return NITI_OK;
}

// partial != null, direct == 0: CTA (split, tile) stores its sums to partial[split] (the caller folds them);
// direct == 1: `partial` is the gradient itself, zeroed by the caller, and every CTA adds into it.
int umma_conv_wgrad_partials(const int8_t* x, const int8_t* err, int32_t* partial, int* splits_out, int max_splits,
                             int Nimg, int H, int W, int C, int K, int R, int S, int pad, int32_t* status, cudaStream_t st,
                             int direct) {
    WgradParams p{};
    wgrad_plan(Nimg, H, W, C, K, R, max_splits, &p);
    CUtensorMap me, mx, mp;
    if (int e = wgrad_setup(x, err, partial, direct, Nimg, H, W, C, K, R, S, pad, status, &p, &me, &mx, &mp)) return e;
    *splits_out = p.splits;
    cudaError_t e = cudaFuncSetAttribute(umma_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM_BYTES);
    if (e != cudaSuccess) return set_cuda_error(e);
    dim3 grid(p.splits, R * p.k_tiles * p.c_tiles);
    umma_wgrad_kernel<<<grid, UMMA_THREADS, WG_SMEM_BYTES, st>>>(me, mx, mp, p);
    return set_cuda_error(cudaGetLastError());
}

int umma_wgrad_multi_max() { return WG_MULTI_MAX; }

// Up to WG_MULTI_MAX layers' gradients added into their (zeroed or accumulating) int32 buffers by one launch.
int umma_conv_wgrad_multi(const WgradJob* jobs, int count, int32_t* status, cudaStream_t st) {
    if (count < 1 || count > WG_MULTI_MAX) return NITI_ERR_BAD_ARG;
    WgradMultiParams mp{};
    WgradMultiMaps maps;
    int items[WG_MULTI_MAX];
    long long work = 0;  // item-chunks of the whole launch
    for (int l = 0; l < count; ++l) {
        const WgradJob& j = jobs[l];
        wgrad_plan(j.N, j.H, j.W, j.C, j.K, j.R, 0, &mp.layer[l]);
        items[l] = j.R * mp.layer[l].k_tiles * mp.layer[l].c_tiles;
        work += static_cast<long long>(items[l]) * mp.layer[l].chunks;
    }
    // chunks per CTA: the smallest number for which the launch still fits in one wave
    const int sms = sm_count();
    long long per_cta = (work + sms - 1) / sms;
    if (per_cta < 1) per_cta = 1;
    for (;; ++per_cta) {
        int ctas = 0;
        for (int l = 0; l < count; ++l) {
            int sp = static_cast<int>((mp.layer[l].chunks + per_cta - 1) / per_cta);
            if (sp < 1) sp = 1;
            mp.layer[l].splits = sp;
            ctas += sp * items[l];
        }
        bool whole = true;  // nothing left to merge: every layer is down to one split
        for (int l = 0; l < count; ++l) whole = whole && mp.layer[l].splits == 1;
        if (ctas <= sms || whole) break;
    }
    int grid = 0;
    for (int l = 0; l < count; ++l) {
        const WgradJob& j = jobs[l];
        if (int e = wgrad_setup(j.x, j.err, j.g32, 1, j.N, j.H, j.W, j.C, j.K, j.R, j.S, j.pad, status, &mp.layer[l], &maps.err[l],
                                &maps.x[l], &maps.g[l])) return e;
        mp.first_cta[l] = grid;
        grid += mp.layer[l].splits * items[l];
    }
    mp.first_cta[count] = grid;
    mp.count = count;
    cudaError_t e = cudaFuncSetAttribute(umma_wgrad_multi_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM_BYTES);
    if (e != cudaSuccess) return set_cuda_error(e);
    umma_wgrad_multi_kernel<<<grid, UMMA_THREADS, WG_SMEM_BYTES, st>>>(maps, mp);
    return set_cuda_error(cudaGetLastError());
}

}  // namespace niti
