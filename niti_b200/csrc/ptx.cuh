// Inline-PTX wrappers for the sm_100a features the contraction kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tensor memory (tcgen05.alloc/ld) and the
// 5th-generation tensor-core MMA (tcgen05.mma kind::i8).
//
// Every wait in this file is bounded: after WAIT_LIMIT_NS without progress the caller
// is told to give up (the kernel then records an error status and drains), so a
// protocol bug can never leave the GPU spinning.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace niti {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\t"
        "elect.sync R|P, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// Non-blocking probe of a phase: lets a loop ask about the NEXT stage before it works on the current one, so that
// the barrier's shared-memory round trip is hidden behind that work.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// Bounded wait on an mbarrier phase.  `abort_flag` is a CTA-wide word in shared memory:
// once any role gives up, every other role's wait returns false on its next poll.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 0x3FF) == 0) {
            if (*abort_flag) return false;
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
        }
    }
}

// The same bounded wait for loops whose control flow must stay warp-uniform (the TMA producer and the MMA issuer:
// their TMA / MMA instructions take operands from uniform registers, and the compiler keeps loop counters,
// addresses and descriptors there only while it can prove that every lane follows the same path).  The spin is
// inside ONE asm block, so no C++ branch depends on a per-lane value; the verdict is made warp-uniform with a
// vote.  All 32 lanes must call it.  Returns false when the limit ran out or another role raised the abort flag.
__device__ __forceinline__ bool mbar_wait_uniform(uint32_t bar, uint32_t parity, uint32_t abort_flag_smem) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred P, Q;\n\t"
        ".reg .u64 t0, t1;\n\t"
        ".reg .u32 a;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "@P bra WAIT_DONE;\n\t"
        "mov.u64 t0, %%globaltimer;\n\t"
        "WAIT_SPIN:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "@P bra WAIT_DONE;\n\t"
        "ld.volatile.shared.u32 a, [%3];\n\t"
        "setp.ne.u32 Q, a, 0;\n\t"
        "@Q bra WAIT_DONE;\n\t"
        "mov.u64 t1, %%globaltimer;\n\t"
        "sub.u64 t1, t1, t0;\n\t"
        "setp.lt.u64 Q, t1, %4;\n\t"
        "@Q bra WAIT_SPIN;\n\t"
        "WAIT_DONE:\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(abort_flag_smem), "l"(WAIT_LIMIT_NS)
        : "memory");
    return __all_sync(0xFFFFFFFFu, done != 0);
}

// ----------------------------------------------------------------------------- TMA
// start moving the 128-byte line at p towards the L2 (no register, nothing to wait for)
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

// TMA stores: shared memory tile -> global tensor, tracked by the thread's bulk async-group.
// Elements of the box that fall outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int x, int y, int z, int w) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// TMA reduction: global[box] += shared tile (element type and add come from the tensor map: int32 here);
// performed at the L2, exact and order-independent for integers
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, uint32_t src, int x, int y, int z, int w) {
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's bulk groups still READ their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
// named barrier among `count` threads (ids 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_barrier(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// barrier + OR-reduction of a per-thread flag: every participating thread gets the same answer
__device__ __forceinline__ uint32_t barrier_or(int id, int count, uint32_t flag) {
    uint32_t res;
    asm volatile(
        "{\n\t.reg .pred P, Q;\n\t"
        "setp.ne.u32 Q, %1, 0;\n\t"
        "bar.red.or.pred P, %2, %3, Q;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(res) : "r"(flag), "r"(id), "r"(count) : "memory");
    return res;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ----------------------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], int8 x int8 -> int32, issued by one thread.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "setp.ne.b32 P, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, P;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Bounded wait without a verdict: spins inside the asm until the phase completes, the CTA's abort flag is up, or the
// limit runs out -- in which case it raises the abort flag itself -- and then simply returns.  Nothing of the caller's
// control flow depends on it, which keeps the loops of the TMA producer and the MMA issuer straight-line uniform code;
// once the flag is up every later wait falls through at its first poll, so a role that runs on after a failed wait
// finishes in microseconds (its loads and MMAs are harmless: the kernel's results are discarded with the status).
// All 32 lanes of the (converged) warp call it.
#define NITI_QUIET_WAIT_ASM(LBL, BAR, PAR, ABRT, LIM)                           \
    "mbarrier.try_wait.parity.shared::cta.b64 Q, [" BAR "], " PAR ";\n\t"       \
    "@Q bra " LBL "_GO;\n\t"                                                    \
    "mov.u64 t0, %%globaltimer;\n\t"                                            \
    LBL "_SPIN:\n\t"                                                            \
    "mbarrier.try_wait.parity.shared::cta.b64 Q, [" BAR "], " PAR ";\n\t"       \
    "@Q bra " LBL "_GO;\n\t"                                                    \
    "ld.volatile.shared.u32 ab, [" ABRT "];\n\t"                                \
    "setp.ne.u32 P, ab, 0;\n\t"                                                 \
    "@P bra " LBL "_GO;\n\t"                                                    \
    "mov.u64 t1, %%globaltimer;\n\t"                                            \
    "sub.u64 t1, t1, t0;\n\t"                                                   \
    "setp.lt.u64 P, t1, " LIM ";\n\t"                                           \
    "@P bra " LBL "_SPIN;\n\t"                                                  \
    "mov.u32 ab, 1;\n\t"                                                        \
    "st.volatile.shared.u32 [" ABRT "], ab;\n\t"                                \
    LBL "_GO:\n\t"

__device__ __forceinline__ void mbar_wait_quiet(uint32_t bar, uint32_t parity, uint32_t abort_flag_smem) {
    asm volatile(
        "{\n\t"
        ".reg .pred P, Q;\n\t"
        ".reg .u64 t0, t1;\n\t"
        ".reg .u32 ab;\n\t"
        NITI_QUIET_WAIT_ASM("QW", "%0", "%1", "%2", "%3")
        "}"
        :: "r"(bar), "r"(parity), "r"(abort_flag_smem), "l"(WAIT_LIMIT_NS)
        : "memory");
}

// One reduction block of the MMA issuer's main loop as ONE asm statement with no outputs: wait (quietly, see above) for
// the stage's "full" barrier, then an elected lane issues the block's four MMAs (K = 32 each, operand descriptors a,
// a + a_step, ...; the first one accumulates only if `accumulate`) and the commit that hands the stage back.
template <bool PAIR>
__device__ __forceinline__ void umma_block4_wait(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint64_t a_step, uint64_t b_step,
                                                 uint32_t idesc, uint32_t accumulate, uint32_t commit_bar, uint32_t full_bar,
                                                 uint32_t parity, uint32_t abort_flag_smem) {
    if (PAIR) {
        asm volatile(
            "{\n\t"
            ".reg .pred P, Q, E, T;\n\t"
            ".reg .b32 r, ab;\n\t"
            ".reg .u64 t0, t1;\n\t"
            ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
            NITI_QUIET_WAIT_ASM("BWP", "%8", "%9", "%10", "%11")
            "elect.sync r|E, 0xFFFFFFFF;\n\t"
            "setp.ne.b32 P, %6, 0;\n\t"
            "setp.eq.b32 T, 0, 0;\n\t"
            "add.u64 a1, %1, %3;\n\t"
            "add.u64 b1, %2, %4;\n\t"
            "add.u64 a2, a1, %3;\n\t"
            "add.u64 b2, b1, %4;\n\t"
            "add.u64 a3, a2, %3;\n\t"
            "add.u64 b3, b2, %4;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %5, P;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%0], a1, b1, %5, T;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%0], a2, b2, %5, T;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%0], a3, b3, %5, T;\n\t"
            "@E tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%7], %12;\n\t"
            "}"
            :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "l"(a_step), "l"(b_step), "r"(idesc), "r"(accumulate), "r"(commit_bar),
               "r"(full_bar), "r"(parity), "r"(abort_flag_smem), "l"(WAIT_LIMIT_NS), "h"(static_cast<uint16_t>(3))
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred P, Q, E, T;\n\t"
            ".reg .b32 r, ab;\n\t"
            ".reg .u64 t0, t1;\n\t"
            ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
            NITI_QUIET_WAIT_ASM("BW", "%8", "%9", "%10", "%11")
            "elect.sync r|E, 0xFFFFFFFF;\n\t"
            "setp.ne.b32 P, %6, 0;\n\t"
            "setp.eq.b32 T, 0, 0;\n\t"
            "add.u64 a1, %1, %3;\n\t"
            "add.u64 b1, %2, %4;\n\t"
            "add.u64 a2, a1, %3;\n\t"
            "add.u64 b2, b1, %4;\n\t"
            "add.u64 a3, a2, %3;\n\t"
            "add.u64 b3, b2, %4;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %5, P;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %5, T;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%0], a2, b2, %5, T;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%0], a3, b3, %5, T;\n\t"
            "@E tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
            "}"
            :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "l"(a_step), "l"(b_step), "r"(idesc), "r"(accumulate), "r"(commit_bar),
               "r"(full_bar), "r"(parity), "r"(abort_flag_smem), "l"(WAIT_LIMIT_NS)
            : "memory");
    }
}

// One reduction block of the main loop as ONE asm statement, run by the whole (converged) warp: a non-blocking probe of
// the NEXT stage's "full" barrier is started, an elected lane issues the block's four MMAs (K = 32 each, operand
// descriptors a, a + a_step, ... ; the first one accumulates only if `accumulate`) and the commit that hands the stage
// back, and only then is the probe's answer read -- its shared-memory round trip runs under the MMA issue instead of
// in front of the next block.  Returns the probe's answer (per lane; make it uniform with a vote).
template <bool PAIR>
__device__ __forceinline__ uint32_t umma_block4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint64_t a_step, uint64_t b_step,
                                                uint32_t idesc, uint32_t accumulate, uint32_t commit_bar, uint32_t next_full_bar,
                                                uint32_t next_parity) {
    uint32_t ready;
    if (PAIR) {
        asm volatile(
            "{\n\t"
            ".reg .pred P, Q, E, T;\n\t"
            ".reg .b32 r;\n\t"
            ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 Q, [%9], %10;\n\t"
            "elect.sync r|E, 0xFFFFFFFF;\n\t"
            "setp.ne.b32 P, %7, 0;\n\t"
            "setp.eq.b32 T, 0, 0;\n\t"
            "add.u64 a1, %2, %4;\n\t"
            "add.u64 b1, %3, %5;\n\t"
            "add.u64 a2, a1, %4;\n\t"
            "add.u64 b2, b1, %5;\n\t"
            "add.u64 a3, a2, %4;\n\t"
            "add.u64 b3, b2, %5;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%1], %2, %3, %6, P;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%1], a1, b1, %6, T;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%1], a2, b2, %6, T;\n\t"
            "@E tcgen05.mma.cta_group::2.kind::i8 [%1], a3, b3, %6, T;\n\t"
            "@E tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%8], %11;\n\t"
            "selp.u32 %0, 1, 0, Q;\n\t"
            "}"
            : "=r"(ready)
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "l"(a_step), "l"(b_step), "r"(idesc), "r"(accumulate), "r"(commit_bar),
              "r"(next_full_bar), "r"(next_parity), "h"(static_cast<uint16_t>(3))
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred P, Q, E, T;\n\t"
            ".reg .b32 r;\n\t"
            ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 Q, [%9], %10;\n\t"
            "elect.sync r|E, 0xFFFFFFFF;\n\t"
            "setp.ne.b32 P, %7, 0;\n\t"
            "setp.eq.b32 T, 0, 0;\n\t"
            "add.u64 a1, %2, %4;\n\t"
            "add.u64 b1, %3, %5;\n\t"
            "add.u64 a2, a1, %4;\n\t"
            "add.u64 b2, b1, %5;\n\t"
            "add.u64 a3, a2, %4;\n\t"
            "add.u64 b3, b2, %5;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%1], %2, %3, %6, P;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%1], a1, b1, %6, T;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%1], a2, b2, %6, T;\n\t"
            "@E tcgen05.mma.cta_group::1.kind::i8 [%1], a3, b3, %6, T;\n\t"
            "@E tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%8];\n\t"
            "selp.u32 %0, 1, 0, Q;\n\t"
            "}"
            : "=r"(ready)
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "l"(a_step), "l"(b_step), "r"(idesc), "r"(accumulate), "r"(commit_bar),
              "r"(next_full_bar), "r"(next_parity)
            : "memory");
    }
    return ready;
}
// Four MMAs (K = 32 each, descriptors a, a + a_step, ...) issued by an elected lane of the converged warp, in one asm
// statement; no commit (more MMAs on the same stage follow).
__device__ __forceinline__ void umma_seq4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint64_t a_step, uint64_t b_step,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred P, E, T;\n\t"
        ".reg .b32 r;\n\t"
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        "elect.sync r|E, 0xFFFFFFFF;\n\t"
        "setp.ne.b32 P, %6, 0;\n\t"
        "setp.eq.b32 T, 0, 0;\n\t"
        "add.u64 a1, %1, %3;\n\t"
        "add.u64 b1, %2, %4;\n\t"
        "add.u64 a2, a1, %3;\n\t"
        "add.u64 b2, b1, %4;\n\t"
        "add.u64 a3, a2, %3;\n\t"
        "add.u64 b3, b2, %4;\n\t"
        "@E tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %5, P;\n\t"
        "@E tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %5, T;\n\t"
        "@E tcgen05.mma.cta_group::1.kind::i8 [%0], a2, b2, %5, T;\n\t"
        "@E tcgen05.mma.cta_group::1.kind::i8 [%0], a3, b3, %5, T;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "l"(a_step), "l"(b_step), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrives once all tcgen05 operations issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 0 and 1) act as one MMA unit: rank 0 issues M = 256 MMAs whose A rows and
// B columns are split between the two CTAs' shared memories and whose accumulator rows are split
// between their tensor memories.  Every CTA fetches its own operand halves with its own loads.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of both CTAs
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in the CTA of rank `rank` (shared::cluster window)
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of a CTA pair: data lands in the executing CTA, the byte count is reported to `bar`, which
// may live in either CTA of the pair (a shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "setp.ne.b32 P, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, P;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the mbarrier at this shared-memory offset in BOTH CTAs of the pair once the pair's MMAs so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

// ----------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor (64 bit): start address >> 4 in bits [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48), swizzle
// mode in [61,64) (2 = 128 B, 4 = 64 B, 6 = 32 B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle_code) {
    uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
    uint32_t hi = ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (swizzle_code << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
    return desc + (bytes >> 4);  // start-address field is the low 14 bits; tiles never wrap it
}
// Instruction descriptor for kind::i8: D = S32 (2 at bit 4), A/B = signed 8-bit (1 at bits 7 and
// 10), operand majors at bits 15/16 (1 = MN-major), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n, int a_mn_major, int b_mn_major) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace niti
