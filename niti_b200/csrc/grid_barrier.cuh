// A bounded barrier across the thread blocks of a cooperative launch (all blocks co-resident).
#pragma once
#include <cstdint>

namespace niti {

constexpr unsigned long long GRID_WAIT_LIMIT_NS = 500000000ull;  // 0.5 s

__device__ __forceinline__ unsigned long long grid_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Arrival without a separate fence and without waiting for the atomic's result: one fire-and-forget reduction with
// release semantics (a full __threadfence + atomicAdd costs two more round trips to the L2).
__device__ __forceinline__ void red_release_add(int32_t* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_max(unsigned* p, unsigned v) {
    asm volatile("red.relaxed.gpu.global.max.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const void* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Every block calls this with the same, monotonically growing `target` (blocks x number of the barrier);
// `counter` starts at zero.  Returns false when the other blocks did not arrive within the limit: the
// caller must then leave the kernel (status, when given, receives {code, block, target}).
__device__ __forceinline__ bool bounded_grid_barrier(int32_t* counter, int target, int32_t* status, int code, int* flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        red_release_add(counter, 1);  // release: this block's earlier global writes are visible to whoever sees the count
        const unsigned long long t0 = grid_timer_ns();
        bool arrived = false;
        for (unsigned spin = 0;; ++spin) {
            if (ld_acquire_gpu(counter) >= target) { arrived = true; break; }  // a load: waiters do not queue at the L2's atomic unit
            if ((spin & 63) == 63 && grid_timer_ns() - t0 > GRID_WAIT_LIMIT_NS) break;
        }
        *flag = arrived ? 1 : 0;
        if (!arrived && status != nullptr && atomicCAS(status, 0, code) == 0) {
            status[1] = static_cast<int32_t>(blockIdx.x);
            status[2] = target;
        }
    }
    __syncthreads();
    return *flag != 0;
}

}  // namespace niti
