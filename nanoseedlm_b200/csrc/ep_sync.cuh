// Flags and tickets of the peer-memory exchange (see ep_p2p.cu for the protocol): device helpers shared by its kernels.
#pragma once
#include "common.cuh"
#include "../../include/nslm_ep.h"

namespace nsl {

constexpr unsigned long long EP_WAIT_NS = 2000000000ull;
enum { EPW_EPOCH = 0, EPW_TICKET_REDUCE = 3, EPW_STATUS = 4 };
constexpr int EP_FLAG_STRIDE = 32;   // flag words are 128 bytes apart

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t* local_words(const NslEpWindow& w) {
    return (uint32_t*) ((char*) w.win[w.me] + w.local_off);
}

// Thread r < n waits until counter r of this rank's window has reached `target` (wrap-safe); then the block meets at a
// barrier.
__device__ __forceinline__ void wait_flags(const NslEpWindow& w, uint64_t flag_off, uint32_t target, int code) {
    if ((int) threadIdx.x < w.n) {
        const uint32_t* f = (const uint32_t*) ((const char*) w.win[w.me] + flag_off) + threadIdx.x * EP_FLAG_STRIDE;
        const unsigned long long t0 = now_ns();
        unsigned it = 0;
        while ((int32_t) (ld_acquire_sys(f) - target) < 0) {
            if (((++it & 63u) == 0 && now_ns() - t0 > EP_WAIT_NS) || it > (1u << 28)) {
                atomicExch(local_words(w) + EPW_STATUS, (uint32_t) (code * 256 + (int) threadIdx.x + 1));
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void red_add_sys(uint32_t* p, uint32_t v) {       // after a system-scope fence: a release
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t* flag_of(const NslEpWindow& w, int rank, uint64_t flag_off, int slot) {
    return (uint32_t*) ((char*) w.win[rank] + flag_off) + slot * EP_FLAG_STRIDE;
}

}   // namespace nsl
