// Expert-parallel dispatch and combine over peer memory (include/nslm_ep.h, the NslEpWindow part): the producer kernels
// store straight into the consumers' windows over NVLink and raise a flag there; the consumer kernels wait on flags in
// their OWN memory.  No collective library call and no host synchronisation sits inside a step, so a whole step is
// kernels on one stream (one CUDA graph).
//
// Ordering.  A producer block finishes its stores, fences at system scope and takes a ticket; the block with the last
// ticket fences again and writes the step's epoch number into the flag word `me` of every rank's window (release,
// system scope).  A consumer thread reads its flag with an acquire at system scope until it holds the epoch, then the
// block passes a barrier and reads the data.  Flags only grow, so no reset race exists; a window's data slots are
// reused only after the step's own chain (dispatch -> plan -> mat-vecs -> combine -> reduce) has consumed them on every
// rank, which the flags themselves enforce (a rank cannot dispatch step s+1 before it has reduced step s, which needs
// every rank's combine of step s, which follows that rank's reads of step s's rows).
//
// Every wait is bounded (about two seconds): a wait that runs out records a code in the window's status word and the
// kernel carries on with whatever the window holds, so the stream always drains and the host can read the status.
#include "common.cuh"
#include "../../include/nslm_ep.h"

#include <cstring>

namespace nsl {

constexpr unsigned long long EP_WAIT_NS = 2000000000ull;
enum { EPW_EPOCH = 0, EPW_TICKET_DISPATCH = 1, EPW_TICKET_COMBINE = 2, EPW_TICKET_REDUCE = 3, EPW_STATUS = 4 };
constexpr int EP_FLAG_STRIDE = 32;   // flag words are 128 bytes apart

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t* local_words(const NslEpWindow& w) {
    return (uint32_t*) ((char*) w.win[w.me] + w.local_off);
}

// Thread r < n waits until flag r of this rank's window holds epoch e or later; then the block meets at a barrier.
__device__ __forceinline__ void wait_flags(const NslEpWindow& w, uint64_t flag_off, uint32_t e, int code) {
    if ((int) threadIdx.x < w.n) {
        const uint32_t* f = (const uint32_t*) ((const char*) w.win[w.me] + flag_off) + threadIdx.x * EP_FLAG_STRIDE;
        const unsigned long long t0 = now_ns();
        unsigned it = 0;
        while ((int32_t) (ld_acquire_sys(f) - e) < 0) {
            if (((++it & 63u) == 0 && now_ns() - t0 > EP_WAIT_NS) || it > (1u << 28)) {
                atomicExch(local_words(w) + EPW_STATUS, (uint32_t) (code * 256 + (int) threadIdx.x + 1));
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
}

// Called by every thread after its stores: the last block of the grid raises flag `me` in every window.
__device__ __forceinline__ void signal_when_grid_done(const NslEpWindow& w, uint64_t flag_off, int ticket_word, uint32_t e,
                                                      unsigned blocks) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t* lw = local_words(w);
        if (atomicAdd(lw + ticket_word, 1u) == blocks - 1) {
            lw[ticket_word] = 0;
            __threadfence_system();
            for (int r = 0; r < w.n; ++r)
                st_release_sys((uint32_t*) ((char*) w.win[r] + flag_off) + w.me * EP_FLAG_STRIDE, e);
        }
    }
}

// Dispatch: this rank's chunk (token rows as bf16, expert ids, routing weights) into slot `me` of every rank.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(NslEpWindow w, const uint4* __restrict__ chunk) {
    grid_dependents_go();
    grid_dependency_wait();
    const uint32_t e = local_words(w)[EPW_EPOCH] + 1;
    const size_t n16 = w.chunk_bytes / 16, total = n16 * (size_t) w.n;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t) gridDim.x * blockDim.x) {
        const int r = (int) (i / n16);
        const size_t j = i - (size_t) r * n16;
        ((uint4*) ((char*) w.win[r] + w.recv_off + (size_t) w.me * w.chunk_bytes))[j] = chunk[j];
    }
    signal_when_grid_done(w, w.dflag_off, EPW_TICKET_DISPATCH, e, gridDim.x);
}

// The plan's wait: one block that returns when every rank's chunk of this step has landed.  (The plan kernel proper
// follows in the stream and reads the window's receive area.)
__global__ void __launch_bounds__(32) ep_wait_dispatch_kernel(NslEpWindow w) {
    grid_dependents_go();
    wait_flags(w, w.dflag_off, local_words(w)[EPW_EPOCH] + 1, 1);
}

// Combine: token g's pre-summed row goes into slot `me` of the parts area of the rank that owns the token.
__global__ void __launch_bounds__(256) ep_combine_p2p_kernel(NslEpWindow w, const float* __restrict__ D, const float* __restrict__ wsel,
                                                             const int32_t* __restrict__ tok_off, int t_loc, int d) {
    grid_dependents_go();
    grid_dependency_wait();
    const uint32_t e = local_words(w)[EPW_EPOCH] + 1;
    const int g = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < d) {
        const int p0 = tok_off[g], p1 = tok_off[g + 1];
        float acc = 0.0f;
        for (int p = p0; p < p1; ++p) acc += wsel[p] * D[(size_t) p * d + c];
        const int owner = g / t_loc, t = g - owner * t_loc;
        ((float*) ((char*) w.win[owner] + w.parts_off))[((size_t) w.me * t_loc + t) * d + c] = acc;
    }
    signal_when_grid_done(w, w.cflag_off, EPW_TICKET_COMBINE, e, gridDim.x * gridDim.y);
}

// Reduce: wait for every rank's partial rows, add them in rank order, and let the last block close the step.
__global__ void __launch_bounds__(256) ep_reduce_p2p_kernel(NslEpWindow w, int t_loc, int d, float* __restrict__ out) {
    grid_dependents_go();
    uint32_t* lw = local_words(w);
    const uint32_t e = lw[EPW_EPOCH] + 1;
    wait_flags(w, w.cflag_off, e, 2);
    const float* parts = (const float*) ((const char*) w.win[w.me] + w.parts_off);
    const size_t n = (size_t) t_loc * d;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t) gridDim.x * blockDim.x) {
        float acc = parts[i];
        for (int r = 1; r < w.n; ++r) acc += parts[(size_t) r * n + i];
        out[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(lw + EPW_TICKET_REDUCE, 1u) == gridDim.x - 1) {
        lw[EPW_TICKET_REDUCE] = 0;
        lw[EPW_EPOCH] = e;   // the next step's kernels follow in the stream
    }
}

static bool window_ok(const NslEpWindow& w, const char* who) {
    bool ok = w.n >= 1 && w.n <= NSL_EP_MAX_RANKS && w.me >= 0 && w.me < w.n && w.chunk_bytes % 16 == 0 && w.chunk_bytes > 0;
    for (int r = 0; ok && r < w.n; ++r) ok = w.win[r] != NULL && ((uintptr_t) w.win[r] & 255u) == 0;
    const uint64_t ends[5] = {w.recv_off + (uint64_t) w.n * w.chunk_bytes, w.parts_off, w.dflag_off + (uint64_t) w.n * 128,
                              w.cflag_off + (uint64_t) w.n * 128, w.local_off + 64};
    for (uint64_t end : ends) ok = ok && end <= w.bytes;
    ok = ok && w.recv_off % 256 == 0 && w.parts_off % 256 == 0 && w.dflag_off % 128 == 0 && w.cflag_off % 128 == 0 && w.local_off % 128 == 0;
    if (!ok) set_error("%s: the window description is inconsistent (ranks, alignment or offsets beyond its size)", who);
    return ok;
}

}   // namespace nsl

using namespace nsl;

extern "C" {

int nsl_ep_window_alloc(size_t bytes, void** ptr, void* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    *ptr = NULL;
    if (cudaMalloc(ptr, bytes) != cudaSuccess || cudaMemset(*ptr, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        set_error("nsl_ep_window_alloc: %zu bytes: %s", bytes, cudaGetErrorString(cudaGetLastError()));
        return -1;
    }
    cudaIpcMemHandle_t h;
    if (handle64) {
        if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) {
            set_error("nsl_ep_window_alloc: no inter-process handle: %s", cudaGetErrorString(cudaGetLastError()));
            return -1;
        }
        memcpy(handle64, &h, 64);
    }
    return 0;
}

int nsl_ep_window_open(const void* handle64, void** ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    *ptr = NULL;
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        set_error("nsl_ep_window_open: %s", cudaGetErrorString(cudaGetLastError()));
        return -1;
    }
    return 0;
}

int nsl_ep_window_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
int nsl_ep_window_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }

void nsl_ep_p2p_dispatch(cudaStream_t s, NslEpWindow w, const void* chunk) {
    if (!window_ok(w, "nsl_ep_p2p_dispatch")) return;
    if (!aligned16(chunk)) { set_error("nsl_ep_p2p_dispatch: the chunk must be 16-byte aligned"); return; }
    const size_t n16 = w.chunk_bytes / 16 * (size_t) w.n;
    const size_t blocks = (n16 + 255) / 256;
    launch(ep_dispatch_kernel, (unsigned) (blocks < 64 ? blocks : 64), 256, 0, s, w, (const uint4*) chunk);
    count_launch();
}

void nsl_ep_p2p_wait_dispatch(cudaStream_t s, NslEpWindow w) {
    if (!window_ok(w, "nsl_ep_p2p_wait_dispatch")) return;
    ep_wait_dispatch_kernel<<<1, 32, 0, s>>>(w);
    count_launch();
}

void nsl_ep_p2p_combine(cudaStream_t s, NslEpWindow w, const float* D, const float* wsel, const int32_t* tok_off, int t_loc,
                        int d) {
    if (!window_ok(w, "nsl_ep_p2p_combine")) return;
    if (t_loc < 1 || d < 1 || w.parts_off + (uint64_t) w.n * t_loc * d * 4 > w.bytes) {
        set_error("nsl_ep_p2p_combine: %d tokens of width %d do not fit the window's partial-row area", t_loc, d);
        return;
    }
    launch(ep_combine_p2p_kernel, dim3((unsigned) (d + 255) / 256, (unsigned) (w.n * t_loc)), 256, 0, s, w, D, wsel, tok_off, t_loc, d);
    count_launch();
}

void nsl_ep_p2p_reduce(cudaStream_t s, NslEpWindow w, int t_loc, int d, float* out) {
    if (!window_ok(w, "nsl_ep_p2p_reduce")) return;
    if (t_loc < 1 || d < 1 || w.parts_off + (uint64_t) w.n * t_loc * d * 4 > w.bytes) {
        set_error("nsl_ep_p2p_reduce: %d tokens of width %d do not fit the window's partial-row area", t_loc, d);
        return;
    }
    const size_t n = (size_t) t_loc * d, blocks = (n + 255) / 256;
    ep_reduce_p2p_kernel<<<(unsigned) (blocks < 128 ? blocks : 128), 256, 0, s>>>(w, t_loc, d, out);
    count_launch();
}

// The window's status word (0 = no wait ever ran out; else code * 256 + the rank waited for + 1; code 1 = dispatch,
// 2 = combine), read after the stream has drained; the word is cleared.
int nsl_ep_p2p_status(NslEpWindow w) {
    if (!window_ok(w, "nsl_ep_p2p_status")) return -1;
    uint32_t v = 0, zero = 0;
    uint32_t* word = (uint32_t*) ((char*) w.win[w.me] + w.local_off) + EPW_STATUS;
    if (cudaMemcpy(&v, word, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemcpy(word, &zero, 4, cudaMemcpyHostToDevice);
    return (int) v;
}

}   // extern "C"
