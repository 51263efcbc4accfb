// Expert-parallel dispatch and combine over peer memory (include/nslm_ep.h, the NslEpWindow part): the producer kernels
// store straight into the consumers' windows over NVLink and raise a flag there; the consumer kernels wait on flags in
// their OWN memory.  No collective library call and no host synchronisation sits inside a step, so a whole step is
// kernels on one stream (one CUDA graph).
//
// Ordering.  Every window holds, per producer rank, a dispatch counter and a combine counter.  A producer block stores its
// data into ONE destination window, meets at a barrier, and its first thread fences at system scope and adds the number
// of token rows it delivered to that window's counter `me` (a fence followed by a relaxed add is a release; one fence
// deep, no grid-wide ticket).  A step delivers t_loc rows per (producer, destination) in either direction, so after e
// steps a counter stands at e * t_loc: a consumer thread reads its counter with an acquire at system scope until it has
// reached that value, then the block passes a barrier and reads the data.  Counters only grow, so no reset race
// exists; a window's data slots are reused only after the step's own chain (dispatch -> plan -> mat-vecs -> combine ->
// reduce) has consumed them on every rank, which the counters themselves enforce (a rank cannot dispatch step s+1
// before it has reduced step s, which needs every rank's combine of step s, which follows that rank's reads of step
// s's rows).
//
// Every wait is bounded (about two seconds): a wait that runs out records a code in the window's status word and the
// kernel carries on with whatever the window holds, so the stream always drains and the host can read the status.
#include "ep_sync.cuh"
#include "route.cuh"
#include "seed_block.cuh"

#include <cstring>

namespace nsl {

__device__ __forceinline__ char* recv_slot(const NslEpWindow& w, int rank) {   // this rank's chunk inside rank's window
    return (char*) w.win[rank] + w.recv_off + (size_t) w.me * w.chunk_bytes;
}

// Dispatch of a ready-made chunk: block r copies it into slot `me` of rank r's receive area.
__global__ void __launch_bounds__(1024) ep_dispatch_kernel(NslEpWindow w, const uint4* __restrict__ chunk) {
    grid_dependents_go();
    grid_dependency_wait();
    const int r = blockIdx.x;
    uint4* dst = (uint4*) recv_slot(w, r);
    for (size_t j = threadIdx.x; j < w.chunk_bytes / 16; j += blockDim.x) dst[j] = chunk[j];
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        red_add_sys(flag_of(w, r, w.dflag_off, w.me), (uint32_t) w.t_loc);
    }
}

// Router + bf16 packing + dispatch in one kernel.  Block (t, r) serves local token t and destination rank r: warp 0 routes
// the token (every destination's block repeats the few microseconds of routing rather than wait for one block's picks),
// the other warps convert the token's row to bf16 and store it into rank r's receive area; then the ids and weights follow
// and the block signals one row to rank r.  One block per (token, destination) keeps each block's remote stores short: with
// a block per token the eight destinations' stores ran one after the other.
template <int PER>
__global__ void __launch_bounds__(256) ep_route_dispatch_kernel(NslEpWindow w, const float* __restrict__ logits, int ld,
                                                               const float* __restrict__ x, int E, int k, int d,
                                                               uint64_t ind_off, uint64_t wt_off, int32_t* __restrict__ ind_out,
                                                               float* __restrict__ wt_out) {
    __shared__ int32_t s_ind[32];
    __shared__ float s_wt[32];
    grid_dependents_go();
    const int t = blockIdx.x, r = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    char* slot = recv_slot(w, r);
    if (warp == 0) {
        route_row<PER>(E, k, logits + (size_t) t * ld, lane, s_ind, s_wt);
    } else {
        const float4* xr = (const float4*) (x + (size_t) t * d);
        uint4* dst = (uint4*) (slot + (size_t) t * d * 2);
        for (int i = threadIdx.x - 32; i < d / 8; i += 224) {
            const float4 a = __ldg(xr + 2 * i), b = __ldg(xr + 2 * i + 1);
            uint4 o;
            o.x = bf16_bits(a.x) | ((uint32_t) bf16_bits(a.y) << 16);
            o.y = bf16_bits(a.z) | ((uint32_t) bf16_bits(a.w) << 16);
            o.z = bf16_bits(b.x) | ((uint32_t) bf16_bits(b.y) << 16);
            o.w = bf16_bits(b.z) | ((uint32_t) bf16_bits(b.w) << 16);
            dst[i] = o;
        }
    }
    __syncthreads();
    if ((int) threadIdx.x < k) {
        ((int32_t*) (slot + ind_off))[t * k + threadIdx.x] = s_ind[threadIdx.x];
        ((float*) (slot + wt_off))[t * k + threadIdx.x] = s_wt[threadIdx.x];
        if (ind_out && r == 0) {      // the caller's own copy of its tokens' routing
            ind_out[t * k + threadIdx.x] = s_ind[threadIdx.x];
            wt_out[t * k + threadIdx.x] = s_wt[threadIdx.x];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        red_add_sys(flag_of(w, r, w.dflag_off, w.me), 1u);
    }
}

// The plan's wait as a kernel of its own (nsl_ep_p2p_plan has it built in): returns when every rank's rows have landed.
__global__ void __launch_bounds__(32) ep_wait_dispatch_kernel(NslEpWindow w) {
    grid_dependents_go();
    wait_flags(w, w.dflag_off, (local_words(w)[EPW_EPOCH] + 1) * (uint32_t) w.t_loc, 1);
}

// Combine: block g pre-sums token g's local experts and stores the row into slot `me` of the partial-row area of the
// rank that owns the token, then signals one row to that rank.
__global__ void __launch_bounds__(256) ep_combine_p2p_kernel(NslEpWindow w, const float* __restrict__ D, const float* __restrict__ wsel,
                                                             const int32_t* __restrict__ tok_off, int d) {
    grid_dependents_go();
    grid_dependency_wait();
    const int g = blockIdx.x, owner = g / w.t_loc, t = g - owner * w.t_loc;
    const int p0 = tok_off[g], p1 = tok_off[g + 1];
    float* dst = (float*) ((char*) w.win[owner] + w.parts_off) + ((size_t) w.me * w.t_loc + t) * d;
    for (int c = threadIdx.x * 4; c < d; c += 1024) {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int p = p0; p < p1; ++p) {
            const float wv = wsel[p];
            const float4 v = *(const float4*) (D + (size_t) p * d + c);
            acc.x += wv * v.x; acc.y += wv * v.y; acc.z += wv * v.z; acc.w += wv * v.w;
        }
        *(float4*) (dst + c) = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        red_add_sys(flag_of(w, owner, w.cflag_off, w.me), 1u);
    }
}

// Reduce: wait for every rank's partial rows, add them in rank order, and let the last block close the step.
__global__ void __launch_bounds__(256) ep_reduce_p2p_kernel(NslEpWindow w, int d, float* __restrict__ out) {
    grid_dependents_go();
    uint32_t* lw = local_words(w);
    const uint32_t e = lw[EPW_EPOCH] + 1;
    wait_flags(w, w.cflag_off, e * (uint32_t) w.t_loc, 2);
    const float4* parts = (const float4*) ((const char*) w.win[w.me] + w.parts_off);
    const size_t n4 = (size_t) w.t_loc * d / 4;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t) gridDim.x * blockDim.x) {
        float4 acc = parts[i];
        for (int r = 1; r < w.n; ++r) {
            const float4 v = parts[(size_t) r * n4 + i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        ((float4*) out)[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(lw + EPW_TICKET_REDUCE, 1u) == gridDim.x - 1) {
        lw[EPW_TICKET_REDUCE] = 0;
        lw[EPW_EPOCH] = e;   // the next step's kernels follow in the stream
    }
}

static bool window_ok(const NslEpWindow& w, const char* who) {
    bool ok = w.n >= 1 && w.n <= NSL_EP_MAX_RANKS && w.me >= 0 && w.me < w.n && w.chunk_bytes % 16 == 0 && w.chunk_bytes > 0 &&
              w.t_loc >= 1;
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
    launch(ep_dispatch_kernel, (unsigned) w.n, 1024, 0, s, w, (const uint4*) chunk);
    count_launch();
}

void nsl_ep_p2p_route_dispatch(cudaStream_t s, NslEpWindow w, int n_exp, int top_k, const float* logits, int ld, const float* x,
                               int d, uint64_t ind_off, uint64_t wt_off, int32_t* ind_out, float* wt_out) {
    if (!window_ok(w, "nsl_ep_p2p_route_dispatch")) return;
    const uint64_t meta = (uint64_t) w.t_loc * top_k * 4;
    if (n_exp < 1 || n_exp > 1024 || top_k < 1 || top_k > 32 || top_k > n_exp || d < 8 || d % 8 || !aligned16(x) ||
        ind_off % 4 || wt_off % 4 || (uint64_t) w.t_loc * d * 2 > ind_off || ind_off + meta > wt_off ||
        wt_off + meta > w.chunk_bytes) {
        set_error("nsl_ep_p2p_route_dispatch: %d experts (<= 1024), top %d (<= 32), width %d (a multiple of 8) or chunk offsets out of range",
                  n_exp, top_k, d);
        return;
    }
    const dim3 grid((unsigned) w.t_loc, (unsigned) w.n);
    if (n_exp <= 128) ep_route_dispatch_kernel<4><<<grid, 256, 0, s>>>(w, logits, ld, x, n_exp, top_k, d, ind_off, wt_off, ind_out, wt_out);
    else if (n_exp <= 512) ep_route_dispatch_kernel<16><<<grid, 256, 0, s>>>(w, logits, ld, x, n_exp, top_k, d, ind_off, wt_off, ind_out, wt_out);
    else ep_route_dispatch_kernel<32><<<grid, 256, 0, s>>>(w, logits, ld, x, n_exp, top_k, d, ind_off, wt_off, ind_out, wt_out);
    count_launch();
}

void nsl_ep_p2p_wait_dispatch(cudaStream_t s, NslEpWindow w) {
    if (!window_ok(w, "nsl_ep_p2p_wait_dispatch")) return;
    ep_wait_dispatch_kernel<<<1, 32, 0, s>>>(w);
    count_launch();
}

static bool parts_fit(const NslEpWindow& w, int d, const char* who) {
    if (d < 4 || d % 4 || w.parts_off + (uint64_t) w.n * w.t_loc * d * 4 > w.bytes) {
        set_error("%s: rows of width %d (a multiple of 4) do not fit the window's partial-row area", who, d);
        return false;
    }
    return true;
}

void nsl_ep_p2p_combine(cudaStream_t s, NslEpWindow w, const float* D, const float* wsel, const int32_t* tok_off, int d) {
    if (!window_ok(w, "nsl_ep_p2p_combine") || !parts_fit(w, d, "nsl_ep_p2p_combine")) return;
    if (!aligned16(D)) { set_error("nsl_ep_p2p_combine: D must be 16-byte aligned"); return; }
    launch(ep_combine_p2p_kernel, (unsigned) (w.n * w.t_loc), 256, 0, s, w, D, wsel, tok_off, d);
    count_launch();
}

void nsl_ep_p2p_reduce(cudaStream_t s, NslEpWindow w, int d, float* out) {
    if (!window_ok(w, "nsl_ep_p2p_reduce") || !parts_fit(w, d, "nsl_ep_p2p_reduce")) return;
    if (!aligned16(out)) { set_error("nsl_ep_p2p_reduce: out must be 16-byte aligned"); return; }
    const size_t n4 = (size_t) w.t_loc * d / 4, blocks = (n4 + 255) / 256;
    ep_reduce_p2p_kernel<<<(unsigned) (blocks < 128 ? blocks : 128), 256, 0, s>>>(w, d, out);
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
