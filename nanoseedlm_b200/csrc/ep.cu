// Device steps of the expert-parallel layer (include/nslm_ep.h): the per-rank pair plan, the per-token pre-sum of the
// local experts' outputs and the rank-order sum of the returned partial rows.  They read and write local memory only.
#include "ep_sync.cuh"

namespace nsl {

constexpr uint32_t FULL = 0xFFFFFFFFu;

// One block.  Pairs are visited in token order in rounds of 1024; a ballot prefix inside each warp and a scan of the
// 32 warp counts give every kept pair its slot, so the compacted list keeps token order.
//
// Mirrored pairs of ranks (lo2 < hi2): this rank also holds the experts [lo2, hi2) of its partner, and the partner holds
// this rank's.  Both plan the same list -- the pairs whose expert lies in either range, in token order -- and split it
// in the middle: the lower rank of the two takes the first ceil(n/2) pairs, the upper rank the rest.  Either rank's
// share differs from the other's by at most one pair whatever the routing.  Local slice index: e - lo for the own
// range, (hi - lo) + e - lo2 for the partner's.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int32_t* __restrict__ ind, const float* __restrict__ wt, int n_ranks,
                                                       int t_loc, int k, int rank_stride, int row_stride, int lo, int hi,
                                                       int32_t* __restrict__ sel, int32_t* __restrict__ xrow,
                                                       float* __restrict__ wsel, int32_t* __restrict__ tok_off,
                                                       int32_t* __restrict__ count, NslEpWindow win, int wait, int lo2, int hi2,
                                                       int upper) {
    __shared__ int wsum[32];
    __shared__ int base;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int T = n_ranks * t_loc, n = T * k;
    grid_dependents_go();   // a dependent launch of the next kernel may bring its blocks in already
    if (wait) wait_flags(win, win.dflag_off, (local_words(win)[EPW_EPOCH] + 1) * (uint32_t) win.t_loc, 1);   // peer-memory form: every rank's chunk has landed
    const bool mirror = lo2 < hi2;
    int first = 0, last = 0x7FFFFFFF;          // this rank keeps the list positions [first, last)
    if (mirror) {                              // pass 1: the length of the shared list
        if (tid == 0) base = 0;
        __syncthreads();
        for (int c0 = 0; c0 < n; c0 += 1024) {
            const int i = c0 + tid;
            int e = -1;
            if (i < n) {
                const int g = i / k, j = i % k, r = g / t_loc, t = g % t_loc;
                e = ind[(size_t) r * rank_stride + (size_t) t * k + j];
            }
            const uint32_t m = __ballot_sync(FULL, (e >= lo && e < hi) || (e >= lo2 && e < hi2));
            if (lane == 0 && m) atomicAdd(&base, __popc(m));
        }
        __syncthreads();
        const int half = (base + 1) / 2;
        if (upper) first = half; else last = half;
        __syncthreads();
    }
    if (tid == 0) base = 0;
    __syncthreads();
    for (int c0 = 0; c0 < n; c0 += 1024) {
        const int i = c0 + tid;
        int e = -1, g = 0, r = 0, t = 0, j = 0;
        float wv = 0.0f;
        if (i < n) {
            g = i / k; j = i % k; r = g / t_loc; t = g % t_loc;
            const size_t at = (size_t) r * rank_stride + (size_t) t * k + j;
            e = ind[at];
            wv = wt[at];
        }
        const bool own = e >= lo && e < hi, member = own || (e >= lo2 && e < hi2);
        const uint32_t m = __ballot_sync(FULL, member);
        if (lane == 0) wsum[w] = __popc(m);
        __syncthreads();
        int before = base, total = 0;
        for (int q = 0; q < 32; ++q) { if (q < w) before += wsum[q]; total += wsum[q]; }
        const int lpos = before + __popc(m & ((1u << lane) - 1u));     // position in the (shared) list
        const int pos = min(max(lpos, first), last) - first;           // position among the pairs this rank keeps
        if (member && lpos >= first && lpos < last) {
            sel[pos] = own ? e - lo : (hi - lo) + e - lo2;
            xrow[pos] = r * row_stride + t;
            wsel[pos] = wv;
        }
        if (i < n && j == 0) tok_off[g] = pos;   // pairs of token g start here (kept or not, the running position)
        __syncthreads();
        if (tid == 0) base += total;
        __syncthreads();
    }
    if (tid == 0) {
        const int kept = min(max(base, first), last) - first;
        tok_off[T] = kept;
        *count = kept;
    }
}

__global__ void ep_combine_kernel(const float* __restrict__ D, const float* __restrict__ wsel, const int32_t* __restrict__ tok_off,
                                  int d, float* __restrict__ partial) {
    const int g = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    grid_dependents_go();
    grid_dependency_wait();
    if (c >= d) return;
    const int p0 = tok_off[g], p1 = tok_off[g + 1];
    float acc = 0.0f;
    for (int p = p0; p < p1; ++p) acc += wsel[p] * D[(size_t) p * d + c];
    partial[(size_t) g * d + c] = acc;
}

__global__ void ep_reduce_kernel(const float* __restrict__ parts, int n_ranks, int t_loc, int d, float* __restrict__ out) {
    const size_t n = (size_t) t_loc * d;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t) gridDim.x * blockDim.x) {
        float acc = parts[i];
        for (int r = 1; r < n_ranks; ++r) acc += parts[(size_t) r * n + i];
        out[i] = acc;
    }
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void nsl_ep_plan(cudaStream_t s, const int32_t* ind, const float* wt, int n_ranks, int t_loc, int k, int rank_stride,
                 int row_stride, int lo, int hi, int32_t* sel, int32_t* xrow, float* wsel, int32_t* tok_off,
                 int32_t* count) {
    if ((long long) n_ranks * t_loc * k > 65536 || n_ranks < 1 || t_loc < 1 || k < 1) {
        set_error("nsl_ep_plan: %d ranks x %d tokens x top %d is out of range", n_ranks, t_loc, k);
        return;
    }
    ep_plan_kernel<<<1, 1024, 0, s>>>(ind, wt, n_ranks, t_loc, k, rank_stride, row_stride, lo, hi, sel, xrow, wsel, tok_off, count,
                                      NslEpWindow{}, 0, 0, 0, 0);
    count_launch();
}

// The plan on the window's receive area, after waiting (inside the kernel) for every rank's dispatch of this step.
void nsl_ep_p2p_plan(cudaStream_t s, NslEpWindow w, uint64_t ind_off, uint64_t wt_off, int k, int row_stride, int lo, int hi,
                     int lo2, int hi2, int upper, int32_t* sel, int32_t* xrow, float* wsel, int32_t* tok_off, int32_t* count) {
    if (w.n < 1 || w.n > NSL_EP_MAX_RANKS || w.me < 0 || w.me >= w.n || !w.win[w.me] || w.t_loc < 1 || k < 1 ||
        (long long) w.n * w.t_loc * k > 65536 || ind_off % 4 || wt_off % 4 || w.chunk_bytes % 4 ||
        ind_off + (uint64_t) w.t_loc * k * 4 > w.chunk_bytes || wt_off + (uint64_t) w.t_loc * k * 4 > w.chunk_bytes ||
        w.recv_off + (uint64_t) w.n * w.chunk_bytes > w.bytes) {
        set_error("nsl_ep_p2p_plan: window, offsets or sizes out of range");
        return;
    }
    const char* recv = (const char*) w.win[w.me] + w.recv_off;
    ep_plan_kernel<<<1, 1024, 0, s>>>((const int32_t*) (recv + ind_off), (const float*) (recv + wt_off), w.n, w.t_loc, k,
                                      (int) (w.chunk_bytes / 4), row_stride, lo, hi, sel, xrow, wsel, tok_off, count, w, 1,
                                      lo2, hi2, upper);
    count_launch();
}

void nsl_ep_combine(cudaStream_t s, const float* D, const float* wsel, const int32_t* tok_off, int T, int d, float* partial) {
    if (T < 1 || d < 1) return;
    launch(ep_combine_kernel, dim3((unsigned) (d + 255) / 256, (unsigned) T), 256, 0, s, D, wsel, tok_off, d, partial);
    count_launch();
}

void nsl_ep_reduce(cudaStream_t s, const float* parts, int n_ranks, int t_loc, int d, float* out) {
    if (n_ranks < 1 || t_loc < 1 || d < 1) return;
    const size_t n = (size_t) t_loc * d;
    const unsigned blocks = (unsigned) ((n + 255) / 256 < (size_t) sm_count() * 4 ? (n + 255) / 256 : (size_t) sm_count() * 4);
    ep_reduce_kernel<<<blocks, 256, 0, s>>>(parts, n_ranks, t_loc, d, out);
    count_launch();
}

}   // extern "C"
