// The small kernels either side of the seed mat-vec on the MoE path: router top-k, SwiGLU, the two combines, grouping
// of (token, expert) pairs by expert, activation packing, and the expert cache's admit and copy.
// Reference behaviour they reproduce: engine/kernels_qwen4.cu:385-422 (router), :506-515 (combine);
// engine/kernels_moe.cu:775-788 (SwiGLU, MoVA combine), :527-573 (grouping), :2023-2112 (cache), :2196-2201 (pack).
#include <math.h>

#include "common.cuh"
#include "route.cuh"
#include "seed_block.cuh"

namespace nsl {

// ---- router ------------------------------------------------------------------------------------------------------------
// One warp per row (route_row in route.cuh).
template <int PER>                   // experts per lane held in registers: E <= 32 * PER
__global__ void __launch_bounds__(128) route_kernel(int E, int k, const float* __restrict__ logits, int ld,
                                                    int32_t* __restrict__ ind, float* __restrict__ wt, int T) {
    const int lane = threadIdx.x & 31, t = blockIdx.x * 4 + (threadIdx.x >> 5);
    grid_dependents_go();   // a dependent launch of the next kernel may bring its blocks in as these retire
    if (t >= T) return;
    route_row<PER>(E, k, logits + (size_t) t * ld, lane, ind + (size_t) t * k, wt + (size_t) t * k);
}

// ---- elementwise --------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_bf16(float g) {
    const float s = bf16_round(1.0f / (1.0f + expf(-g)));
    return bf16_round(g * s);
}
__global__ void swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ a, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        a[i] = bf16_round(silu_bf16(g[i]) * u[i]);
}

// The same values as bf16 bits (they are bf16 values already): the packed input of the down projection's GEMM.
__global__ void swiglu_packed_kernel(const float* __restrict__ g, const float* __restrict__ u, uint16_t* __restrict__ a, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n / 2; i += gridDim.x * blockDim.x) {
        const float2 gv = ((const float2*) g)[i], uv = ((const float2*) u)[i];
        const uint32_t lo = __float_as_uint(bf16_round(silu_bf16(gv.x) * uv.x)) >> 16, hi = __float_as_uint(bf16_round(silu_bf16(gv.y) * uv.y)) & 0xFFFF0000u;
        ((uint32_t*) a)[i] = lo | hi;
    }
}

// out[t][i] = sigmoid(sg[t*sgld]) sh[t][i] + sum_j wt[t][j] D[t*k+j][i], plain f32, j ascending; sh == NULL: no shared
// expert term.
__global__ void q4_combine_kernel(int d, int k, const float* __restrict__ D, const float* __restrict__ wt,
                                  const float* __restrict__ sh, const float* __restrict__ sg, int sgld, float* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    grid_dependents_go();
    grid_dependency_wait();
    if (i >= d) return;
    float a = 0.0f;
    if (sh) a = (1.0f / (1.0f + expf(-sg[(size_t) t * sgld]))) * sh[(size_t) t * d + i];
    for (int j = 0; j < k; ++j) a += wt[t * k + j] * D[((size_t) t * k + j) * d + i];
    out[(size_t) t * d + i] = a;
}

// x = bf16(x + bf16(bf16(sum_j bf16(D_j bf16(w_j))) + shared))
__global__ void moe_combine_kernel(const float* __restrict__ D, const float* __restrict__ w, const float* __restrict__ shared,
                                   float* __restrict__ x, int d, int k) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (c >= d) return;
    float s = 0.0f;
    for (int j = 0; j < k; ++j) s += bf16_round(__fmul_rn(D[((size_t) t * k + j) * d + c], bf16_round(w[t * k + j])));
    const size_t i = (size_t) t * d + c;
    x[i] = bf16_round(x[i] + bf16_round(bf16_round(s) + shared[i]));
}

__global__ void pack_bf16_kernel(const float* __restrict__ x, uint16_t* __restrict__ y, size_t n) {
    const size_t n8 = n / 8;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t) gridDim.x * blockDim.x) {
        const float4 a = ((const float4*) x)[2 * i], b = ((const float4*) x)[2 * i + 1];
        uint4 o;
        o.x = bf16_bits(a.x) | ((uint32_t) bf16_bits(a.y) << 16);
        o.y = bf16_bits(a.z) | ((uint32_t) bf16_bits(a.w) << 16);
        o.z = bf16_bits(b.x) | ((uint32_t) bf16_bits(b.y) << 16);
        o.w = bf16_bits(b.z) | ((uint32_t) bf16_bits(b.w) << 16);
        ((uint4*) y)[i] = o;
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) y[n8 * 8 + threadIdx.x] = bf16_bits(x[n8 * 8 + threadIdx.x]);
}

// ---- grouping ---------------------------------------------------------------------------------------------------------
// work (2n+3 ints): [0] tile count, [1..n+1] pair offset of each expert, [n+2..2n+2] tile offset of each expert.
// One block: histogram by shared-memory atomics, then an inclusive scan of pairs and tiles over the experts.
__global__ void __launch_bounds__(1024) bucket_count_kernel(const int32_t* __restrict__ inds, int count, int n,
                                                            int32_t* __restrict__ work) {
    __shared__ int cnt[BUCKET_MAX_EXPERTS];
    __shared__ int psum[BUCKET_MAX_EXPERTS], tsum[BUCKET_MAX_EXPERTS];
    const int tid = threadIdx.x;
    cnt[tid] = 0;
    __syncthreads();
    for (int i = tid; i < count; i += 1024) {
        const int e = inds[i];
        if (e >= 0 && e < n) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    const int c = tid < n ? cnt[tid] : 0;
    psum[tid] = c;
    tsum[tid] = (c + MMT_BN - 1) / MMT_BN;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {   // Hillis-Steele inclusive scan
        const int pv = tid >= o ? psum[tid - o] : 0, tv = tid >= o ? tsum[tid - o] : 0;
        __syncthreads();
        psum[tid] += pv;
        tsum[tid] += tv;
        __syncthreads();
    }
    if (tid < n) {
        work[1 + tid] = psum[tid] - c;
        work[2 + n + tid] = tsum[tid] - (c + MMT_BN - 1) / MMT_BN;
    }
    if (tid == n - 1 || (n == 0 && tid == 0)) {
        work[1 + n] = n ? psum[tid] : 0;
        work[2 + 2 * n] = n ? tsum[tid] : 0;
        work[0] = n ? tsum[tid] : 0;
    }
}
// One block per expert.  Each warp owns a contiguous range of the pair list: it counts its matches, the block scans the
// 32 counts, then each warp writes its matches in order (a ballot prefix), so perm is ascending within the expert.
__global__ void __launch_bounds__(1024) bucket_place_kernel(const int32_t* __restrict__ inds, int count,
                                                            const int32_t* __restrict__ work, int32_t* __restrict__ perm,
                                                            MmTile* __restrict__ tiles) {
    __shared__ int wcount[32];
    const int e = blockIdx.x, n = gridDim.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int begin = work[1 + e], total = work[2 + e] - begin;
    if (total > 0) {
        const int per = ((count + 31) / 32 + 31) & ~31;   // pairs per warp, a multiple of 32
        const int lo = w * per, hi = lo + per < count ? lo + per : count;
        int mine = 0;
        for (int i = lo + lane; i - lane < hi; i += 32) {
            const bool f = i < hi && inds[i] == e;
            mine += __popc(__ballot_sync(FULL, f));
        }
        if (lane == 0) wcount[w] = mine;
        __syncthreads();
        int at = begin;
        for (int q = 0; q < w; ++q) at += wcount[q];
        for (int i = lo + lane; i - lane < hi; i += 32) {
            const bool f = i < hi && inds[i] == e;
            const uint32_t m = __ballot_sync(FULL, f);
            if (f) perm[at + __popc(m & ((1u << lane) - 1u))] = i;
            at += __popc(m);
        }
        const int t0 = work[2 + n + e];
        for (int t = tid; t * MMT_BN < total; t += 1024) {
            MmTile tl = {e, begin + t * MMT_BN, total - t * MMT_BN < MMT_BN ? total - t * MMT_BN : MMT_BN, 0};
            tiles[t0 + t] = tl;
        }
    }
}

// ---- expert cache -----------------------------------------------------------------------------------------------------
// Policy (engine/kernels_cuda.h:26-55): the units a call needs are marked; hits get the new tick; misses, in expert order,
// take the least recently used slots (ties: lowest slot) among those this call has not touched and, with
// CACHE_PROTECT_PREV, the previous admit did not touch; a taken slot's old unit is evicted, the unit's slice tables are
// pointed at the slot and a (unit, slot) copy job is queued.  When fewer slots may be replaced than there are misses,
// the remaining misses are left out (njobs = admitted count).
//
// How it is computed here (one block, no serial loop over the misses).  Taking the LRU slot m times in a row is the
// same as taking the m smallest (last use, slot) keys among the replaceable slots, in order.  So: (1) an MSB-first
// radix select over the 32-bit last-use ticks finds the tick of the m-th victim and how many slots lie below it;
// (2) one ordered pass in slot order collects the victims: every replaceable slot below that tick, and of those equal to
// it the lowest slots that are still needed; (3) the victims (at most 1024, in shared memory) are ranked by counting;
// (4) thread r pairs the r-th miss with the victim of rank r and rewrites the tables for it -- all misses at once.
constexpr int ADMIT_T = CACHE_MAX_PER_LAYER;   // threads of the block = the most units one layer has

__device__ __forceinline__ bool slot_replaceable(uint32_t last, uint32_t now, uint32_t prev) { return last != now && last != prev; }

// Exclusive position of this thread's flag among the block's flags (thread order) and their total; `carry` is shared.
__device__ __forceinline__ int block_rank(bool flag, int* wsum, int& total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const uint32_t m = __ballot_sync(FULL, flag);
    __syncthreads();            // wsum may still be read from the previous call
    if (lane == 0) wsum[w] = __popc(m);
    __syncthreads();
    int before = 0, all = 0;
    for (int q = 0; q < ADMIT_T / 32; ++q) { const int c = wsum[q]; if (q < w) before += c; all += c; }
    total = all;
    return before + __popc(m & ((1u << lane) - 1u));
}

__global__ void __launch_bounds__(ADMIT_T) cache_admit_kernel(CachePool p, int sl, const int32_t* __restrict__ inds,
                                                              int count, int flags) {
    __shared__ int need[ADMIT_T];                    // expert -> needed by this call
    __shared__ int miss_of[ADMIT_T];                 // r -> the r-th missing expert (ascending)
    __shared__ unsigned long long vict[ADMIT_T];     // victims' (last use, slot) keys, in slot order
    __shared__ int hist[256];
    __shared__ int wsum[ADMIT_T / 32];
    __shared__ uint32_t sel_prefix;
    __shared__ int sel_remaining;
    const int tid = threadIdx.x;
    const uint32_t prev = (flags & CACHE_PROTECT_PREV) ? p.tick[0] : 0xFFFFFFFFu;
    const uint32_t now = p.tick[0] + 1;
    need[tid] = 0;
    __syncthreads();
    for (int i = tid; i < count; i += ADMIT_T) {
        const int e = inds[i];
        if (e >= 0 && e < p.per_layer) need[e] = 1;
    }
    __syncthreads();
    // hits are touched, misses listed in expert order
    const bool wanted = tid < p.per_layer && need[tid];
    const int held = wanted ? p.unit_slot[(size_t) sl * p.per_layer + tid] : -1;
    if (wanted && held >= 0) p.slot_last[held] = now;
    int n_need, n_miss;
    block_rank(wanted, wsum, n_need);
    const bool missing = wanted && held < 0;
    const int mpos = block_rank(missing, wsum, n_miss);
    if (missing) miss_of[mpos] = tid;
    __syncthreads();          // the hits' new ticks are visible to the whole block from here on
    // how many slots may be replaced
    int mine = 0;
    for (int s = tid; s < p.slots; s += ADMIT_T) mine += slot_replaceable(p.slot_last[s], now, prev);
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    if (mine) atomicAdd(&hist[0], mine);
    __syncthreads();
    const int n_free = hist[0];
    const int n_adm = n_miss < n_free ? n_miss : n_free;      // victims wanted
    if (tid == 0) {
        p.tick[0] = now;
        p.stats[0] += (uint32_t) (n_need - n_miss);
        p.stats[1] += (uint32_t) n_miss;
        *p.njobs = n_adm;
        sel_prefix = 0u;
        sel_remaining = n_adm;
    }
    __syncthreads();
    if (n_adm == 0) return;
    // (1) the tick of the n_adm-th smallest replaceable slot, one byte per pass from the top
    uint32_t known = 0u;      // mask of the bits already fixed
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = sel_prefix;
        for (int s = tid; s < p.slots; s += ADMIT_T) {
            const uint32_t last = p.slot_last[s];
            if (slot_replaceable(last, now, prev) && (last & known) == prefix) atomicAdd(&hist[(last >> shift) & 255u], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int left = sel_remaining, b = 0;
            while (b < 255 && hist[b] < left) left -= hist[b++];
            sel_remaining = left;                 // rank inside bin b, 1-based
            sel_prefix = prefix | ((uint32_t) b << shift);
        }
        known |= 255u << shift;
        __syncthreads();
    }
    const uint32_t cut = sel_prefix;               // every replaceable slot older than `cut` is a victim,
    const int want_eq = sel_remaining;             // and the `want_eq` lowest slots whose tick equals it
    // (2) the victims, gathered in slot order
    int n_lt = 0, n_eq = 0;
    for (int base = 0; base < p.slots; base += ADMIT_T) {
        const int s = base + tid;
        const uint32_t last = s < p.slots ? p.slot_last[s] : now;
        const bool ok = s < p.slots && slot_replaceable(last, now, prev);
        int t_lt, t_eq;
        const int r_lt = block_rank(ok && last < cut, wsum, t_lt);
        const int r_eq = block_rank(ok && last == cut, wsum, t_eq);
        const unsigned long long key = ((unsigned long long) last << 32) | (uint32_t) s;
        // older slots fill the list's front part from the left, equal ones its last want_eq entries
        if (ok && last < cut) vict[n_lt + r_lt] = key;
        if (ok && last == cut && n_eq + r_eq < want_eq) vict[(n_adm - want_eq) + n_eq + r_eq] = key;
        n_lt += t_lt;
        n_eq += t_eq;
    }
    __syncthreads();
    // (3) + (4): thread t owns victim t, finds its rank among the victims and serves the miss of that rank
    if (tid < n_adm) {
        const unsigned long long key = vict[tid];
        int rank = 0;
        for (int j = 0; j < n_adm; ++j) rank += vict[j] < key;
        const int slot = (int) (key & 0xFFFFFFFFu), x = miss_of[rank], u = sl * p.per_layer + x;
        const int old = p.slot_unit[slot];
        if (old >= 0) p.unit_slot[old] = -1;
        p.slot_unit[slot] = u;
        p.unit_slot[u] = slot;
        p.slot_last[slot] = now;
        p.jobs[2 * rank] = u;
        p.jobs[2 * rank + 1] = slot;
        uint8_t* base = p.vram + (uint64_t) slot * p.unit_bytes;
        for (int i = 0; i < p.ntens; ++i) {
            WSlice* t = p.tab + ((size_t) sl * p.ntens + i) * p.per_layer + x;
            for (int st = 0; st < 4; ++st)
                if (p.off[i][st] != 0xFFFFFFFFu) t->p[st] = base + p.off[i][st];
        }
    }
}

// Copy (grid = the caller's block count): the queued units, as one long run of 16-byte words (job after job), are dealt
// to the blocks in contiguous shares, so a block streams a few long host ranges (mapped pinned memory, read over PCIe by
// the kernel itself) instead of striding over every unit; eight loads in flight per thread.
__global__ void __launch_bounds__(512) cache_copy_kernel(CachePool p) {
    const int nj = *p.njobs;
    if (nj <= 0) return;
    const uint64_t per_unit = p.unit_bytes / 16, total = per_unit * (uint64_t) nj;
    const uint64_t lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    uint64_t at = lo;
    while (at < hi) {
        const int j = (int) (at / per_unit);
        const uint64_t w0 = at - (uint64_t) j * per_unit;
        const uint64_t n = (hi - at) < (per_unit - w0) ? (hi - at) : (per_unit - w0);     // words of job j in this share
        const uint4* src = (const uint4*) (p.host + (uint64_t) p.jobs[2 * j] * p.unit_bytes) + w0;
        uint4* dst = (uint4*) (p.vram + (uint64_t) p.jobs[2 * j + 1] * p.unit_bytes) + w0;
        uint64_t i = threadIdx.x;
        for (; i + 7 * 512 < n; i += 8 * 512) {
            uint4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) v[q] = src[i + q * 512];
#pragma unroll
            for (int q = 0; q < 8; ++q) dst[i + q * 512] = v[q];
        }
        for (; i < n; i += 512) dst[i] = src[i];
        at += n;
    }
}


// ---- grouping without caller-provided work memory ---------------------------------------------------------------------
// The offsets that bucket_count_kernel hands to bucket_place_kernel (2 n + 3 ints) live here instead of in a buffer the
// caller allocates.  One array per GPU that loads the library, held until the process exits; sized for the largest
// expert count the grouping accepts.
constexpr int BUCKET_SCRATCH_INTS = 2 * BUCKET_MAX_EXPERTS + 3;
static __device__ __align__(256) int32_t g_bucket_scratch[BUCKET_SCRATCH_INTS];

__global__ void bucket_publish_kernel(const int32_t* __restrict__ work, int32_t* __restrict__ ntiles_out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) ntiles_out[0] = work[0];
}

// The array's device address on the current device.  In host code the symbol's name is only a host-side handle, not an
// address a kernel can use, so the address is asked for once per device with that device current.
static int32_t* bucket_scratch_ptr() {
    static int32_t* ptr[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_error("nsl_bucket_noalloc: no current device"); return NULL; }
    if (!ptr[dev]) {
        void* p = NULL;
        const cudaError_t rc = cudaGetSymbolAddress(&p, g_bucket_scratch);
        if (rc != cudaSuccess || !p) { set_error("nsl_bucket_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(rc)); return NULL; }
        ptr[dev] = (int32_t*) p;
    }
    return ptr[dev];
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void nsl_route(cudaStream_t s, int n_exp, int top_k, const float* logits, int ld, int32_t* ind, float* wt, int T) {
    if (T <= 0) return;
    if (n_exp < 1 || n_exp > 32 * ROUTE_PER_LANE || top_k < 1 || top_k > 32 || top_k > n_exp) {
        set_error("router: %d experts (at most %d), top %d (at most 32)", n_exp, 32 * ROUTE_PER_LANE, top_k);
        return;
    }
    const dim3 grid((unsigned) (T + 3) / 4);
    if (n_exp <= 128) route_kernel<4><<<grid, 128, 0, s>>>(n_exp, top_k, logits, ld, ind, wt, T);
    else if (n_exp <= 512) route_kernel<16><<<grid, 128, 0, s>>>(n_exp, top_k, logits, ld, ind, wt, T);
    else route_kernel<32><<<grid, 128, 0, s>>>(n_exp, top_k, logits, ld, ind, wt, T);
    count_launch();
}
void kq4_route_ld(cudaStream_t s, const void* cfg, const float* logits, int ld, int32_t* ind, float* wt, int T) {
    const int* c = (const int*) cfg;   // Qwen4Cfg: n_exp and top_k are its 22nd and 23rd ints
    nsl_route(s, c[21], c[22], logits, ld, ind, wt, T);
}
void kq4_route(cudaStream_t s, const void* cfg, const float* logits, int32_t* ind, float* wt, int T) {
    kq4_route_ld(s, cfg, logits, ((const int*) cfg)[21], ind, wt, T);
}

void kq4_moe_combine(cudaStream_t s, int d, int k, const float* D, const float* wt, const float* sh, const float* sg,
                     int sgld, float* out, int T) {
    if (T <= 0 || d <= 0) return;
    launch(q4_combine_kernel, dim3((unsigned) (d + 255) / 256, (unsigned) T), 256, 0, s, d, k, D, wt, sh, sg, sgld, out);
    count_launch();
}

void kc_swiglu(cudaStream_t s, const float* g, const float* u, float* a, int n) {
    if (n <= 0) return;
    const int blocks = (n + 255) / 256;
    swiglu_kernel<<<blocks < sm_count() * 16 ? blocks : sm_count() * 16, 256, 0, s>>>(g, u, a, n);
    count_launch();
}

// kc_swiglu with the result as packed bf16 (n even): what kc_mm_grouped_packed reads.
void nsl_swiglu_packed(cudaStream_t s, const float* g, const float* u, uint16_t* a, int n) {
    if (n <= 0) return;
    const int blocks = (n / 2 + 255) / 256;
    swiglu_packed_kernel<<<blocks < sm_count() * 16 ? blocks : sm_count() * 16, 256, 0, s>>>(g, u, a, n);
    count_launch();
}

void kc_moe_combine(cudaStream_t s, const float* D, const float* w, const float* shared, float* x, int d, int k, int T) {
    if (T <= 0 || d <= 0) return;
    moe_combine_kernel<<<dim3((unsigned) (d + 255) / 256, (unsigned) T), 256, 0, s>>>(D, w, shared, x, d, k);
    count_launch();
}

void kc_pack_input_bf16(cudaStream_t s, const float* x, uint16_t* y, size_t n) {
    if (!n) return;
    const size_t blocks = (n / 8 + 255) / 256 + 1;
    pack_bf16_kernel<<<(unsigned) (blocks < (size_t) sm_count() * 16 ? blocks : (size_t) sm_count() * 16), 256, 0, s>>>(x, y, n);
    count_launch();
}

void kc_bucket(cudaStream_t s, const int32_t* inds, int count, int n, int32_t* perm, MmTile* tiles, int32_t* ntiles) {
    if (n < 1 || n > BUCKET_MAX_EXPERTS) { set_error("kc_bucket: %d experts, at most %d", n, BUCKET_MAX_EXPERTS); return; }
    bucket_count_kernel<<<1, 1024, 0, s>>>(inds, count, n, ntiles);
    bucket_place_kernel<<<(unsigned) n, 1024, 0, s>>>(inds, count, ntiles, perm, tiles);
    count_launch(2);
}

void nsl_bucket_noalloc(cudaStream_t s, const int32_t* inds, int count, int n, int32_t* perm, MmTile* tiles, int32_t* ntiles_out) {
    if (n < 1 || n > BUCKET_MAX_EXPERTS) {
        set_error("nsl_bucket_noalloc: %d experts, the built-in work array holds at most %d", n, BUCKET_MAX_EXPERTS);
        return;
    }
    int32_t* work = bucket_scratch_ptr();
    if (!work) return;
    // every entry the placement reads is rewritten by the count kernel, so nothing has to be cleared between calls
    bucket_count_kernel<<<1, 1024, 0, s>>>(inds, count, n, work);
    bucket_place_kernel<<<(unsigned) n, 1024, 0, s>>>(inds, count, work, perm, tiles);
    bucket_publish_kernel<<<1, 32, 0, s>>>(work, ntiles_out);
    count_launch(3);
}

void kc_cache_admit(cudaStream_t s, const CachePool* p, int sl, const int32_t* inds, int count, int flags) {
    if (p->per_layer > CACHE_MAX_PER_LAYER) { set_error("expert cache: %d experts per layer, at most %d", p->per_layer, CACHE_MAX_PER_LAYER); return; }
    cache_admit_kernel<<<1, CACHE_MAX_PER_LAYER, 0, s>>>(*p, sl, inds, count, flags);
    count_launch();
}
void kc_cache_copy(cudaStream_t s, const CachePool* p, int blocks) {
    if (blocks < 1) blocks = 1;
    cache_copy_kernel<<<(unsigned) blocks, 512, 0, s>>>(*p);
    count_launch();
}

}   // extern "C"
