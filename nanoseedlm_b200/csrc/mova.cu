// The MoVA engine's router and its SEED4P4 per-head maps (the projections of its latent attention).
//
// Router (engine/kernels_moe.cu:717-772, nslm/lib_mova_ref.c:171-201): one block per row computes every expert's
// two-partition BF16 logit, the sigmoid scores and the selection scores, then picks the top k by RANK: thread e counts
// the experts that beat expert e (a larger selection score, or an equal one with a lower id), and the experts with rank
// < k land in rank order.  No rounds of arg max, no serial dependency on k.
//
// Per-head maps (engine/kernels_moe.cu:1147-1175, 1325-1335): a stacked [H*O][I] seed matrix whose exponent bias changes
// per head.  The mat-vec shares one expansion of a block among up to 8 rows of input; lanes of a warp split a weight row's
// blocks, several weight rows per warp when a row has fewer than 32 blocks.
#include "common.cuh"
#include "seed_block.cuh"

namespace nsl {

#define ROUTER_MAX_N 1024
#define ROUTER_MAX_K 64
#define ROUTER_THREADS 256

__device__ __forceinline__ float warp_total(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// The k best of n by selection score (ties to the lowest id), from shared memory; every thread of the block calls it.
__device__ __forceinline__ void topk_by_rank(const float* s_sc, const float* s_sel, int* s_ch, int n, int k, float scale,
                                             int32_t* inds, float* wts) {
    for (int j = threadIdx.x; j < k; j += blockDim.x) s_ch[j] = 0;
    __syncthreads();
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
        const float my = s_sel[e];
        int rank = 0;
        for (int j = 0; j < n; ++j) {
            const float v = s_sel[j];
            rank += (v > my) || (v == my && j < e);
        }
        if (rank < k) s_ch[rank] = e;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (int j = 0; j < k; ++j) sum += s_sc[s_ch[j]];   // in pick order, as the reference sums
        for (int j = 0; j < k; ++j) {
            inds[j] = s_ch[j];
            wts[j] = s_sc[s_ch[j]] / sum * scale;
        }
    }
}

__global__ void __launch_bounds__(ROUTER_THREADS) router_kernel(RouterArgs a, const uint16_t* __restrict__ W,
                                                               const uint16_t* __restrict__ bias, const float* __restrict__ x,
                                                               float* score, float* sel, int32_t* inds, float* wts) {
    __shared__ float s_sc[ROUTER_MAX_N], s_sel[ROUTER_MAX_N];
    __shared__ int s_ch[ROUTER_MAX_K];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* xr = x + (size_t) t * a.d;
    for (int e = warp; e < a.n; e += ROUTER_THREADS / 32) {
        const uint16_t* wr = W + (size_t) e * a.d;
        float s0 = 0.0f, s1 = 0.0f;
        for (int c = lane * 8; c < a.d; c += 256) {
            const uint4 w = __ldg((const uint4*) (wr + c));
            const float4 x0 = __ldg((const float4*) (xr + c)), x1 = __ldg((const float4*) (xr + c + 4));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float wf = __uint_as_float((i & 1) ? (ww[i >> 1] & 0xFFFF0000u) : (ww[i >> 1] << 16));
                if (c + i < a.hw) s0 = fmaf(wf, xv[i], s0);
                else s1 = fmaf(wf, xv[i], s1);
            }
        }
        s0 = warp_total(s0);
        s1 = warp_total(s1);
        if (lane == 0) {
            const float sg = 1.0f / (1.0f + expf(-(bf16_round(s0) + bf16_round(s1))));
            const float se = sg + __uint_as_float((uint32_t) bias[e] << 16);
            s_sc[e] = sg;
            s_sel[e] = se;
            score[(size_t) t * a.n + e] = sg;
            sel[(size_t) t * a.n + e] = se;
        }
    }
    __syncthreads();
    topk_by_rank(s_sc, s_sel, s_ch, a.n, a.top_k, a.scale, inds + (size_t) t * a.top_k, wts + (size_t) t * a.top_k);
}

__global__ void __launch_bounds__(ROUTER_THREADS) router_topk_kernel(RouterArgs a, const float* __restrict__ score,
                                                                    const float* __restrict__ sel, int32_t* inds, float* wts) {
    __shared__ float s_sc[ROUTER_MAX_N], s_sel[ROUTER_MAX_N];
    __shared__ int s_ch[ROUTER_MAX_K];
    const int t = blockIdx.x;
    for (int e = threadIdx.x; e < a.n; e += ROUTER_THREADS) {
        s_sc[e] = score[(size_t) t * a.n + e];
        s_sel[e] = sel[(size_t) t * a.n + e];
    }
    __syncthreads();
    topk_by_rank(s_sc, s_sel, s_ch, a.n, a.top_k, a.scale, inds + (size_t) t * a.top_k, wts + (size_t) t * a.top_k);
}

// ---- per-head maps ----------------------------------------------------------------------------------------------------
#define HMV_THREADS 256
#define HMV_TOKENS 8

__device__ __forceinline__ float softplus_gate(float g) {   // softplus with beta = ln 2 in f32, then BF16
    const float gx = g * 0.69314718055994531f;
    return bf16_round((fmaxf(gx, 0.0f) + logf(1.0f + expf(-fabsf(gx)))) / 0.69314718055994531f);
}

// lpr lanes share a weight row (a power of two <= 32); blockIdx.y picks a group of HMV_TOKENS rows of input.
__global__ void __launch_bounds__(HMV_THREADS) heads_mv_kernel(HmvArgs a, WSlice W, KConst kc, const uint32_t* __restrict__ G,
                                                              const float* __restrict__ x, const float* __restrict__ g,
                                                              float* __restrict__ y, int T, int lpr) {
    __shared__ StreamTab tab;
    load_stream_tab(tab, G, threadIdx.x, HMV_THREADS);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nb = a.I / 8, rpw = 32 / lpr, sub = lane / lpr, ln = lane % lpr;
    const int rows = a.H * a.O, t0 = blockIdx.y * HMV_TOKENS, nt = min(HMV_TOKENS, T - t0);
    const int32_t* head_bias = (const int32_t*) W.p[2];
    for (int base = (blockIdx.x * (HMV_THREADS / 32) + warp) * rpw; base < rows; base += gridDim.x * (HMV_THREADS / 32) * rpw) {
        const bool ok = base + sub < rows;
        const int row = ok ? base + sub : rows - 1;
        const int h = row / a.O, o = row - h * a.O;
        float s[HMV_TOKENS];
#pragma unroll
        for (int t = 0; t < HMV_TOKENS; ++t) s[t] = 0.0f;
        for (int j = ln; j < nb; j += lpr) {
            const size_t gidx = (size_t) row * nb + j;
            const uint32_t seed = __ldg((const uint16_t*) W.p[0] + gidx), cw = __ldg((const uint16_t*) W.p[1] + gidx);
            const uint32_t code = (__ldg((const uint8_t*) W.p[3] + (gidx >> 1)) >> ((gidx & 1) * 4)) & 15u;
            const uint32_t sb = stream_bits(tab, seed);
            float v[32], q[4];
            block_states(seed | (sb << 16), sb, v);
            block_coefs(cw, kc, q);
            const float e2 = __uint_as_float((code << 23) | 0x38000000u);
#pragma unroll
            for (int t = 0; t < HMV_TOKENS; ++t) {
                if (t >= nt) break;
                const float* xp = x + (size_t) (t0 + t) * a.xs + (size_t) h * a.hs + (size_t) j * 8;
                float xr[8], xo[4];
#pragma unroll
                for (int c = 0; c < 8; ++c) xr[c] = __ldg(xp + c) * NSL_XSCALE;
                block_offsets(xr, xo);
                s[t] = fmaf(states_dot(v, q, xr, xo), e2, s[t]);
            }
        }
        const float sc = slice_scale(__ldg(head_bias + h));
#pragma unroll
        for (int t = 0; t < HMV_TOKENS; ++t) {
            if (t >= nt) break;
            float st = s[t];
            for (int d = lpr >> 1; d > 0; d >>= 1) st += __shfl_xor_sync(0xFFFFFFFFu, st, d);
            if (ok && ln == 0) {
                const size_t yi = ((size_t) (t0 + t) * a.H + h) * a.O + o;
                float r = bf16_round(st * sc);
                if (a.gate) r = bf16_round(r * softplus_gate(__ldg(g + yi)));
                y[yi] = r;
            }
        }
    }
}

// One thread per block of 8 weights: the exact f32 weights rounded to BF16, the exponent bias by head.
__global__ void __launch_bounds__(256) heads_deq_kernel(WSlice W, KConst kc, const uint32_t* __restrict__ G, int O, int nb,
                                                        size_t nblk, uint4* __restrict__ out) {
    __shared__ StreamTab tab;
    load_stream_tab(tab, G, threadIdx.x, 256);
    __syncthreads();
    const int32_t* head_bias = (const int32_t*) W.p[2];
    for (size_t gidx = (size_t) blockIdx.x * 256 + threadIdx.x; gidx < nblk; gidx += (size_t) gridDim.x * 256) {
        const uint32_t seed = __ldg((const uint16_t*) W.p[0] + gidx), cw = __ldg((const uint16_t*) W.p[1] + gidx);
        const int code = (__ldg((const uint8_t*) W.p[3] + (gidx >> 1)) >> ((gidx & 1) * 4)) & 15;
        const int h = (int) (gidx / (size_t) nb / (size_t) O);
        const uint32_t sb = stream_bits(tab, seed);
        float wv[8];
        block_weights(seed | (sb << 16), sb, cw, exact_scale45(__ldg(head_bias + h) + code), kc, wv);
        out[gidx] = make_uint4(bf16x2_bits(wv[0], wv[1]), bf16x2_bits(wv[2], wv[3]), bf16x2_bits(wv[4], wv[5]),
                               bf16x2_bits(wv[6], wv[7]));
    }
}

static bool router_args_ok(const RouterArgs& a, const char* who) {
    if (a.n < 1 || a.n > ROUTER_MAX_N || a.top_k < 1 || a.top_k > ROUTER_MAX_K || a.top_k > a.n) {
        set_error("%s: n %d (1..%d) or top_k %d (1..%d, <= n) out of range", who, a.n, ROUTER_MAX_N, a.top_k, ROUTER_MAX_K);
        return false;
    }
    return true;
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void kc_router(cudaStream_t s, RouterArgs a, const uint16_t* W, const uint16_t* bias, const float* x, float* score,
               float* sel, int32_t* inds, float* wts, int T) {
    if (!router_args_ok(a, "kc_router") || T <= 0) return;
    if (a.d % 8 || !aligned16(W) || !aligned16(x)) {
        set_error("kc_router: d %d must be a multiple of 8 and W, x 16-byte aligned", a.d);
        return;
    }
    router_kernel<<<(unsigned) T, ROUTER_THREADS, 0, s>>>(a, W, bias, x, score, sel, inds, wts);
    count_launch();
}

void kc_router_topk(cudaStream_t s, RouterArgs a, const float* score, const float* sel, int32_t* inds, float* wts, int T) {
    if (!router_args_ok(a, "kc_router_topk") || T <= 0) return;
    router_topk_kernel<<<(unsigned) T, ROUTER_THREADS, 0, s>>>(a, score, sel, inds, wts);
    count_launch();
}

void kc_heads_mv(cudaStream_t s, HmvArgs a, int fmt, WSlice W, const uint32_t* G, const float* x, const float* g, float* y,
                 int T) {
    if (fmt != MF_SEED4P4) {
        set_error("kc_heads_mv: weight format %d is not served by this library (SEED4P4 = %d only)", fmt, (int) MF_SEED4P4);
        return;
    }
    if (a.H < 1 || a.O < 1 || a.I < 8 || a.I % 8 || T <= 0 || (a.gate && !g)) {
        set_error("kc_heads_mv: H %d, O %d, I %d (a multiple of 8), T %d or a missing gate", a.H, a.O, a.I, T);
        return;
    }
    int lpr = 32;
    while (lpr > a.I / 8) lpr >>= 1;
    const long long warps = ((long long) a.H * a.O + 32 / lpr - 1) / (32 / lpr);
    const long long blocks = (warps + HMV_THREADS / 32 - 1) / (HMV_THREADS / 32);
    const unsigned gx = (unsigned) (blocks < (long long) sm_count() * 8 ? blocks : (long long) sm_count() * 8);
    heads_mv_kernel<<<dim3(gx, (unsigned) ((T + HMV_TOKENS - 1) / HMV_TOKENS)), HMV_THREADS, 0, s>>>(a, W, kconst(), G, x,
                                                                                                    g ? g : x, y, T, lpr);
    count_launch();
}

void kc_heads_deq(cudaStream_t s, int fmt, WSlice W, const uint32_t* G, int H, int O, int I, uint16_t* out) {
    if (fmt != MF_SEED4P4) {
        set_error("kc_heads_deq: weight format %d is not served by this library (SEED4P4 = %d only)", fmt, (int) MF_SEED4P4);
        return;
    }
    if (H < 1 || O < 1 || I < 8 || I % 8 || !aligned16(out)) {
        set_error("kc_heads_deq: H %d, O %d, I %d (a multiple of 8) or an unaligned output", H, O, I);
        return;
    }
    const size_t nblk = (size_t) H * O * (I / 8);
    const size_t blocks = (nblk + 255) / 256, cap = (size_t) sm_count() * 16;
    heads_deq_kernel<<<(unsigned) (blocks < cap ? blocks : cap), 256, 0, s>>>(W, kconst(), G, O, I / 8, nblk, (uint4*) out);
    count_launch();
}

}   // extern "C"
