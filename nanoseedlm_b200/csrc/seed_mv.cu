// Seed-decode mat-vec kernels for sm_100a: dense (kc_mv), gathered (kc_mv_sel), fused gate+up+SwiGLU (kc_mv_gu), the
// raw-f32 variant and the bit-exact decode.  Replaces the SEED4P4 paths of the reference's k_mv / k_mv1 / k_mv_gu
// (engine/kernels_moe.cu:130-159, 222-348, 2308-2328) and the weight reader used by its tests.
//
// Data movement.  A row of K weights is K/8 blocks; a "chunk" is 8 consecutive blocks = one 16-byte load of seeds, one
// of coefficient words and one 4-byte load of exponent codes.  A lane owns one chunk position of the row (64 inputs),
// so a warp reads a row's streams as contiguous 512 + 512 + 128 bytes, and the lane's 64 inputs (plus the per-block
// centring constants) stay in registers while the warp walks over many rows: the only per-row traffic is the packed
// streams.  Rows shorter than 32 chunks share a warp (K = 512: four rows per step, eight lanes each).
//
// Arithmetic per block: the dot form of seed_block.cuh (32 fused multiply-adds on 32 masked stream words, then the
// four coefficients and the block's 2^code).  A token's sum is formed in the same order whatever the number of tokens
// in the call (chunks ascending within a lane, blocks ascending within a chunk, then a butterfly over the row's
// lanes), so a row of a multi-token call equals the single-token call bit for bit, as the reference requires
// (tests/test_mova_kernels.c:173-183).
#include <math.h>

#include "common.cuh"
#include "seed_block.cuh"

namespace nsl {

constexpr int MV_WARPS = 8;
constexpr int MV_THREADS = 32 * MV_WARPS;
enum { MODE_ROUND = 0, MODE_GU = 2 };   // the raw-f32 store is a run-time flag of MODE_ROUND

struct MvParams {
    const WSlice* ws;     // slice table on the device (gather), or NULL: w0
    const WSlice* wu;     // gate+up: the up slices
    WSlice w0;            // dense: the slice by value
    const int32_t* sel;   // pair -> slice, or NULL (dense)
    const float* x;
    float* y;
    const uint32_t* G;
    int K, R, P, xdiv, xs, ys, add, raw;
    const int32_t* xrow;    // optional: pair p reads input row xrow[p] (instead of p / xdiv)
    const int32_t* count;   // optional: the pair count is read on the device (<= P)
    int xbf16;              // inputs are packed bf16 rows (row stride xs in bf16 elements)
    const int32_t* units;   // optional: [n][4] work units = {pair, second pair or -1 (same slice), weight prefix, 0}
    const int32_t* n_units; // their number, on the device
};

__device__ __forceinline__ float silu_bf(float g) {   // each op rounded to bf16 (engine/kernels_moe.cu:28-31)
    const float s = bf16_round(1.0f / (1.0f + expf(-g)));
    return bf16_round(g * s);
}

struct Chunk { uint4 s, c; uint32_t cd; };

__device__ __forceinline__ Chunk load_chunk(const WSlice& w, size_t chunk_index) {
    Chunk k;
    k.s = __ldg((const uint4*) w.p[0] + chunk_index);
    k.c = __ldg((const uint4*) w.p[1] + chunk_index);
    k.cd = __ldg((const uint32_t*) w.p[3] + chunk_index);
    return k;
}

// One chunk (four block pairs) against one token's 64 inputs held in registers as pairs:
// x2[bp][c] = {x[16 bp + c], x[16 bp + 8 + c]}, xm2[bp][p] likewise.  acc2 = {sum over even blocks, sum over odd blocks}.
__device__ __forceinline__ u64 chunk_dot(const StreamTab& tab, const KConst& kc, const Chunk& k, const u64* x2, const u64* xm2,
                                         u64 acc2) {
    const uint32_t sw[4] = {k.s.x, k.s.y, k.s.z, k.s.w}, cw[4] = {k.c.x, k.c.y, k.c.z, k.c.w};
#pragma unroll
    for (int bp = 0; bp < 4; ++bp) {
        u64 v[32], q[4];
        pair_states(tab, sw[bp], v);
        pair_coefs(cw[bp], kc, q);
        const u64 e2 = code_scale_pair(k.cd, bp, kc);
        acc2 = fma2(pair_dot(v, q, x2 + 8 * bp, xm2 + 4 * bp), e2, acc2);
    }
    return acc2;
}
__device__ __forceinline__ float pair_total(u64 acc2) {
    float lo, hi;
    unpack2(acc2, lo, hi);
    return lo + hi;
}

__device__ __forceinline__ float group_sum(float v, int lpr) {
    for (int o = lpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

template <int MODE>
__device__ __forceinline__ void store_out(const MvParams& a, int pair, int r, float s, float su) {
    float* yo = a.y + (size_t) pair * a.ys + r;
    if (MODE == MODE_GU) *yo = a.raw ? (s / (1.0f + expf(-s))) * su : bf16_round(silu_bf(bf16_round(s)) * bf16_round(su));
    else if (a.raw) *yo = s;
    else *yo = a.add ? bf16_round(*yo + bf16_round(s)) : bf16_round(s);   // engine/kernels_moe.cu:214
}

// ---- one token per pair, inputs in registers: rows of 1, 2, 4, .. 32 chunks (K = 64 .. 2048) -------------------------
// The work is the pair-major sequence of row steps (a step = the 32 / lanes-per-row rows a warp expands at once); every
// warp of the grid takes one contiguous, equal share of it.  A share touches one or two pairs (more only when there are
// more pairs than warps), so a warp loads a pair's inputs into registers at most that often, the shares differ by at
// most one step, and inside a share the next row's streams are prefetched while the current row is expanded.
template <int MODE>
__global__ void __launch_bounds__(MV_THREADS, 1) mv_regx_kernel(MvParams a, KConst kc, int lpr_log2) {
    __shared__ StreamTab tab;
    load_stream_tab(tab, a.G, threadIdx.x, MV_THREADS);
    grid_dependents_go();
    grid_dependency_wait();   // everything below may read what the previous kernel in the stream wrote
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    const long long nw = (long long) gridDim.x * MV_WARPS, gw = (long long) blockIdx.x * MV_WARPS + warp;
    const int P = a.count ? min(*a.count, a.P) : a.P;
    const int rs = (a.R + rpw - 1) / rpw;                 // row steps per pair
    const long long total = (long long) P * rs;
    const long long begin = gw * total / nw, end = (gw + 1) * total / nw;
    if (begin >= end) return;
    const int p_first = (int) (begin / rs), p_last = (int) ((end - 1) / rs);
    for (int pair = p_first; pair <= p_last; ++pair) {
        const int s_lo = pair == p_first ? (int) (begin - (long long) pair * rs) : 0;
        const int s_hi = pair == p_last ? (int) (end - (long long) pair * rs) : rs;
        const int slice = a.sel ? a.sel[pair] : 0;
        const WSlice wa = a.ws ? a.ws[slice] : a.w0;
        WSlice wb = wa;
        if (MODE == MODE_GU) wb = a.wu[slice];
        u64 x2[32], xm2[16];
        {
            const int xr = a.xrow ? a.xrow[pair] : pair / a.xdiv;
            float x[64], xm[32];
            if (a.xbf16) {
                const uint4* xp = (const uint4*) ((const uint16_t*) a.x + (size_t) xr * a.xs + (size_t) jc * 64);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 t = __ldg(xp + i);
                    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        x[8 * i + 2 * j] = __uint_as_float(u[j] << 16) * NSL_XSCALE;
                        x[8 * i + 2 * j + 1] = __uint_as_float(u[j] & 0xFFFF0000u) * NSL_XSCALE;
                    }
                }
            } else {
                const float4* xp = (const float4*) (a.x + (size_t) xr * a.xs + (size_t) jc * 64);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 t = __ldg(xp + i);
                    x[4 * i] = t.x * NSL_XSCALE; x[4 * i + 1] = t.y * NSL_XSCALE; x[4 * i + 2] = t.z * NSL_XSCALE; x[4 * i + 3] = t.w * NSL_XSCALE;
                }
            }
#pragma unroll
            for (int b = 0; b < 8; ++b) block_offsets(x + 8 * b, xm + 4 * b);
#pragma unroll
            for (int bp = 0; bp < 4; ++bp) {
#pragma unroll
                for (int c = 0; c < 8; ++c) x2[8 * bp + c] = pack2(x[16 * bp + c], x[16 * bp + 8 + c]);
#pragma unroll
                for (int p = 0; p < 4; ++p) xm2[4 * bp + p] = pack2(xm[8 * bp + p], xm[8 * bp + 4 + p]);
            }
        }
        const float sca = slice_scale(wa.eb), scb = slice_scale(wb.eb);
        int r = s_lo * rpw + ro;
        Chunk ka, kb;
        if (r < a.R) {
            ka = load_chunk(wa, (size_t) r * lpr + jc);
            if (MODE == MODE_GU) kb = load_chunk(wb, (size_t) r * lpr + jc);
        }
        for (int st = s_lo; st < s_hi; ++st, r += rpw) {
            const bool ok = r < a.R;
            const int rn = r + rpw;
            Chunk na, nb;
            if (st + 1 < s_hi && rn < a.R) {   // next row's streams in flight during this row's expansion
                na = load_chunk(wa, (size_t) rn * lpr + jc);
                if (MODE == MODE_GU) nb = load_chunk(wb, (size_t) rn * lpr + jc);
            }
            float s = 0.0f, su = 0.0f;
            if (ok) {
                s = pair_total(chunk_dot(tab, kc, ka, x2, xm2, 0ull));
                if (MODE == MODE_GU) su = pair_total(chunk_dot(tab, kc, kb, x2, xm2, 0ull));
            }
            s = group_sum(s, lpr) * sca;
            if (MODE == MODE_GU) su = group_sum(su, lpr) * scb;
            if (ok && jc == 0) store_out<MODE>(a, pair, r, s, su);
            ka = na;
            if (MODE == MODE_GU) kb = nb;
        }
    }
}

// One thread's share of staging a pair's inputs: 16 inputs (two blocks: chunk j of the row, block pair bp), scaled, as
// the f32x2 operands of pair_dot plus their centring constants.
__device__ __forceinline__ void stage_inputs(const MvParams& a, int xr, int j, int bp, ulonglong2* sx, ulonglong2* sm) {
    float x[16], xm[8];
    if (a.xbf16) {
        const uint4* xp = (const uint4*) ((const uint16_t*) a.x + (size_t) xr * a.xs + (size_t) j * 64 + bp * 16);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 t = __ldg(xp + i);
            const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                x[8 * i + 2 * q] = __uint_as_float(u[q] << 16) * NSL_XSCALE;
                x[8 * i + 2 * q + 1] = __uint_as_float(u[q] & 0xFFFF0000u) * NSL_XSCALE;
            }
        }
    } else {
        const float4* xp = (const float4*) (a.x + (size_t) xr * a.xs + (size_t) j * 64 + bp * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 t = __ldg(xp + i);
            x[4 * i] = t.x * NSL_XSCALE; x[4 * i + 1] = t.y * NSL_XSCALE; x[4 * i + 2] = t.z * NSL_XSCALE; x[4 * i + 3] = t.w * NSL_XSCALE;
        }
    }
    block_offsets(x, xm);
    block_offsets(x + 8, xm + 4);
#pragma unroll
    for (int cq = 0; cq < 4; ++cq) {
        ulonglong2 t;
        t.x = pack2(x[2 * cq], x[8 + 2 * cq]);
        t.y = pack2(x[2 * cq + 1], x[8 + 2 * cq + 1]);
        sx[(bp * 4 + cq) * 32 + j] = t;
    }
#pragma unroll
    for (int pq = 0; pq < 2; ++pq) {
        ulonglong2 t;
        t.x = pack2(xm[2 * pq], xm[4 + 2 * pq]);
        t.y = pack2(xm[2 * pq + 1], xm[4 + 2 * pq + 1]);
        sm[(bp * 2 + pq) * 32 + j] = t;
    }
}

// ---- one token per pair, inputs in shared memory, two blocks of 8 warps per SM ------------------------------------------
// The same arithmetic, lane mapping and order as mv_regx_kernel (so results are bit-identical), but the pair's inputs
// sit in shared memory as the f32x2 operands of pair_dot, laid out [block pair][operand pair][lane] so that a warp's
// 16-byte loads are conflict-free.  Without 96 registers of inputs a thread fits in 128 registers and 16 warps per SM
// hide the logic pipe's latencies.  Blocks take contiguous shares of the pair-major row-step sequence; inside a pair
// the block's warps take its steps round-robin.
template <int MODE>
__global__ void __launch_bounds__(MV_THREADS, 2) mv_shx_kernel(MvParams a, KConst kc, int lpr_log2) {
    __shared__ StreamTab tab;
    __shared__ __align__(16) ulonglong2 sx[4 * 4 * 32];   // [bp][c / 2][lane] = {x2[c], x2[c + 1]}
    __shared__ __align__(16) ulonglong2 sm[4 * 2 * 32];   // [bp][p / 2][lane] = {xm2[p], xm2[p + 1]}
    load_stream_tab(tab, a.G, threadIdx.x, MV_THREADS);
    grid_dependents_go();
    grid_dependency_wait();   // everything below may read what the previous kernel in the stream wrote
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    const int P = a.count ? min(*a.count, a.P) : a.P;
    const int rs = (a.R + rpw - 1) / rpw;
    const long long total = (long long) P * rs;
    const long long begin = (long long) blockIdx.x * total / gridDim.x, end = (long long) (blockIdx.x + 1) * total / gridDim.x;
    if (begin >= end) return;
    const int p_first = (int) (begin / rs), p_last = (int) ((end - 1) / rs);
    for (int pair = p_first; pair <= p_last; ++pair) {
        const int s_lo = pair == p_first ? (int) (begin - (long long) pair * rs) : 0;
        const int s_hi = pair == p_last ? (int) (end - (long long) pair * rs) : rs;
        const int slice = a.sel ? a.sel[pair] : 0;
        const WSlice wa = a.ws ? a.ws[slice] : a.w0;
        WSlice wb = wa;
        if (MODE == MODE_GU) wb = a.wu[slice];
        // this warp's first streams are requested before the inputs are staged: their DRAM latency runs under it
        int st = s_lo + warp;
        int r = st * rpw + ro;
        Chunk ka, kb;
        if (st < s_hi && r < a.R) {
            ka = load_chunk(wa, (size_t) r * lpr + jc);
            if (MODE == MODE_GU) kb = load_chunk(wb, (size_t) r * lpr + jc);
        }
        if (pair != p_first) __syncthreads();   // the previous pair's inputs are no longer read
        if (threadIdx.x < lpr * 4) {
            const int j = threadIdx.x & (lpr - 1), bp = threadIdx.x >> lpr_log2;
            stage_inputs(a, a.xrow ? a.xrow[pair] : pair / a.xdiv, j, bp, sx, sm);
        }
        __syncthreads();   // inputs staged (and, for the block's first pair, the stream table loaded)
        const float sca = slice_scale(wa.eb), scb = slice_scale(wb.eb);
        for (; st < s_hi; st += MV_WARPS, r += MV_WARPS * rpw) {
            const bool ok = r < a.R;
            const int rn = r + MV_WARPS * rpw;
            Chunk na, nb;
            if (st + MV_WARPS < s_hi && rn < a.R) {
                na = load_chunk(wa, (size_t) rn * lpr + jc);
                if (MODE == MODE_GU) nb = load_chunk(wb, (size_t) rn * lpr + jc);
            }
            u64 acc = 0ull, accu = 0ull;
            if (ok) {
                const uint32_t swa[4] = {ka.s.x, ka.s.y, ka.s.z, ka.s.w}, cwa[4] = {ka.c.x, ka.c.y, ka.c.z, ka.c.w};
                const uint32_t swb[4] = {kb.s.x, kb.s.y, kb.s.z, kb.s.w}, cwb[4] = {kb.c.x, kb.c.y, kb.c.z, kb.c.w};
#pragma unroll
                for (int bp = 0; bp < 4; ++bp) {
                    u64 x2[8], xm2[4];
#pragma unroll
                    for (int cq = 0; cq < 4; ++cq) { const ulonglong2 t = sx[(bp * 4 + cq) * 32 + jc]; x2[2 * cq] = t.x; x2[2 * cq + 1] = t.y; }
#pragma unroll
                    for (int pq = 0; pq < 2; ++pq) { const ulonglong2 t = sm[(bp * 2 + pq) * 32 + jc]; xm2[2 * pq] = t.x; xm2[2 * pq + 1] = t.y; }
                    {
                        u64 v[32], q[4];
                        pair_states(tab, swa[bp], v);
                        pair_coefs(cwa[bp], kc, q);
                        acc = fma2(pair_dot(v, q, x2, xm2), code_scale_pair(ka.cd, bp, kc), acc);
                    }
                    if (MODE == MODE_GU) {
                        u64 v[32], q[4];
                        pair_states(tab, swb[bp], v);
                        pair_coefs(cwb[bp], kc, q);
                        accu = fma2(pair_dot(v, q, x2, xm2), code_scale_pair(kb.cd, bp, kc), accu);
                    }
                }
            }
            const float s = group_sum(pair_total(acc), lpr) * sca;
            float su = 0.0f;
            if (MODE == MODE_GU) su = group_sum(pair_total(accu), lpr) * scb;
            if (ok && jc == 0) store_out<MODE>(a, pair, r, s, su);
            ka = na;
            if (MODE == MODE_GU) kb = nb;
        }
    }
}

// ---- inputs in shared memory: NT tokens share each expansion (dense verify rows), or rows longer than 32 chunks ------
// Dense: the P = NT tokens are staged once per block and the rows are split over every warp of the grid.  Gather
// (NT = 1): blocks are dealt to pairs and stage their pair's input row.
// Shared layout, per token (K * 6 bytes): the f32x2 operands of pair_dot as 16-byte units, inputs
// [block pair in chunk 0..3][operand pair 0..3][chunk], then centring constants [0..3][0..1][chunk]: the lanes of a warp
// hold consecutive chunks, so their 16-byte loads are consecutive (no bank conflicts).
template <int MODE, int NT>
__global__ void __launch_bounds__(MV_THREADS, 1) mv_smemx_kernel(MvParams a, KConst kc, int lpr_log2, int dense) {
    extern __shared__ __align__(16) float smem_f[];
    __shared__ StreamTab tab;
    load_stream_tab(tab, a.G, threadIdx.x, MV_THREADS);
    grid_dependents_go();
    grid_dependency_wait();   // everything below may read what the previous kernel in the stream wrote
    const int K = a.K, nbp = K / 16, ch = K / 64;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    const int cpp = dense ? (int) gridDim.x : ((int) gridDim.x / a.P > 0 ? (int) gridDim.x / a.P : 1);
    const long long nvc = dense ? (long long) gridDim.x : (long long) a.P * cpp;
    for (long long vc = blockIdx.x; vc < nvc; vc += gridDim.x) {
        const int pair = dense ? 0 : (int) (vc / cpp), ci = dense ? (int) blockIdx.x : (int) (vc % cpp);
        const int slice = a.sel ? a.sel[pair] : 0;
        const WSlice wa = a.ws ? a.ws[slice] : a.w0;
        WSlice wb = wa;
        if (MODE == MODE_GU) wb = a.wu[slice];
        __syncthreads();   // the previous pair's inputs are no longer read
        for (int i = threadIdx.x; i < NT * nbp; i += MV_THREADS) {
            const int t = i / nbp, bp = i % nbp;
            const float* xp = a.x + (size_t) (dense ? t : pair / a.xdiv) * a.xs + 16 * bp;
            float x[16], xm[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 v4 = __ldg((const float4*) xp + j);
                x[4 * j] = v4.x * NSL_XSCALE; x[4 * j + 1] = v4.y * NSL_XSCALE; x[4 * j + 2] = v4.z * NSL_XSCALE; x[4 * j + 3] = v4.w * NSL_XSCALE;
            }
            block_offsets(x, xm);
            block_offsets(x + 8, xm + 4);
            ulonglong2* tok = (ulonglong2*) smem_f + (size_t) t * ch * 24;
            const int jch = bp >> 2, b4 = bp & 3;
#pragma unroll
            for (int cq = 0; cq < 4; ++cq) {
                ulonglong2 v2;
                v2.x = pack2(x[2 * cq], x[8 + 2 * cq]);
                v2.y = pack2(x[2 * cq + 1], x[8 + 2 * cq + 1]);
                tok[(b4 * 4 + cq) * ch + jch] = v2;
            }
#pragma unroll
            for (int pq = 0; pq < 2; ++pq) {
                ulonglong2 v2;
                v2.x = pack2(xm[2 * pq], xm[4 + 2 * pq]);
                v2.y = pack2(xm[2 * pq + 1], xm[4 + 2 * pq + 1]);
                tok[16 * ch + (b4 * 2 + pq) * ch + jch] = v2;
            }
        }
        __syncthreads();
        const float sca = slice_scale(wa.eb), scb = slice_scale(wb.eb);
        const int wi = ci * MV_WARPS + warp, step = cpp * MV_WARPS * rpw;
        for (int rbase = wi * rpw; rbase < a.R; rbase += step) {
            const int r = rbase + ro;
            const bool ok = r < a.R;
            u64 s2[NT], su2[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) s2[t] = su2[t] = 0ull;
            if (ok) {
                for (int j = jc; j < ch; j += lpr) {
                    const Chunk ka = load_chunk(wa, (size_t) r * ch + j);
                    Chunk kb = ka;
                    if (MODE == MODE_GU) kb = load_chunk(wb, (size_t) r * ch + j);
#pragma unroll
                    for (int half = 0; half < (MODE == MODE_GU ? 2 : 1); ++half) {
                        const Chunk& k = half ? kb : ka;
                        const uint32_t sw[4] = {k.s.x, k.s.y, k.s.z, k.s.w}, cw[4] = {k.c.x, k.c.y, k.c.z, k.c.w};
#pragma unroll
                        for (int bp = 0; bp < 4; ++bp) {
                            u64 v[32], q[4];
                            pair_states(tab, sw[bp], v);
                            pair_coefs(cw[bp], kc, q);
                            const u64 e2 = code_scale_pair(k.cd, bp, kc);
#pragma unroll
                            for (int t = 0; t < NT; ++t) {
                                u64 x2[8], xm2[4];
                                const ulonglong2* tok = (const ulonglong2*) smem_f + (size_t) t * ch * 24;
#pragma unroll
                                for (int c = 0; c < 4; ++c) { const ulonglong2 u = tok[(bp * 4 + c) * ch + j]; x2[2 * c] = u.x; x2[2 * c + 1] = u.y; }
#pragma unroll
                                for (int p = 0; p < 2; ++p) { const ulonglong2 u = tok[16 * ch + (bp * 2 + p) * ch + j]; xm2[2 * p] = u.x; xm2[2 * p + 1] = u.y; }
                                const u64 d = pair_dot(v, q, x2, xm2);
                                if (half) su2[t] = fma2(d, e2, su2[t]);
                                else s2[t] = fma2(d, e2, s2[t]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float st = group_sum(pair_total(s2[t]), lpr) * sca;
                float sut = 0.0f;
                if (MODE == MODE_GU) sut = group_sum(pair_total(su2[t]), lpr) * scb;
                if (ok && jc == 0) store_out<MODE>(a, dense ? t : pair, r, st, sut);
            }
        }
    }
}

// ---- two pairs per expansion -----------------------------------------------------------------------------------------
// mv_shx_kernel over work UNITS: a unit is one or two pairs that use the same slice, and a block pair's 32 states and
// coefficients are expanded once for both.  Per pair the arithmetic and its order are those of mv_shx_kernel, so the
// results are bit-identical; what changes is that the logic-pipe work (the expansion) is shared.
// The next row step's streams travel global -> shared memory with cp.async (no registers held while they fly): one slot
// per thread and matrix, read back only by the thread that requested it.
struct ChunkSlots { uint4 s[MV_THREADS], c[MV_THREADS]; uint32_t cd[MV_THREADS]; };

__device__ __forceinline__ void chunk_request(ChunkSlots& sl, const WSlice* __restrict__ w, size_t chunk_index) {
    const unsigned long long* wp = (const unsigned long long*) w->p;   // the slice's stream addresses, re-read (L1) per request
    const void* p0 = (const void*) __ldg(wp);
    const void* p1 = (const void*) __ldg(wp + 1);
    const void* p3 = (const void*) __ldg(wp + 3);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(&sl.s[threadIdx.x])),
                 "l"((const uint4*) p0 + chunk_index) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(&sl.c[threadIdx.x])),
                 "l"((const uint4*) p1 + chunk_index) : "memory");
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned) __cvta_generic_to_shared(&sl.cd[threadIdx.x])),
                 "l"((const uint32_t*) p3 + chunk_index) : "memory");
}
__device__ __forceinline__ Chunk chunk_take(const ChunkSlots& sl) {
    Chunk k;
    k.s = sl.s[threadIdx.x];
    k.c = sl.c[threadIdx.x];
    k.cd = sl.cd[threadIdx.x];
    return k;
}

// One matrix's share of a row step for a unit: four block pairs expanded once, dotted with one or two inputs.
__device__ __forceinline__ void unit_chunk_dot(const StreamTab& tab, const KConst& kc, const Chunk& k, const ulonglong2 (*sx)[4 * 4 * 32],
                                               const ulonglong2 (*sm)[4 * 2 * 32], int jc, bool two, u64& acc0, u64& acc1) {
    const uint32_t sw[4] = {k.s.x, k.s.y, k.s.z, k.s.w}, cw[4] = {k.c.x, k.c.y, k.c.z, k.c.w};
#pragma unroll
    for (int bp = 0; bp < 4; ++bp) {
        u64 v[32], q[4];
        pair_states(tab, sw[bp], v);
        pair_coefs(cw[bp], kc, q);
        const u64 e2 = code_scale_pair(k.cd, bp, kc);
        {
            u64 x2[8], xm2[4];
#pragma unroll
            for (int cq = 0; cq < 4; ++cq) { const ulonglong2 t = sx[0][(bp * 4 + cq) * 32 + jc]; x2[2 * cq] = t.x; x2[2 * cq + 1] = t.y; }
#pragma unroll
            for (int pq = 0; pq < 2; ++pq) { const ulonglong2 t = sm[0][(bp * 2 + pq) * 32 + jc]; xm2[2 * pq] = t.x; xm2[2 * pq + 1] = t.y; }
            acc0 = fma2(pair_dot(v, q, x2, xm2), e2, acc0);
        }
        if (two) {
            u64 x2[8], xm2[4];
#pragma unroll
            for (int cq = 0; cq < 4; ++cq) { const ulonglong2 t = sx[1][(bp * 4 + cq) * 32 + jc]; x2[2 * cq] = t.x; x2[2 * cq + 1] = t.y; }
#pragma unroll
            for (int pq = 0; pq < 2; ++pq) { const ulonglong2 t = sm[1][(bp * 2 + pq) * 32 + jc]; xm2[2 * pq] = t.x; xm2[2 * pq + 1] = t.y; }
            acc1 = fma2(pair_dot(v, q, x2, xm2), e2, acc1);
        }
    }
}

constexpr int UNIT_W1 = 3, UNIT_W2 = 4;   // relative cost of a row step for one pair and for two pairs sharing an expansion

// Position x of the weighted (unit, step) sequence -> the unit that holds it and the step inside (floor).
__device__ __forceinline__ void unit_position(const int32_t* __restrict__ units, int U, int rs, long long x, int& u, int& step) {
    int lo = 0, hi = U;      // the last unit whose start (units[4u+2] * rs) is <= x
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long) units[4 * mid + 2] * rs <= x) lo = mid; else hi = mid;
    }
    const int w = units[4 * lo + 1] >= 0 ? UNIT_W2 : UNIT_W1;
    const long long in = x - (long long) units[4 * lo + 2] * rs;
    u = lo;
    step = (int) (in / w);
    if (step >= rs) { u = lo + 1; step = 0; }
}

template <int MODE>
__global__ void __launch_bounds__(MV_THREADS, 2) mv_shx2_kernel(MvParams a, KConst kc, int lpr_log2) {
    constexpr int NM = MODE == MODE_GU ? 2 : 1;
    __shared__ StreamTab tab;
    __shared__ __align__(16) ulonglong2 sx[2][4 * 4 * 32];
    __shared__ __align__(16) ulonglong2 sm[2][4 * 2 * 32];
    __shared__ __align__(16) ChunkSlots slots[NM];
    load_stream_tab(tab, a.G, threadIdx.x, MV_THREADS);
    grid_dependents_go();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    const int U = *a.n_units;
    if (U <= 0) return;
    const int rs = (a.R + rpw - 1) / rpw;
    // Blocks take equal shares of the WEIGHTED sequence of (unit, row step): a step of a two-pair unit counts
    // UNIT_W2, of a single UNIT_W1; units[4u + 2] = the weights of the units before u.
    const long long wtotal = (long long) (a.units[4 * (U - 1) + 2] + (a.units[4 * (U - 1) + 1] >= 0 ? UNIT_W2 : UNIT_W1)) * rs;
    const long long begin = (long long) blockIdx.x * wtotal / gridDim.x, end = (long long) (blockIdx.x + 1) * wtotal / gridDim.x;
    if (begin >= end) return;
    int u_first, s_first, u_last, s_last;     // [first, last) in (unit, step) order
    bool staged = false;
    unit_position(a.units, U, rs, begin, u_first, s_first);
    unit_position(a.units, U, rs, end, u_last, s_last);
    if (blockIdx.x == gridDim.x - 1) { u_last = U; s_last = 0; }
    for (int u = u_first; u <= u_last; ++u) {
        const int s_lo = u == u_first ? s_first : 0;
        const int s_hi = u == u_last ? s_last : rs;
        if (u >= U || s_lo >= s_hi) continue;
        const int pa = a.units[4 * u], pb = a.units[4 * u + 1];
        const bool two = pb >= 0;
        const int slice = a.sel[pa];
        const WSlice* wa = a.ws + slice;
        const WSlice* wb = MODE == MODE_GU ? a.wu + slice : wa;
        int st = s_lo + warp;
        int r = st * rpw + ro;
        if (st < s_hi && r < a.R) {      // this warp's first streams fly while the inputs are staged
            chunk_request(slots[0], wa, (size_t) r * lpr + jc);
            if (MODE == MODE_GU) chunk_request(slots[NM - 1], wb, (size_t) r * lpr + jc);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (staged) __syncthreads();   // the previous unit's inputs are no longer read
        staged = true;
        {
            const int half = threadIdx.x >> 7, tl = threadIdx.x & 127;   // threads 0..127 stage the first pair, 128..255 the second
            const int pair = half ? pb : pa;
            if (tl < lpr * 4 && pair >= 0)
                stage_inputs(a, a.xrow ? a.xrow[pair] : pair / a.xdiv, tl & (lpr - 1), tl >> lpr_log2, sx[half], sm[half]);
        }
        __syncthreads();
        for (; st < s_hi; st += MV_WARPS, r += MV_WARPS * rpw) {
            const bool ok = r < a.R;
            const int rn = r + MV_WARPS * rpw;
            const bool more = st + MV_WARPS < s_hi && rn < a.R;
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            u64 acc0 = 0ull, accu0 = 0ull, acc1 = 0ull, accu1 = 0ull;
            {
                Chunk k;
                if (ok) k = chunk_take(slots[0]);
                if (more) chunk_request(slots[0], wa, (size_t) rn * lpr + jc);   // the slot is free again: next step's streams
                asm volatile("cp.async.commit_group;" ::: "memory");
                if (ok) unit_chunk_dot(tab, kc, k, sx, sm, jc, two, acc0, acc1);
            }
            if (MODE == MODE_GU) {
                Chunk k;
                if (ok) k = chunk_take(slots[NM - 1]);
                if (more) chunk_request(slots[NM - 1], wb, (size_t) rn * lpr + jc);
                asm volatile("cp.async.commit_group;" ::: "memory");
                if (ok) unit_chunk_dot(tab, kc, k, sx, sm, jc, two, accu0, accu1);
            }
            const float sca = slice_scale(__ldg(&wa->eb)), scb = slice_scale(__ldg(&wb->eb));
            {
                const float s0 = group_sum(pair_total(acc0), lpr) * sca;
                float su0 = 0.0f;
                if (MODE == MODE_GU) su0 = group_sum(pair_total(accu0), lpr) * scb;
                if (ok && jc == 0) store_out<MODE>(a, pa, r, s0, su0);
            }
            if (two) {
                const float s1 = group_sum(pair_total(acc1), lpr) * sca;
                float su1 = 0.0f;
                if (MODE == MODE_GU) su1 = group_sum(pair_total(accu1), lpr) * scb;
                if (ok && jc == 0) store_out<MODE>(a, pb, r, s1, su1);
            }
        }
    }
}

// ---- any K that is a multiple of 8, any alignment: one warp per (pair or dense, row), lanes over single blocks -------
// P = 4 (SEED4P4) or 3 (SEED4: the exponent code rides in the nibble word, there is no code stream).
template <int MODE, int P>
__global__ void __launch_bounds__(MV_THREADS) mv_generic_kernel(MvParams a, KConst kc, int T) {
    __shared__ StreamTab tab;
    load_stream_tab(tab, a.G, threadIdx.x, MV_THREADS);
    grid_dependents_go();
    grid_dependency_wait();   // everything below may read what the previous kernel in the stream wrote
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nb = a.K / 8, dense = a.sel == NULL;
    const long long ntask = (long long) (dense ? 1 : a.P) * a.R;
    for (long long task = (long long) blockIdx.x * MV_WARPS + warp; task < ntask; task += (long long) gridDim.x * MV_WARPS) {
        const int pair = (int) (task / a.R), r = (int) (task % a.R);
        const int slice = a.sel ? a.sel[pair] : 0;
        const WSlice wa = a.ws ? a.ws[slice] : a.w0;
        WSlice wb = wa;
        if (MODE == MODE_GU) wb = a.wu[slice];
        float s[MV_MAXT], su[MV_MAXT];
#pragma unroll
        for (int t = 0; t < MV_MAXT; ++t) s[t] = su[t] = 0.0f;
        for (int j = lane; j < nb; j += 32) {
            const size_t gidx = (size_t) r * nb + j;
#pragma unroll
            for (int half = 0; half < (MODE == MODE_GU ? 2 : 1); ++half) {
                const WSlice& w = half ? wb : wa;
                const uint32_t seed = ((const uint16_t*) w.p[0])[gidx], cwi = ((const uint16_t*) w.p[1])[gidx];
                const uint32_t code = P == 4 ? (((const uint8_t*) w.p[3])[gidx >> 1] >> ((gidx & 1) * 4)) & 15u : cwi & 15u;
                const uint32_t g = stream_bits(tab, seed);
                const uint32_t aw = seed | (g << 16);
                float v[32], q[4];
                if (P == 4) { block_states(aw, g, v); block_coefs(cwi, kc, q); }
                else { block_states3(aw, g, v); block_coefs3(cwi, kc, q); }
                const float e2 = __uint_as_float((code << 23) | 0x38000000u);
#pragma unroll
                for (int t = 0; t < MV_MAXT; ++t) {
                    if (t >= T) break;
                    const float* xp = a.x + (size_t) (dense ? t : pair / a.xdiv) * a.xs + (size_t) j * 8;
                    float xr[8], xo[4];
#pragma unroll
                    for (int c = 0; c < 8; ++c) xr[c] = __ldg(xp + c) * NSL_XSCALE;
                    block_offsets(xr, xo);
                    const float d = P == 4 ? states_dot(v, q, xr, xo) : states_dot3(v, q, xr, xo);
                    if (half) su[t] = fmaf(d, e2, su[t]);
                    else s[t] = fmaf(d, e2, s[t]);
                }
            }
        }
        const float sca = slice_scale(wa.eb + (4 - P)), scb = slice_scale(wb.eb + (4 - P));   // P = 3 products are half as large
#pragma unroll
        for (int t = 0; t < MV_MAXT; ++t) {
            if (t >= T) break;
            const float st = group_sum(s[t], 32) * sca;
            float sut = 0.0f;
            if (MODE == MODE_GU) sut = group_sum(su[t], 32) * scb;
            if (lane == 0) store_out<MODE>(a, dense ? t : pair, r, st, sut);
        }
    }
}

// ---- bit-exact decode: one thread per block ---------------------------------------------------------------------------
template <bool BF16, int P>
__global__ void __launch_bounds__(256) decode_kernel(WSlice w, KConst kc, int K, int R, void* out, const uint32_t* G) {
    __shared__ StreamTab tab;
    load_stream_tab(tab, G, threadIdx.x, 256);
    __syncthreads();
    const size_t nblk = (size_t) R * (K / 8);
    for (size_t gidx = (size_t) blockIdx.x * 256 + threadIdx.x; gidx < nblk; gidx += (size_t) gridDim.x * 256) {
        const uint32_t seed = ((const uint16_t*) w.p[0])[gidx], cw = ((const uint16_t*) w.p[1])[gidx];
        const int code = P == 4 ? (((const uint8_t*) w.p[3])[gidx >> 1] >> ((gidx & 1) * 4)) & 15 : (int) (cw & 15u);
        const uint32_t g = stream_bits(tab, seed);
        float wv[8];
        if (P == 4) block_weights(seed | (g << 16), g, cw, exact_scale45(w.eb + code), kc, wv);
        else block_weights3(seed | (g << 16), g, cw, exact_scale45(w.eb + code + 1), kc, wv);
        if (BF16) {
            uint4 o;
            o.x = bf16_bits(wv[0]) | ((uint32_t) bf16_bits(wv[1]) << 16);
            o.y = bf16_bits(wv[2]) | ((uint32_t) bf16_bits(wv[3]) << 16);
            o.z = bf16_bits(wv[4]) | ((uint32_t) bf16_bits(wv[5]) << 16);
            o.w = bf16_bits(wv[6]) | ((uint32_t) bf16_bits(wv[7]) << 16);
            ((uint4*) out)[gidx] = o;
        } else {
            ((float4*) out)[2 * gidx] = make_float4(wv[0], wv[1], wv[2], wv[3]);
            ((float4*) out)[2 * gidx + 1] = make_float4(wv[4], wv[5], wv[6], wv[7]);
        }
    }
}

// ---- work units: pairs grouped two by two per slice -------------------------------------------------------------------
// One block.  Pairs are counted per slice, a scan gives each slice its range of pairs and of units, pairs are placed
// (in any order inside a slice: a pair's result does not depend on its partner) and every slice writes its units.
constexpr int UNITS_MAX_PAIRS = 4096, UNITS_MAX_SLICES = 1024;
__global__ void __launch_bounds__(1024) mv_units_kernel(const int32_t* __restrict__ sel, int max_pairs, const int32_t* __restrict__ count,
                                                        int n_slices, int32_t* __restrict__ units, int32_t* __restrict__ n_units) {
    __shared__ int cnt[UNITS_MAX_SLICES], poff[UNITS_MAX_SLICES], uoff[UNITS_MAX_SLICES], woff[UNITS_MAX_SLICES];
    __shared__ int sorted[UNITS_MAX_PAIRS];
    grid_dependents_go();
    grid_dependency_wait();
    const int tid = threadIdx.x;
    const int P = count ? min(*count, max_pairs) : max_pairs;
    cnt[tid] = 0;
    __syncthreads();
    for (int i = tid; i < P; i += 1024) atomicAdd(&cnt[sel[i]], 1);
    __syncthreads();
    const int n = tid < n_slices ? cnt[tid] : 0;
    poff[tid] = n;
    uoff[tid] = (n + 1) / 2;
    woff[tid] = (n / 2) * UNIT_W2 + (n & 1) * UNIT_W1;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {      // inclusive scans
        const int a = tid >= o ? poff[tid - o] : 0, b = tid >= o ? uoff[tid - o] : 0, c = tid >= o ? woff[tid - o] : 0;
        __syncthreads();
        poff[tid] += a; uoff[tid] += b; woff[tid] += c;
        __syncthreads();
    }
    const int p0 = poff[tid] - n, u0 = uoff[tid] - (n + 1) / 2, w0 = woff[tid] - ((n / 2) * UNIT_W2 + (n & 1) * UNIT_W1);
    if (tid == 1023) *n_units = uoff[1023];
    __syncthreads();
    poff[tid] = p0;           // exclusive offsets; cnt becomes the placement cursor
    cnt[tid] = 0;
    __syncthreads();
    for (int i = tid; i < P; i += 1024) {
        const int e = sel[i];
        sorted[poff[e] + atomicAdd(&cnt[e], 1)] = i;
    }
    __syncthreads();
    for (int j = 0; 2 * j < n; ++j) {
        const bool two = 2 * j + 1 < n;
        int32_t* u = units + 4 * (u0 + j);
        u[0] = sorted[p0 + 2 * j];
        u[1] = two ? sorted[p0 + 2 * j + 1] : -1;
        u[2] = w0 + j * UNIT_W2;     // units before it in this slice are all two-pair units
        u[3] = 0;
    }
}

static int g_mv_variant = 1;   // 1 (default): inputs in shared memory, 16 warps / SM; 0: inputs in registers, 8 warps / SM

// ---- launch selection ---------------------------------------------------------------------------------------------------
static int log2_floor(int v) { int l = 0; while ((2 << l) <= v) ++l; return l; }

template <int MODE, int NT>
static void launch_smemx(cudaStream_t s, const MvParams& a, int lpr_log2, int dense, int grid, size_t smem) {
    static bool attr_set[16];   // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 15]) {
        cudaFuncSetAttribute(mv_smemx_kernel<MODE, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin() - 4096);
        attr_set[dev & 15] = true;
    }
    launch(mv_smemx_kernel<MODE, NT>, grid, MV_THREADS, smem, s, a, kconst(), lpr_log2, dense);
}

template <int MODE>
static void launch_mv(cudaStream_t s, const MvParams& a, int T, int p_hint = 0) {
    if (a.R <= 0 || a.P <= 0 || T <= 0) return;
    if (a.K <= 0 || a.K % 8) { set_error("seed mat-vec: K = %d is not a multiple of 8", a.K); return; }
    if (T > MV_MAXT) { set_error("seed mat-vec: %d tokens, at most %d", T, MV_MAXT); return; }
    const int dense = a.sel == NULL, sms = sm_count();
    const int ch = a.K / 64;
    // The chunked kernels need whole chunks and 16-byte aligned rows of inputs; streams come 16-byte aligned from
    // every allocator the callers use, and a row's chunks are contiguous, so only the inputs are checked here.
    const bool chunked = a.K % 64 == 0 && aligned16(a.x) && a.xs % 4 == 0;
    const bool pow2 = ch > 0 && (ch & (ch - 1)) == 0;
    if ((a.xrow || a.count || a.xbf16 || a.units) && !(chunked && pow2 && ch <= 32 && T == 1)) {
        set_error("seed mat-vec: the row-index / device-count / bf16-input forms need K = 64 * 2^j <= 2048 (K = %d)", a.K);
        return;
    }
    if (chunked && T == 1 && pow2 && ch <= 32) {
        if (a.units) launch(mv_shx2_kernel<MODE>, sms * 2, MV_THREADS, 0, s, a, kconst(), log2_floor(ch));
        else if (g_mv_variant == 1) launch(mv_shx_kernel<MODE>, sms * 2, MV_THREADS, 0, s, a, kconst(), log2_floor(ch));
        else launch(mv_regx_kernel<MODE>, sms, MV_THREADS, 0, s, a, kconst(), log2_floor(ch));
        count_launch();
        return;
    }
    const size_t smem = (size_t) (dense ? T : 1) * a.K * 6;   // inputs [K] and centring constants [K/2] per token
    if (chunked && smem <= (size_t) max_smem_optin() - 4096) {
        const int lpr_log2 = log2_floor(ch < 32 ? ch : 32);
        if constexpr (MODE == MODE_GU) launch_smemx<MODE, 1>(s, a, lpr_log2, dense, sms, smem);
        else switch (dense ? T : 1) {
#define NSL_CASE(N) case N: launch_smemx<MODE, N>(s, a, lpr_log2, dense, sms, smem); break;
            NSL_CASE(1) NSL_CASE(2) NSL_CASE(3) NSL_CASE(4) NSL_CASE(5) NSL_CASE(6) NSL_CASE(7) NSL_CASE(8)
#undef NSL_CASE
        }
        count_launch();
        return;
    }
    launch(mv_generic_kernel<MODE, 4>, sms * 2, MV_THREADS, 0, s, a, kconst(), dense ? T : 1);
    count_launch();
}

// P = 3 (SEED4): the any-shape kernel serves every form.
template <int MODE>
static void launch_mv3(cudaStream_t s, const MvParams& a, int T) {
    if (a.R <= 0 || a.P <= 0 || T <= 0) return;
    if (a.K <= 0 || a.K % 8) { set_error("seed mat-vec: K = %d is not a multiple of 8", a.K); return; }
    if (T > MV_MAXT) { set_error("seed mat-vec: %d tokens, at most %d", T, MV_MAXT); return; }
    launch(mv_generic_kernel<MODE, 3>, sm_count() * 2, MV_THREADS, 0, s, a, kconst(), a.sel ? 1 : T);
    count_launch();
}

bool launch_q4_mv(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add);

static bool seed_fmt(int fmt, const char* who) {      // the mat-vec entry points: P = 4 and P = 3 seeds
    if (fmt == MF_SEED4P4 || fmt == MF_SEED4) return true;
    set_error("%s: weight format %d is not served by this library (SEED4P4 = %d, SEED4 = %d)", who, fmt, (int) MF_SEED4P4, (int) MF_SEED4);
    return false;
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void kc_mv(cudaStream_t s, int fmt, WSlice w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add,
           const uint32_t* G) {
    if (fmt == MF_Q4) { launch_q4_mv(s, w, K, R, x, xs, y, ys, T, add); return; }   // the LM head's affine int4 (q4_head.cu)
    if (!seed_fmt(fmt, "kc_mv")) return;
    MvParams a = {NULL, NULL, w, NULL, x, y, G, K, R, T, 1, xs, ys, add, 0, NULL, NULL, 0, NULL, NULL};
    if (fmt == MF_SEED4) launch_mv3<MODE_ROUND>(s, a, T);
    else launch_mv<MODE_ROUND>(s, a, T);
}

void kc_mv_sel(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
               const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    if (!seed_fmt(fmt, "kc_mv_sel")) return;
    MvParams a = {ws, NULL, WSlice{}, sel, x, y, G, K, R, P, xdiv, xs, ys, 0, 0, NULL, NULL, 0, NULL, NULL};
    if (fmt == MF_SEED4) launch_mv3<MODE_ROUND>(s, a, 1);
    else launch_mv<MODE_ROUND>(s, a, 1);
}

void kc_mv_gu(cudaStream_t s, int fmt, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* out,
              int ys, const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    if (!seed_fmt(fmt, "kc_mv_gu")) return;
    MvParams a = {wg, wu, WSlice{}, sel, x, out, G, K, R, P, xdiv, xs, ys, 0, 0, NULL, NULL, 0, NULL, NULL};
    if (fmt == MF_SEED4) launch_mv3<MODE_GU>(s, a, 1);
    else launch_mv<MODE_GU>(s, a, 1);
}

void nsl_mv_raw(cudaStream_t s, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    MvParams a = {sel ? ws : NULL, NULL, WSlice{}, sel, x, y, G, K, R, P, xdiv > 0 ? xdiv : 1, xs, ys, 0, 1, NULL, NULL, 0, NULL, NULL};
    if (!sel) a.w0 = *ws;   // dense: ws is a host pointer to the one slice
    launch_mv<MODE_ROUND>(s, a, sel ? 1 : P);
}

void nsl_mv_gu_raw(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* out,
                   int ys, const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    MvParams a = {wg, wu, WSlice{}, sel, x, out, G, K, R, P, xdiv, xs, ys, 0, 1, NULL, NULL, 0, NULL, NULL};
    launch_mv<MODE_GU>(s, a, 1);
}

// Expert-parallel forms: a compacted pair list whose length lives on the device.  Pair p uses slice sel[p] and input
// row xrow[p] of x, which holds packed bf16 rows when x_bf16 is set; at most max_pairs pairs, *count of them valid.
void nsl_mv_gu_rows(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const void* x, int xs, int x_bf16,
                    float* out, int ys, const int32_t* sel, const int32_t* xrow, int max_pairs, const int32_t* count,
                    int expected_pairs, const uint32_t* G) {
    MvParams a = {wg, wu, WSlice{}, sel, (const float*) x, out, G, K, R, max_pairs, 1, xs, ys, 0, 0, xrow, count, x_bf16, NULL, NULL};
    launch_mv<MODE_GU>(s, a, 1, expected_pairs);
}
void nsl_mv_sel_rows(cudaStream_t s, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                     const int32_t* sel, int max_pairs, const int32_t* count, int expected_pairs, const uint32_t* G) {
    MvParams a = {ws, NULL, WSlice{}, sel, x, y, G, K, R, max_pairs, 1, xs, ys, 0, 0, NULL, count, 0};
    launch_mv<MODE_ROUND>(s, a, 1, expected_pairs);
}

// Work units over a pair list (see include/nslm_kernels.h): the grouping kernel and the two mat-vec forms that use it.
void nsl_mv_units(cudaStream_t s, const int32_t* sel, int max_pairs, const int32_t* count, int n_slices, int32_t* units,
                  int32_t* n_units) {
    if (max_pairs < 1 || max_pairs > UNITS_MAX_PAIRS || n_slices < 1 || n_slices > UNITS_MAX_SLICES) {
        set_error("nsl_mv_units: %d pairs (at most %d) or %d slices (at most %d)", max_pairs, UNITS_MAX_PAIRS, n_slices, UNITS_MAX_SLICES);
        return;
    }
    launch(mv_units_kernel, 1, 1024, 0, s, sel, max_pairs, count, n_slices, units, n_units);
    count_launch();
}

void nsl_mv_gu_units(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const void* x, int xs, int x_bf16, float* out,
                     int ys, const int32_t* sel, const int32_t* xrow, int xdiv, const int32_t* units, const int32_t* n_units,
                     int max_pairs, int raw, const uint32_t* G) {
    MvParams a = {wg, wu, WSlice{}, sel, (const float*) x, out, G, K, R, max_pairs, xdiv > 0 ? xdiv : 1, xs, ys, 0, raw, xrow, NULL, x_bf16,
                  units, n_units};
    launch_mv<MODE_GU>(s, a, 1);
}

void nsl_mv_sel_units(cudaStream_t s, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys, const int32_t* sel,
                      const int32_t* units, const int32_t* n_units, int max_pairs, int raw, const uint32_t* G) {
    MvParams a = {ws, NULL, WSlice{}, sel, x, y, G, K, R, max_pairs, 1, xs, ys, 0, raw, NULL, NULL, 0, units, n_units};
    launch_mv<MODE_ROUND>(s, a, 1);
}

void nsl_mv_set_variant(int v) { g_mv_variant = v; }

void nsl_decode_f32(cudaStream_t s, WSlice w, int K, int R, float* out, const uint32_t* G) {
    if (K <= 0 || K % 8 || R <= 0) { if (K % 8) set_error("nsl_decode_f32: K = %d is not a multiple of 8", K); return; }
    const size_t nblk = (size_t) R * (K / 8);
    const int grid = (int) ((nblk + 255) / 256 < (size_t) sm_count() * 8 ? (nblk + 255) / 256 : (size_t) sm_count() * 8);
    decode_kernel<false, 4><<<grid, 256, 0, s>>>(w, kconst(), K, R, out, G);
    count_launch();
}

void nsl_decode_bf16(cudaStream_t s, WSlice w, int K, int R, uint16_t* out, const uint32_t* G) {
    if (K <= 0 || K % 8 || R <= 0) { if (K % 8) set_error("nsl_decode_bf16: K = %d is not a multiple of 8", K); return; }
    const size_t nblk = (size_t) R * (K / 8);
    const int grid = (int) ((nblk + 255) / 256 < (size_t) sm_count() * 8 ? (nblk + 255) / 256 : (size_t) sm_count() * 8);
    decode_kernel<true, 4><<<grid, 256, 0, s>>>(w, kconst(), K, R, out, G);
    count_launch();
}

// P = 3 (SEED4) slices decoded bit for bit: w.p[0] seeds, w.p[1] nibble words, w.eb the exponent bias.
void nsl_decode3_f32(cudaStream_t s, WSlice w, int K, int R, float* out, const uint32_t* G) {
    if (K <= 0 || K % 8 || R <= 0) { if (K % 8) set_error("nsl_decode3_f32: K = %d is not a multiple of 8", K); return; }
    const size_t nblk = (size_t) R * (K / 8);
    const int grid = (int) ((nblk + 255) / 256 < (size_t) sm_count() * 8 ? (nblk + 255) / 256 : (size_t) sm_count() * 8);
    decode_kernel<false, 3><<<grid, 256, 0, s>>>(w, kconst(), K, R, out, G);
    count_launch();
}

void nsl_decode3_bf16(cudaStream_t s, WSlice w, int K, int R, uint16_t* out, const uint32_t* G) {
    if (K <= 0 || K % 8 || R <= 0) { if (K % 8) set_error("nsl_decode3_bf16: K = %d is not a multiple of 8", K); return; }
    const size_t nblk = (size_t) R * (K / 8);
    const int grid = (int) ((nblk + 255) / 256 < (size_t) sm_count() * 8 ? (nblk + 255) / 256 : (size_t) sm_count() * 8);
    decode_kernel<true, 3><<<grid, 256, 0, s>>>(w, kconst(), K, R, out, G);
    count_launch();
}

}   // extern "C"
