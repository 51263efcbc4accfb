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
#include "route.cuh"
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
};

__device__ __forceinline__ float silu_bf(float g) {   // each op rounded to bf16 (engine/kernels_moe.cu:28-31)
    const float s = bf16_round(1.0f / (1.0f + expf(-g)));
    return bf16_round(g * s);
}

struct Chunk { uint4 s, c; uint32_t cd; };

// The conversion constants (seed_block.cuh: KConst) as a module constant for code outside the kernels' own bodies: a
// function that is not inlined cannot take them as constant-bank kernel arguments.
constexpr float pow2_f(int e) {
    float v = 1.0f;
    for (int i = 0; i < (e < 0 ? -e : e); ++i) v = e < 0 ? v * 0.5f : v * 2.0f;
    return v;
}
constexpr KConst kconst_static() {
    KConst k = {};
    for (int p = 0; p < 4; ++p) {
        k.cxor[p] = ((uint32_t) (215 - 5 * p) << 23) | (8u << (4 * p));
        k.coff[p] = -(pow2_f(88 - 5 * p) + pow2_f(68 - p));
        k.cxor_x[p] = ((uint32_t) (250 - 5 * p) << 23) | (8u << (4 * p));
        k.coff_x[p] = -(pow2_f(123 - 5 * p) + pow2_f(103 - p));
    }
    k.cor = 112u << 23;
    return k;
}
__constant__ KConst c_kc = kconst_static();

// What a unit's row loop needs, by value (it runs in a function of its own: see unit_rows).
struct UnitArgs {
    const uint4 *sa, *ca, *sb, *cb;      // seeds and coefficient words of the (gate or only) matrix and of the up matrix
    const uint32_t *da, *db;              // their exponent codes
    int eba, ebb;
    float* y;
    int ys, R, raw, add;
    int pid[4];                           // the unit's pairs (output rows)
    int s_lo, s_hi, lpr_log2;
};
__device__ __forceinline__ Chunk load_chunk3(const uint4* s, const uint4* c, const uint32_t* d, size_t chunk_index) {
    Chunk k;
    k.s = __ldg(s + chunk_index);
    k.c = __ldg(c + chunk_index);
    k.cd = __ldg(d + chunk_index);
    return k;
}

template <int PF = 4>      // PF = 3: the SEED4 format has no code stream (a block's code rides in its nibble word)
__device__ __forceinline__ Chunk load_chunk(const WSlice& w, size_t chunk_index) {
    Chunk k;
    k.s = __ldg((const uint4*) w.p[0] + chunk_index);
    k.c = __ldg((const uint4*) w.p[1] + chunk_index);
    k.cd = PF == 4 ? __ldg((const uint32_t*) w.p[3] + chunk_index) : 0u;
    return k;
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

// One thread's share of staging a pair's inputs: 16 inputs (two blocks: chunk j of the row, block pair bp), scaled, as
// the f32x2 operands of pair_dot plus the two blocks' input sums (2^-64 of them), from which the consumer forms the
// centring constants: xm[p] = -2^(p-66) * sum, an exact scaling, so the bits are those of block_offsets.
__device__ __forceinline__ float block_sum(const float* xs) {      // the order of block_offsets
    return (((xs[0] + xs[4]) + (xs[1] + xs[5])) + ((xs[2] + xs[6]) + (xs[3] + xs[7]))) * 5.421010862427522e-20f;   // 2^-64
}
__device__ __forceinline__ void offsets_from_sum(u64 s2, u64* xm2) {
    xm2[0] = mul2(s2, pack2(-1.3552527156068805e-20f, -1.3552527156068805e-20f));   // -2^-66
    xm2[1] = mul2(s2, pack2(-2.710505431213761e-20f, -2.710505431213761e-20f));     // -2^-65
    xm2[2] = mul2(s2, pack2(-5.421010862427522e-20f, -5.421010862427522e-20f));     // -2^-64
    xm2[3] = mul2(s2, pack2(-1.0842021724855044e-19f, -1.0842021724855044e-19f));   // -2^-63
}
__device__ __forceinline__ void stage_load(const MvParams& a, int xr, int j, int bp, float* x) {
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
}
__device__ __forceinline__ void stage_store(const float* x, int j, int bp, ulonglong2* sx, u64* ss) {
#pragma unroll
    for (int cq = 0; cq < 4; ++cq) {
        ulonglong2 t;
        t.x = pack2(x[2 * cq], x[8 + 2 * cq]);
        t.y = pack2(x[2 * cq + 1], x[8 + 2 * cq + 1]);
        sx[(bp * 4 + cq) * 32 + j] = t;
    }
    ss[bp * 32 + j] = pack2(block_sum(x), block_sum(x + 8));
}


struct RouteFuse {        // the router folded into the prologue (logits == NULL: the pair list comes from MvParams.sel)
    const float* logits;
    int ld, n_exp, top_k, T;
    int32_t* ind_out;
    float* wt_out;
};

// One thread's share of staging a pair's inputs: 16 inputs (two blocks: chunk j of the row, block pair bp), scaled, as
// the f32x2 operands of pair_dot plus their centring constants.
__device__ __forceinline__ void stage_pair_inputs(const MvParams& a, int xr, int j, int bp, ulonglong2* sx, ulonglong2* sm) {
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

// ---- one expansion per pair, inputs in shared memory, two blocks of 8 warps per SM ----------------------------------------
// Rows of 1, 2, 4, .. 32 chunks (K = 64 .. 2048).  The pair's inputs sit in shared memory as the f32x2 operands of pair_dot,
// laid out [block pair][operand pair][lane] so that a warp's 16-byte loads are conflict-free; a thread fits in 128
// registers and 16 warps per SM hide the logic pipe's latencies.  The work is the pair-major sequence of row steps (a
// step = the 32 / lanes-per-row rows a warp expands at once); blocks take contiguous equal shares of it, inside a pair the
// block's warps take its steps round-robin, and the next row's streams are prefetched while the current row is expanded.
// Optionally the block first ROUTES: with logits given, warp t picks token t's top-k experts (route.cuh) and the pair
// list is the T * top_k (token, expert) pairs; block 0 also stores ids and weights for the kernels that follow.
// PF: coefficients per block.  4: SEED4P4; 3: SEED4 (24 states, the nibble word; the products are half as large, which the
// slice scale makes up).
template <int MODE, int PF>
__global__ void __launch_bounds__(MV_THREADS, 2) mv_pair_kernel(MvParams a, KConst kc, int lpr_log2, RouteFuse rf) {
    __shared__ StreamTab tab;
    __shared__ int32_t r_ind[256];   // the fused router's picks
    __shared__ float r_wt[256];
    __shared__ __align__(16) ulonglong2 sx[4 * 4 * 32];   // [bp][c / 2][lane] = {x2[c], x2[c + 1]}
    __shared__ __align__(16) ulonglong2 sm[4 * 2 * 32];   // [bp][p / 2][lane] = {xm2[p], xm2[p + 1]}
    load_stream_tab(tab, a.G, threadIdx.x, MV_THREADS);
    grid_dependents_go();
    grid_dependency_wait();   // everything below may read what the previous kernel in the stream wrote
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    int P = a.count ? min(*a.count, a.P) : a.P;
    if (rf.logits) {          // the router: one warp per token, every block the same picks; block 0 stores them
        if (warp < rf.T) {
            const float* l = rf.logits + (size_t) warp * rf.ld;
            if (rf.n_exp <= 128) route_row<4>(rf.n_exp, rf.top_k, l, lane, r_ind + warp * rf.top_k, r_wt + warp * rf.top_k);
            else if (rf.n_exp <= 512) route_row<16>(rf.n_exp, rf.top_k, l, lane, r_ind + warp * rf.top_k, r_wt + warp * rf.top_k);
            else route_row<32>(rf.n_exp, rf.top_k, l, lane, r_ind + warp * rf.top_k, r_wt + warp * rf.top_k);
        }
        P = rf.T * rf.top_k;
        __syncthreads();
        if (blockIdx.x == 0 && (int) threadIdx.x < P) {
            rf.ind_out[threadIdx.x] = r_ind[threadIdx.x];
            rf.wt_out[threadIdx.x] = r_wt[threadIdx.x];
        }
    }
    const int rs = (a.R + rpw - 1) / rpw;
    const long long total = (long long) P * rs;
    const long long begin = (long long) blockIdx.x * total / gridDim.x, end = (long long) (blockIdx.x + 1) * total / gridDim.x;
    if (begin >= end) return;
    const int p_first = (int) (begin / rs), p_last = (int) ((end - 1) / rs);
    for (int pair = p_first; pair <= p_last; ++pair) {
        const int s_lo = pair == p_first ? (int) (begin - (long long) pair * rs) : 0;
        const int s_hi = pair == p_last ? (int) (end - (long long) pair * rs) : rs;
        const int slice = rf.logits ? r_ind[pair] : (a.sel ? a.sel[pair] : 0);
        const WSlice wa = a.ws ? a.ws[slice] : a.w0;
        WSlice wb = wa;
        if (MODE == MODE_GU) wb = a.wu[slice];
        // this warp's first streams are requested before the inputs are staged: their DRAM latency runs under it
        int st = s_lo + warp;
        int r = st * rpw + ro;
        Chunk ka, kb;
        if (st < s_hi && r < a.R) {
            ka = load_chunk<PF>(wa, (size_t) r * lpr + jc);
            if (MODE == MODE_GU) kb = load_chunk<PF>(wb, (size_t) r * lpr + jc);
        }
        if (pair != p_first) __syncthreads();   // the previous pair's inputs are no longer read
        if (threadIdx.x < lpr * 4) {
            const int j = threadIdx.x & (lpr - 1), bp = threadIdx.x >> lpr_log2;
            stage_pair_inputs(a, a.xrow ? a.xrow[pair] : pair / a.xdiv, j, bp, sx, sm);
        }
        __syncthreads();   // inputs staged (and, for the block's first pair, the stream table loaded)
        const float sca = slice_scale(wa.eb + (4 - PF)), scb = slice_scale(wb.eb + (4 - PF));
        for (; st < s_hi; st += MV_WARPS, r += MV_WARPS * rpw) {
            const bool ok = r < a.R;
            const int rn = r + MV_WARPS * rpw;
            Chunk na, nb;
            if (st + MV_WARPS < s_hi && rn < a.R) {
                na = load_chunk<PF>(wa, (size_t) rn * lpr + jc);
                if (MODE == MODE_GU) nb = load_chunk<PF>(wb, (size_t) rn * lpr + jc);
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
                    if (PF == 4) {
                        u64 q[4];
                        pair_coefs(cwa[bp], kc, q);
                        acc = fma2(pair_expand_dot(tab, swa[bp], q, x2, xm2), code_scale_pair(ka.cd, bp, kc), acc);
                    } else {
                        u64 q[3];
                        pair_coefs3(cwa[bp], kc, q);
                        acc = fma2(pair_expand_dot3(tab, swa[bp], q, x2, xm2), code_scale_pair3(cwa[bp], kc), acc);
                    }
                    if (MODE == MODE_GU && PF == 4) {
                        u64 q[4];
                        pair_coefs(cwb[bp], kc, q);
                        accu = fma2(pair_expand_dot(tab, swb[bp], q, x2, xm2), code_scale_pair(kb.cd, bp, kc), accu);
                    } else if (MODE == MODE_GU) {
                        u64 q[3];
                        pair_coefs3(cwb[bp], kc, q);
                        accu = fma2(pair_expand_dot3(tab, swb[bp], q, x2, xm2), code_scale_pair3(cwb[bp], kc), accu);
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


// ---- the whole decode step of an expert layer in one launch -----------------------------------------------------------------
// Router, gate + up + SwiGLU, down projection and weighted combine as three phases of one grid of two blocks an SM, instead
// of three dependent launches: a launch boundary costs the step its predecessor's tail (the last blocks' row steps with
// the other SMs idle), the successor's ramp and the prologue (stream table, router) again, ~4 us each on a step of
// 26 .. 114 us.  Here a block that has finished its share of a phase starts on the next one at once; what it needs from
// other blocks it waits for on counters in device memory:
//   ready[p]  row steps of pair p's gate + up rows stored           (the down projection of pair p reads all of them)
//   done[t]   row steps of token t's down projections stored        (the combine of token t reads all top_k of them)
// Each phase is the pair kernel's: the pair-major sequence of row steps cut into contiguous equal shares, so block b
// works on the same pairs in phases 1 and 2 and waits for its neighbours b - 1 and b + 1 at most; blocks are dispatched
// in index order and no block waits for a higher-numbered block other than b + 1 before it has finished phase 2, so the
// grid makes progress even when not all of it is resident.  Every wait is bounded: when one runs out the block records
// status 1, every other wait ends on seeing it, and the launch returns with its counters cleared (the last block to
// finish clears them for the next launch; fin counts finished blocks and wraps to zero by itself).
// Arithmetic and rounding points are those of the three kernels it replaces, operation for operation.
// Measured (config 1, CUDA graph replay, us per step at 8 / 4 / 1 rows): 126.3 / 70.1 / 26.7 against 114.2 / 65.5 / 26.2
// for the three dependent launches, so the host layer does not use it by default.  Under ncu the one launch lasts what
// the three last back to back (130.5 against 129.2 us; the same 75.0 M instructions and 217 k active cycles an SM); what
// the dependent launches hide between steps -- the next kernel's blocks resident with table, router and first streams
// ready when the wait ends -- this form cannot, and its barrier stalls are 0.78 per issued instruction against 0.10:
// at each phase change a block waits for the slowest of the ~6 blocks that share its pairs.
struct StepSync {
    unsigned* ready;      // [T * top_k]
    unsigned* done;       // [T]
    unsigned* fin;
    int* status;
};
struct StepParams {
    const WSlice *wg, *wu, *wd;
    const float* x;       // [T][d]
    const float* logits;  // [T][ld]
    float* A;             // [T * top_k][ff]
    float* D;             // [T * top_k][d]
    float* out;           // [T][d]
    int32_t* ind_out;
    float* wt_out;
    const uint32_t* G;
    int xs, ld, n_exp, top_k, T, d, ff, raw;
    StepSync sy;
};
constexpr unsigned STEP_WAIT_LIMIT = 1u << 19;      // polls of ~0.1 us

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// false: the limit ran out, or another block has reported that its wait did
__device__ __forceinline__ bool step_wait(const unsigned* counter, unsigned target, int* status) {
    for (unsigned i = 0; i < STEP_WAIT_LIMIT; ++i) {
        if (ld_acquire(counter) >= target) return true;
        if ((i & 63u) == 63u && *(volatile int*) status) return false;
        __nanosleep(i < 16 ? 32 : 128);
    }
    atomicCAS(status, 0, 1);
    return false;
}

// A pair's inputs from memory that other blocks of this grid have written: the loads bypass the non-coherent path.
__device__ __forceinline__ void stage_pair_inputs_cg(const float* xrow, int j, int bp, ulonglong2* sx, ulonglong2* sm) {
    float x[16], xm[8];
    const float4* xp = (const float4*) (xrow + (size_t) j * 64 + bp * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 t = __ldcg(xp + i);
        x[4 * i] = t.x * NSL_XSCALE; x[4 * i + 1] = t.y * NSL_XSCALE; x[4 * i + 2] = t.z * NSL_XSCALE; x[4 * i + 3] = t.w * NSL_XSCALE;
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

struct StepShared {
    StreamTab tab;
    int32_t r_ind[256];
    float r_wt[256];
    __align__(16) ulonglong2 sx[4 * 4 * 32];
    __align__(16) ulonglong2 sm[4 * 2 * 32];
    int abort;
};

// One phase: MODE_GU (x -> A, signals ready[pair]) or MODE_ROUND (A -> D, waits for ready[pair], signals done[token]).
template <int MODE>
__device__ __forceinline__ void step_phase(const StepParams& p, const KConst& kc, StepShared& sh, int P, int lpr_log2, unsigned rs_gu) {
    const int K = MODE == MODE_GU ? p.d : p.ff, R = MODE == MODE_GU ? p.ff : p.d;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    const int rs = (R + rpw - 1) / rpw;
    const long long total = (long long) P * rs;
    const long long begin = (long long) blockIdx.x * total / gridDim.x, end = (long long) (blockIdx.x + 1) * total / gridDim.x;
    if (begin >= end) return;
    const int p_first = (int) (begin / rs), p_last = (int) ((end - 1) / rs);
    MvParams a = {};
    a.y = MODE == MODE_GU ? p.A : p.D;
    a.ys = R;
    a.R = R;
    a.raw = p.raw;
    for (int pair = p_first; pair <= p_last; ++pair) {
        const int s_lo = pair == p_first ? (int) (begin - (long long) pair * rs) : 0;
        const int s_hi = pair == p_last ? (int) (end - (long long) pair * rs) : rs;
        const int slice = sh.r_ind[pair];
        const WSlice wa = MODE == MODE_GU ? p.wg[slice] : p.wd[slice];
        WSlice wb = wa;
        if (MODE == MODE_GU) wb = p.wu[slice];
        int st = s_lo + warp;
        int r = st * rpw + ro;
        Chunk ka, kb;
        if (st < s_hi && r < R) {      // the streams do not depend on other blocks: requested before any wait
            ka = load_chunk<4>(wa, (size_t) r * lpr + jc);
            if (MODE == MODE_GU) kb = load_chunk<4>(wb, (size_t) r * lpr + jc);
        }
        if (MODE == MODE_ROUND && threadIdx.x == 0 && !step_wait(p.sy.ready + pair, rs_gu, p.sy.status)) sh.abort = 1;
        __syncthreads();   // the previous pair's inputs are no longer read; the wait's outcome is known
        if (sh.abort) return;
        if (threadIdx.x < lpr * 4) {
            const int j = threadIdx.x & (lpr - 1), bp = threadIdx.x >> lpr_log2;
            if (MODE == MODE_GU) {
                MvParams ax = {};
                ax.x = p.x;
                ax.xs = p.xs;
                stage_pair_inputs(ax, pair / p.top_k, j, bp, sh.sx, sh.sm);
            } else stage_pair_inputs_cg(p.A + (size_t) pair * p.ff, j, bp, sh.sx, sh.sm);
        }
        __syncthreads();
        const float sca = slice_scale(wa.eb), scb = slice_scale(wb.eb);
        for (; st < s_hi; st += MV_WARPS, r += MV_WARPS * rpw) {
            const bool ok = r < R;
            const int rn = r + MV_WARPS * rpw;
            Chunk na, nb;
            if (st + MV_WARPS < s_hi && rn < R) {
                na = load_chunk<4>(wa, (size_t) rn * lpr + jc);
                if (MODE == MODE_GU) nb = load_chunk<4>(wb, (size_t) rn * lpr + jc);
            }
            u64 acc = 0ull, accu = 0ull;
            if (ok) {
                const uint32_t swa[4] = {ka.s.x, ka.s.y, ka.s.z, ka.s.w}, cwa[4] = {ka.c.x, ka.c.y, ka.c.z, ka.c.w};
                const uint32_t swb[4] = {kb.s.x, kb.s.y, kb.s.z, kb.s.w}, cwb[4] = {kb.c.x, kb.c.y, kb.c.z, kb.c.w};
#pragma unroll
                for (int bp = 0; bp < 4; ++bp) {
                    u64 x2[8], xm2[4];
#pragma unroll
                    for (int cq = 0; cq < 4; ++cq) { const ulonglong2 t = sh.sx[(bp * 4 + cq) * 32 + jc]; x2[2 * cq] = t.x; x2[2 * cq + 1] = t.y; }
#pragma unroll
                    for (int pq = 0; pq < 2; ++pq) { const ulonglong2 t = sh.sm[(bp * 2 + pq) * 32 + jc]; xm2[2 * pq] = t.x; xm2[2 * pq + 1] = t.y; }
                    {
                        u64 q[4];
                        pair_coefs(cwa[bp], kc, q);
                        acc = fma2(pair_expand_dot(sh.tab, swa[bp], q, x2, xm2), code_scale_pair(ka.cd, bp, kc), acc);
                    }
                    if (MODE == MODE_GU) {
                        u64 q[4];
                        pair_coefs(cwb[bp], kc, q);
                        accu = fma2(pair_expand_dot(sh.tab, swb[bp], q, x2, xm2), code_scale_pair(kb.cd, bp, kc), accu);
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
        // this block's row steps of the pair are stored: publish their number
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) atomicAdd(MODE == MODE_GU ? p.sy.ready + pair : p.sy.done + pair / p.top_k, (unsigned) (s_hi - s_lo));
    }
}

__global__ void __launch_bounds__(MV_THREADS, 2) mv_step_kernel(StepParams p, KConst kc, int lg_d, int lg_ff) {
    __shared__ StepShared sh;
    load_stream_tab(sh.tab, p.G, threadIdx.x, MV_THREADS);
    if (threadIdx.x == 0) sh.abort = 0;
    grid_dependents_go();
    grid_dependency_wait();   // everything below may read what the previous kernel in the stream wrote
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int P = p.T * p.top_k;
    if (warp < p.T) {         // the router: one warp per token, every block the same picks; block 0 stores them
        const float* l = p.logits + (size_t) warp * p.ld;
        if (p.n_exp <= 128) route_row<4>(p.n_exp, p.top_k, l, lane, sh.r_ind + warp * p.top_k, sh.r_wt + warp * p.top_k);
        else if (p.n_exp <= 512) route_row<16>(p.n_exp, p.top_k, l, lane, sh.r_ind + warp * p.top_k, sh.r_wt + warp * p.top_k);
        else route_row<32>(p.n_exp, p.top_k, l, lane, sh.r_ind + warp * p.top_k, sh.r_wt + warp * p.top_k);
    }
    __syncthreads();
    if (blockIdx.x == 0 && (int) threadIdx.x < P) {
        p.ind_out[threadIdx.x] = sh.r_ind[threadIdx.x];
        p.wt_out[threadIdx.x] = sh.r_wt[threadIdx.x];
    }
    const unsigned rs_gu = (unsigned) ((p.ff + (32 >> lg_d) - 1) / (32 >> lg_d));      // row steps of a pair's gate + up rows
    step_phase<MODE_GU>(p, kc, sh, P, lg_d, rs_gu);
    if (!sh.abort) step_phase<MODE_ROUND>(p, kc, sh, P, lg_ff, rs_gu);
    // combine: out[t][i] = sum_j wt[t][j] D[t * k + j][i], plain f32, j ascending (q4_combine_kernel's sum); item = (token, 256 columns)
    if (!sh.abort) {
        const int cpr = (p.d + MV_THREADS - 1) / MV_THREADS, rpw_d = 32 >> lg_ff;
        const unsigned rs_down = (unsigned) ((p.d + rpw_d - 1) / rpw_d) * (unsigned) p.top_k;
        for (int item = blockIdx.x; item < p.T * cpr; item += gridDim.x) {
            const int t = item / cpr, i = (item - t * cpr) * MV_THREADS + (int) threadIdx.x;
            if (threadIdx.x == 0 && !step_wait(p.sy.done + t, rs_down, p.sy.status)) sh.abort = 1;
            __syncthreads();
            if (sh.abort) break;
            if (i < p.d) {
                float acc = 0.0f;
                for (int j = 0; j < p.top_k; ++j) acc += sh.r_wt[t * p.top_k + j] * __ldcg(p.D + ((size_t) t * p.top_k + j) * p.d + i);
                p.out[(size_t) t * p.d + i] = acc;
            }
        }
    }
    // the last block to finish clears the counters for the next launch
    __syncthreads();
    if (threadIdx.x == 0) sh.abort = atomicInc(p.sy.fin, gridDim.x - 1) == gridDim.x - 1 ? 2 : 0;
    __syncthreads();
    if (sh.abort == 2) {
        for (int i = threadIdx.x; i < P; i += MV_THREADS) p.sy.ready[i] = 0u;
        for (int i = threadIdx.x; i < p.T; i += MV_THREADS) p.sy.done[i] = 0u;
    }
}


// ---- pairs grouped by expert: one expansion per distinct slice ---------------------------------------------------------
// Rows of 1, 2, 4, .. 32 chunks (K = 64 .. 2048).  Every block builds the same plan in its prologue: the pair list is
// sorted by slice in shared memory, runs of pairs that use the same slice are cut into UNITS of at most GRP_NT pairs, and
// a unit's rows are expanded once for all its pairs (the logic-pipe work is shared; each pair keeps its own sums, formed in
// the same order as when it is alone, so a pair's result does not depend on its partners).  The work is the sequence of
// (unit, row step) items, an item of a unit with n pairs weighing GRP_W[n]; blocks take contiguous equal shares of the
// weighted sequence, inside a unit the block's warps take its row steps round-robin, a row step being the 32 /
// lanes-per-row rows a warp expands at once.  A unit's inputs sit in shared memory as the f32x2 operands of pair_dot,
// laid out [pair][block pair][operand pair][lane] so that a warp's 16-byte loads are conflict-free.
//
// Optionally the block first ROUTES: with logits given, warp t picks token t's top-k experts (route.cuh) and the pair
// list is the T * top_k (token, expert) pairs; block 0 also stores ids and weights for the kernels that follow.
#ifndef NSL_GRP_NT
#define NSL_GRP_NT 2
#endif
constexpr int GRP_NT = NSL_GRP_NT;                         // pairs that share one expansion at most
constexpr int GRP_MAX_PAIRS = 1024;               // pairs a block can sort; longer lists run ungrouped
constexpr int GRP_SMALL = 128;                    // lists up to this length are ranked by counting (no sorting network)
#ifndef NSL_GRP_W2
#define NSL_GRP_W2 12
#define NSL_GRP_W3 18
#define NSL_GRP_W4 23
#endif
#ifndef NSL_GRP_MINB
#define NSL_GRP_MINB 2
#endif
__device__ constexpr int GRP_W[5] = {0, 8, NSL_GRP_W2, NSL_GRP_W3, NSL_GRP_W4};   // relative cost of a row step for a unit of n pairs
constexpr int GRP_SX = 4 * 4 * 32, GRP_SS = 4 * 32;               // entries of one pair's inputs (ulonglong2) / block sums (u64)

struct GrpShared {
    StreamTab tab;
    uint32_t key[GRP_MAX_PAIRS];                  // sorted (slice << 10 | pair)
    int32_t prefix[GRP_MAX_PAIRS + 1];            // weight of the units that start before sorted position i
    uint32_t tmp[GRP_SMALL];                      // short lists: unsorted keys, then unit weights
    int32_t r_ind[256];                           // the fused router's picks
    float r_wt[256];
    __align__(16) ulonglong2 sx[GRP_NT][GRP_SX];
    __align__(16) u64 ss[GRP_NT][GRP_SS];
};


// One row step of one matrix for NT pairs: four block pairs expanded once each, dotted with every pair's inputs.
// The state-value pairs of weights 4H .. 4H+3 of two adjacent blocks (half of pair_states): v[4 (c - 4H) + p].
template <int H>
__device__ __forceinline__ void half_states(uint32_t a0, uint32_t a1, uint32_t g0, uint32_t g1, u64* v) {
#define NSL_VH(C)                                                                                \
    {                                                                                            \
        const uint32_t y0 = weight_word<4 * H + C>(a0, g0), y1 = weight_word<4 * H + C>(a1, g1);  \
        v[4 * C + 0] = pack2(state_value<0>(y0), state_value<0>(y1));                            \
        v[4 * C + 1] = pack2(state_value<1>(y0), state_value<1>(y1));                            \
        v[4 * C + 2] = pack2(state_value<2>(y0), state_value<2>(y1));                            \
        v[4 * C + 3] = pack2(state_value<3>(y0), state_value<3>(y1));                            \
    }
    NSL_VH(0) NSL_VH(1) NSL_VH(2) NSL_VH(3)
#undef NSL_VH
}

// One row step of one matrix for NT pairs: each block pair is expanded once, half of its weights at a time (so that only
// 16 state-value pairs are held while every pair's inputs pass), and dotted with every pair's inputs.  Per pair the
// operations and their order are those of pair_dot.
template <int NT>
__device__ __forceinline__ void unit_chunk(const StreamTab& tab, const KConst& kc, const Chunk& k, const ulonglong2 (*sx)[GRP_SX],
                                           const u64 (*ss)[GRP_SS], int jc, u64* acc) {
    const uint32_t sw[4] = {k.s.x, k.s.y, k.s.z, k.s.w}, cw[4] = {k.c.x, k.c.y, k.c.z, k.c.w};
#pragma unroll
    for (int bp = 0; bp < 4; ++bp) {
        const uint32_t g0 = tab.lo[__byte_perm(sw[bp], 0, 0x4440)] ^ tab.hi[__byte_perm(sw[bp], 0, 0x4441)];
        const uint32_t g1 = tab.lo[__byte_perm(sw[bp], 0, 0x4442)] ^ tab.hi[__byte_perm(sw[bp], 0, 0x4443)];
        const uint32_t a0 = __byte_perm(sw[bp], g0, 0x5410), a1 = __byte_perm(sw[bp], g1, 0x5432);
        u64 d[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t) offsets_from_sum(ss[t][bp * 32 + jc], d[t]);
        {
            u64 v[16];
            half_states<0>(a0, a1, g0, g1, v);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
#pragma unroll
                for (int cq = 0; cq < 2; ++cq) {
                    const ulonglong2 u = sx[t][(bp * 4 + cq) * 32 + jc];
#pragma unroll
                    for (int p = 0; p < 4; ++p) d[t][p] = fma2(u.x, v[8 * cq + p], d[t][p]);
#pragma unroll
                    for (int p = 0; p < 4; ++p) d[t][p] = fma2(u.y, v[8 * cq + 4 + p], d[t][p]);
                }
            }
        }
        {
            u64 v[16];
            half_states<1>(a0, a1, g0, g1, v);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
#pragma unroll
                for (int cq = 0; cq < 2; ++cq) {
                    const ulonglong2 u = sx[t][(bp * 4 + 2 + cq) * 32 + jc];
#pragma unroll
                    for (int p = 0; p < 4; ++p) d[t][p] = fma2(u.x, v[8 * cq + p], d[t][p]);
#pragma unroll
                    for (int p = 0; p < 4; ++p) d[t][p] = fma2(u.y, v[8 * cq + 4 + p], d[t][p]);
                }
            }
        }
        u64 q[4];
        pair_coefs(cw[bp], kc, q);
        const u64 e2 = code_scale_pair(k.cd, bp, kc);
#pragma unroll
        for (int t = 0; t < NT; ++t)
            acc[t] = fma2(fma2(q[3], d[t][3], fma2(q[2], d[t][2], fma2(q[1], d[t][1], mul2(q[0], d[t][0])))), e2, acc[t]);
    }
}

// The row steps [s_lo, s_hi) of a unit of NT pairs that fall to this warp.  ka / kb: the streams of its first step,
// requested by the caller before the unit's inputs were staged.
template <int MODE>
__device__ __forceinline__ void store_unit(const UnitArgs& ua, int pair, int r, float s, float su) {
    float* yo = ua.y + (size_t) pair * ua.ys + r;
    if (MODE == MODE_GU) *yo = ua.raw ? (s / (1.0f + expf(-s))) * su : bf16_round(silu_bf(bf16_round(s)) * bf16_round(su));
    else if (ua.raw) *yo = s;
    else *yo = ua.add ? bf16_round(*yo + bf16_round(s)) : bf16_round(s);   // engine/kernels_moe.cu:214
}

template <int MODE, int NT>
__device__ __noinline__ void unit_rows(UnitArgs ua, Chunk ka, Chunk kb) {
    // Not inlined on purpose: each unit size gets a register allocation of its own (inlined into one body, the larger
    // sizes' pressure spilled the single-pair loop too).  Shared memory and the constants are reached by name.
    extern __shared__ __align__(16) unsigned char grp_smem[];
    const GrpShared& sh = *reinterpret_cast<const GrpShared*>(grp_smem);
    const KConst& kc = c_kc;
    const int s_lo = ua.s_lo, s_hi = ua.s_hi, lpr_log2 = ua.lpr_log2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    const float sca = slice_scale(ua.eba), scb = slice_scale(ua.ebb);
    int st = s_lo + warp, r = st * rpw + ro;
    for (; st < s_hi; st += MV_WARPS, r += MV_WARPS * rpw) {
        const bool ok = r < ua.R;
        const int rn = r + MV_WARPS * rpw;
        const bool more = st + MV_WARPS < s_hi && rn < ua.R;
        u64 acc[NT], accu[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = accu[t] = 0ull;
        if (NT == 1) {      // one pair: the pair kernel's loop (its inputs are read once per block pair for both matrices)
            Chunk na, nb;
            if (more) {   // the next step's streams fly during this step's expansion
                na = load_chunk3(ua.sa, ua.ca, ua.da, (size_t) rn * lpr + jc);
                if (MODE == MODE_GU) nb = load_chunk3(ua.sb, ua.cb, ua.db, (size_t) rn * lpr + jc);
            }
            if (ok) {
                const uint32_t swa[4] = {ka.s.x, ka.s.y, ka.s.z, ka.s.w}, cwa[4] = {ka.c.x, ka.c.y, ka.c.z, ka.c.w};
                const uint32_t swb[4] = {kb.s.x, kb.s.y, kb.s.z, kb.s.w}, cwb[4] = {kb.c.x, kb.c.y, kb.c.z, kb.c.w};
#pragma unroll
                for (int bp = 0; bp < 4; ++bp) {
                    u64 x2[8], xm2[4];
#pragma unroll
                    for (int cq = 0; cq < 4; ++cq) { const ulonglong2 u = sh.sx[0][(bp * 4 + cq) * 32 + jc]; x2[2 * cq] = u.x; x2[2 * cq + 1] = u.y; }
                    offsets_from_sum(sh.ss[0][bp * 32 + jc], xm2);
                    {
                        u64 q[4];
                        pair_coefs(cwa[bp], kc, q);
                        acc[0] = fma2(pair_expand_dot(sh.tab, swa[bp], q, x2, xm2), code_scale_pair(ka.cd, bp, kc), acc[0]);
                    }
                    if (MODE == MODE_GU) {
                        u64 q[4];
                        pair_coefs(cwb[bp], kc, q);
                        accu[0] = fma2(pair_expand_dot(sh.tab, swb[bp], q, x2, xm2), code_scale_pair(kb.cd, bp, kc), accu[0]);
                    }
                }
            }
            ka = na;
            if (MODE == MODE_GU) kb = nb;
        } else {
            // several pairs (or one matrix): a matrix's streams for the next step are requested as soon as this step has
            // used them up, into the registers they leave free, so no second set of stream registers is held
            if (MODE == MODE_GU) {
                if (ok) unit_chunk<NT>(sh.tab, kc, ka, sh.sx, sh.ss, jc, acc);
                if (more) ka = load_chunk3(ua.sa, ua.ca, ua.da, (size_t) rn * lpr + jc);
                if (ok) unit_chunk<NT>(sh.tab, kc, kb, sh.sx, sh.ss, jc, accu);
                if (more) kb = load_chunk3(ua.sb, ua.cb, ua.db, (size_t) rn * lpr + jc);
            } else {      // one matrix: its next streams are requested before this step's expansion (a second set of registers)
                Chunk na;
                if (more) na = load_chunk3(ua.sa, ua.ca, ua.da, (size_t) rn * lpr + jc);
                if (ok) unit_chunk<NT>(sh.tab, kc, ka, sh.sx, sh.ss, jc, acc);
                ka = na;
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float s = group_sum(pair_total(acc[t]), lpr) * sca;
            float su = 0.0f;
            if (MODE == MODE_GU) su = group_sum(pair_total(accu[t]), lpr) * scb;
            if (ok && jc == 0) store_unit<MODE>(ua, ua.pid[t], r, s, su);
        }
    }
}

// Ascending bitonic sort of n (a power of two) keys in shared memory by the whole block.
__device__ __forceinline__ void block_sort(uint32_t* key, int n) {
    for (int k = 2; k <= n; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n; i += MV_THREADS) {
                const int o = i ^ j;
                if (o > i) {
                    const uint32_t x = key[i], y = key[o];
                    if ((x > y) == ((i & k) == 0)) { key[i] = y; key[o] = x; }
                }
            }
            __syncthreads();
        }
}

// In-place exclusive prefix sum of a[0..n) by the whole block, a[n] = the total (n <= GRP_MAX_PAIRS).
__device__ __forceinline__ void block_exclusive_scan(int32_t* a, int n) {
    __shared__ int wtot[MV_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = (n + MV_THREADS - 1) / MV_THREADS, lo = threadIdx.x * per;      // a contiguous run per thread
    int sum = 0;
    for (int i = lo; i < lo + per && i < n; ++i) sum += a[i];
    int inc = sum;
    for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xFFFFFFFFu, inc, o); if (lane >= o) inc += v; }
    if (lane == 31) wtot[warp] = inc;
    __syncthreads();
    int base = inc - sum;
    for (int w = 0; w < warp; ++w) base += wtot[w];
    for (int i = lo; i < lo + per && i < n; ++i) { const int v = a[i]; a[i] = base; base += v; }
    if (threadIdx.x == MV_THREADS - 1) { int t = 0; for (int w = 0; w < MV_WARPS; ++w) t += wtot[w]; a[n] = t; }
    __syncthreads();
}


template <int MODE>
__global__ void __launch_bounds__(MV_THREADS, NSL_GRP_MINB) mv_grp_kernel(MvParams a, KConst kc, int lpr_log2, RouteFuse rf) {
    extern __shared__ __align__(16) unsigned char grp_smem[];
    GrpShared& sh = *reinterpret_cast<GrpShared*>(grp_smem);
    load_stream_tab(sh.tab, a.G, threadIdx.x, MV_THREADS);
    grid_dependents_go();
    grid_dependency_wait();   // everything below may read what the previous kernel in the stream wrote
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = 1 << lpr_log2, rpw = 32 >> lpr_log2;
    const int jc = lane & (lpr - 1), ro = lane >> lpr_log2;
    int P = a.count ? min(*a.count, a.P) : a.P;
    if (rf.logits) {          // the router: one warp per token, every block the same picks
        if (warp < rf.T) {
            const float* l = rf.logits + (size_t) warp * rf.ld;
            if (rf.n_exp <= 128) route_row<4>(rf.n_exp, rf.top_k, l, lane, sh.r_ind + warp * rf.top_k, sh.r_wt + warp * rf.top_k);
            else if (rf.n_exp <= 512) route_row<16>(rf.n_exp, rf.top_k, l, lane, sh.r_ind + warp * rf.top_k, sh.r_wt + warp * rf.top_k);
            else route_row<32>(rf.n_exp, rf.top_k, l, lane, sh.r_ind + warp * rf.top_k, sh.r_wt + warp * rf.top_k);
        }
        P = rf.T * rf.top_k;
        __syncthreads();
        if (blockIdx.x == 0 && (int) threadIdx.x < P) {
            rf.ind_out[threadIdx.x] = sh.r_ind[threadIdx.x];
            rf.wt_out[threadIdx.x] = sh.r_wt[threadIdx.x];
        }
    }
    if (P <= 0) return;
    const int rs = (a.R + rpw - 1) / rpw;             // row steps per unit
#ifdef NSL_GRP_FORCE_PLAIN
    const bool grouped = false;
#else
    const bool grouped = P <= GRP_MAX_PAIRS;
#endif
    long long total;
    if (grouped) {
        const bool small = P <= GRP_SMALL;
        auto slice_of = [&](int i) { return rf.logits ? sh.r_ind[i] : (a.sel ? a.sel[i] : 0); };
        if (small) {      // every thread ranks one key among all: two barriers instead of a sorting network's dozens
            const int i = threadIdx.x;
            uint32_t mine = 0xFFFFFFFFu;
            if (i < P) {
                const int sl = slice_of(i);
                mine = ((uint32_t) sl << 10) | (uint32_t) i;
                sh.tmp[i] = mine;
                if (a.ws) {      // the slice's table entries on their way into L2 while the plan is made
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(a.ws + sl));
                    if (MODE == MODE_GU) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.wu + sl));
                }
            }
            __syncthreads();
            if (i < P) {
                int rank = 0;
                for (int j = 0; j < P; ++j) rank += sh.tmp[j] < mine;
                sh.key[rank] = mine;
            }
            __syncthreads();
        } else {
            int n = 32;
            while (n < P) n <<= 1;
            for (int i = threadIdx.x; i < n; i += MV_THREADS) sh.key[i] = i < P ? ((uint32_t) slice_of(i) << 10) | (uint32_t) i : 0xFFFFFFFFu;
            __syncthreads();
            block_sort(sh.key, n);
        }
        // a sorted position starts a unit when it is a multiple of GRP_NT pairs into its slice's run
        for (int i = threadIdx.x; i < P; i += MV_THREADS) {
            const uint32_t first = sh.key[i] & ~1023u;          // the smallest key of this slice
            int lo = 0, hi = i;                                  // lower bound of `first`
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (sh.key[mid] < first) lo = mid + 1; else hi = mid; }
            int w = 0;
            if ((i - lo) % GRP_NT == 0) {
                int cnt = 1;
                while (cnt < GRP_NT && i + cnt < P && (sh.key[i + cnt] >> 10) == (sh.key[i] >> 10)) ++cnt;
                w = GRP_W[cnt];
            }
            if (small) sh.tmp[i] = (uint32_t) w; else sh.prefix[i] = w;
        }
        __syncthreads();
        if (small) {
            for (int i = threadIdx.x; i <= P; i += MV_THREADS) {
                int before = 0;
                for (int j = 0; j < i; ++j) before += (int) sh.tmp[j];
                sh.prefix[i] = before;
            }
            __syncthreads();
        } else block_exclusive_scan(sh.prefix, P);
        total = (long long) sh.prefix[P] * rs;
    } else {
        __syncthreads();
        total = (long long) P * GRP_W[1] * rs;
    }
    const long long begin = (long long) blockIdx.x * total / gridDim.x, end = (long long) (blockIdx.x + 1) * total / gridDim.x;
    if (begin >= end) return;
    // position in the weighted sequence -> (sorted position of the unit's first pair, row step)
    auto locate = [&](long long x, int& u, int& step) {
        if (!grouped) { u = (int) (x / ((long long) GRP_W[1] * rs)); step = (int) ((x - (long long) u * GRP_W[1] * rs) / GRP_W[1]); return; }
        int lo = 0, hi = P;                                      // the last position whose prefix * rs <= x
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if ((long long) sh.prefix[mid] * rs <= x) lo = mid; else hi = mid; }
        u = lo;
        step = (int) ((x - (long long) sh.prefix[lo] * rs) / (sh.prefix[lo + 1] - sh.prefix[lo]));
    };
    int u_first, s_first, u_last, s_last;
    locate(begin, u_first, s_first);
    if (end >= total) { u_last = P; s_last = 0; } else locate(end, u_last, s_last);
    bool staged = false;
    for (int u = u_first; u <= u_last && u < P;) {
        int n = 1, pid[GRP_NT], slice = 0;
#pragma unroll
        for (int t = 0; t < GRP_NT; ++t) pid[t] = u;
        if (grouped) {
            const int w = sh.prefix[u + 1] - sh.prefix[u];
            n = w == GRP_W[1] ? 1 : w == GRP_W[2] ? 2 : w == GRP_W[3] ? 3 : 4;
#pragma unroll
            for (int t = 0; t < GRP_NT; ++t) pid[t] = (int) (sh.key[u + (t < n ? t : 0)] & 1023u);
            slice = (int) (sh.key[u] >> 10);
        } else slice = rf.logits ? sh.r_ind[u] : (a.sel ? a.sel[u] : 0);
        const int s_lo = u == u_first ? s_first : 0, s_hi = u == u_last ? s_last : rs;
        if (s_lo < s_hi) {
            // Two chains of dependent loads start here and run side by side: pair -> input row -> inputs (this thread's share of
            // the staging, held in registers), and slice -> stream addresses -> this warp's first streams.
            const int per = lpr * 4, n_stage = n * per;
            float xin[16];
            int e0 = threadIdx.x, t0 = e0 / per, rem0 = e0 - t0 * per;
            if (e0 < n_stage) {
                const int p = grouped ? (int) (sh.key[u + t0] & 1023u) : u;
                stage_load(a, a.xrow ? a.xrow[p] : p / a.xdiv, rem0 & (lpr - 1), rem0 >> lpr_log2, xin);
            }
            const WSlice wa = a.ws ? a.ws[slice] : a.w0;
            WSlice wb = wa;
            if (MODE == MODE_GU) wb = a.wu[slice];
            const int st0 = s_lo + warp, r0 = st0 * rpw + ro;
            Chunk ka, kb;
            if (st0 < s_hi && r0 < a.R) {
                ka = load_chunk(wa, (size_t) r0 * lpr + jc);
                if (MODE == MODE_GU) kb = load_chunk(wb, (size_t) r0 * lpr + jc);
            }
            if (staged) __syncthreads();   // the previous unit's inputs are no longer read
            staged = true;
            if (e0 < n_stage) stage_store(xin, rem0 & (lpr - 1), rem0 >> lpr_log2, sh.sx[t0], sh.ss[t0]);
            for (int i = threadIdx.x + MV_THREADS; i < n_stage; i += MV_THREADS) {      // units of more than two pairs
                const int t = i / per, rem = i - t * per;
                const int p = grouped ? (int) (sh.key[u + t] & 1023u) : u;
                stage_load(a, a.xrow ? a.xrow[p] : p / a.xdiv, rem & (lpr - 1), rem >> lpr_log2, xin);
                stage_store(xin, rem & (lpr - 1), rem >> lpr_log2, sh.sx[t], sh.ss[t]);
            }
            __syncthreads();
            UnitArgs ua;
            ua.sa = (const uint4*) wa.p[0]; ua.ca = (const uint4*) wa.p[1]; ua.da = (const uint32_t*) wa.p[3]; ua.eba = wa.eb;
            ua.sb = (const uint4*) wb.p[0]; ua.cb = (const uint4*) wb.p[1]; ua.db = (const uint32_t*) wb.p[3]; ua.ebb = wb.eb;
            ua.y = a.y; ua.ys = a.ys; ua.R = a.R; ua.raw = a.raw; ua.add = a.add;
#pragma unroll
            for (int t = 0; t < 4; ++t) ua.pid[t] = pid[t < GRP_NT ? t : 0];
            ua.s_lo = s_lo; ua.s_hi = s_hi; ua.lpr_log2 = lpr_log2;
            if (GRP_NT >= 4 && n == 4) unit_rows<MODE, GRP_NT >= 4 ? 4 : 1>(ua, ka, kb);
            else if (GRP_NT >= 3 && n == 3) unit_rows<MODE, GRP_NT >= 3 ? 3 : 1>(ua, ka, kb);
            else if (GRP_NT >= 2 && n == 2) unit_rows<MODE, GRP_NT >= 2 ? 2 : 1>(ua, ka, kb);
            else unit_rows<MODE, 1>(ua, ka, kb);
        }
        u += n;
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

// ---- launch selection ---------------------------------------------------------------------------------------------------
static int log2_floor(int v) { int l = 0; while ((2 << l) <= v) ++l; return l; }

template <typename K>
static void allow_smem(K kernel, bool* done, size_t bytes) {      // once per device and kernel
    int dev = 0;
    cudaGetDevice(&dev);
    if (!done[dev & 15]) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) bytes);
        done[dev & 15] = true;
    }
}

template <int MODE, int NT>
static void launch_smemx(cudaStream_t s, const MvParams& a, int lpr_log2, int dense, int grid, size_t smem) {
    static bool attr_set[16];
    allow_smem(mv_smemx_kernel<MODE, NT>, attr_set, (size_t) max_smem_optin() - 4096);
    launch(mv_smemx_kernel<MODE, NT>, grid, MV_THREADS, smem, s, a, kconst(), lpr_log2, dense);
}

// Lists of more than GRP_MIN_PAIRS pairs go to the grouped kernel (one expansion per distinct slice, up to GRP_NT pairs a
// unit): its plan and its costlier second pair pay once a good share of the pairs meet on a slice -- an expert-parallel
// rank's list or all of a 64-row batch; a decode step's 8 .. 64 pairs over 128 experts run faster pair by pair.
constexpr int GRP_MIN_PAIRS = 64;
static int g_grp_min_pairs = GRP_MIN_PAIRS;

template <int MODE>
static void launch_grp(cudaStream_t s, const MvParams& a, int lpr_log2, const RouteFuse& rf) {
    if (a.P <= g_grp_min_pairs || rf.logits) {
        launch(mv_pair_kernel<MODE, 4>, sm_count() * 2, MV_THREADS, 0, s, a, kconst(), lpr_log2, rf);
        return;
    }
    static bool attr_set[16];
    allow_smem(mv_grp_kernel<MODE>, attr_set, sizeof(GrpShared));
    launch(mv_grp_kernel<MODE>, sm_count() * NSL_GRP_MINB, MV_THREADS, sizeof(GrpShared), s, a, kconst(), lpr_log2, rf);
}

// The streams of a slice given by value (a dense call) can be checked on the host; slices in a device table are the
// table builder's to check (nsl_wslice_table does).
static bool slice_aligned(const WSlice& w) {
    return aligned16(w.p[0]) && aligned16(w.p[1]) && ((uintptr_t) w.p[3] & 3u) == 0;
}

template <int MODE>
static void launch_mv(cudaStream_t s, const MvParams& a, int T, const RouteFuse& rf = RouteFuse{}) {
    if (a.R <= 0 || a.P <= 0 || T <= 0) return;
    if (a.K <= 0 || a.K % 8) { set_error("seed mat-vec: K = %d is not a multiple of 8", a.K); return; }
    if (T > MV_MAXT) { set_error("seed mat-vec: %d tokens, at most %d", T, MV_MAXT); return; }
    const int dense = a.sel == NULL && rf.logits == NULL, sms = sm_count();
    const int ch = a.K / 64;
    // The chunked kernels read whole chunks with 16-byte loads: rows of inputs and (checked where the slice is on the
    // host) the streams must be aligned for that; anything else goes to the any-shape kernel.
    const bool chunked = a.K % 64 == 0 && aligned16(a.x) && a.xs % (a.xbf16 ? 8 : 4) == 0 && (a.ws != NULL || slice_aligned(a.w0));
    const bool pow2 = ch > 0 && (ch & (ch - 1)) == 0;
    if ((a.xrow || a.count || a.xbf16 || rf.logits) && !(chunked && pow2 && ch <= 32 && T == 1)) {
        set_error("seed mat-vec: the routed / row-index / device-count / bf16-input forms need K = 64 * 2^j <= 2048 and aligned rows (K = %d)", a.K);
        return;
    }
    if (chunked && T == 1 && pow2 && ch <= 32) {
        launch_grp<MODE>(s, a, log2_floor(ch), rf);
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

// P = 3 (SEED4): the pair kernel for rows of 64 * 2^j <= 2048 weights -- the routed experts' gathers, and a dense call as T
// "pairs" on the one slice (token t reads input row t and writes output row t; every token expands the rows itself, so a
// token's result cannot depend on the others) -- the any-shape kernel for everything else.
template <int MODE>
static void launch_mv3(cudaStream_t s, const MvParams& a, int T) {
    if (a.R <= 0 || a.P <= 0 || T <= 0) return;
    if (a.K <= 0 || a.K % 8) { set_error("seed mat-vec: K = %d is not a multiple of 8", a.K); return; }
    if (T > MV_MAXT) { set_error("seed mat-vec: %d tokens, at most %d", T, MV_MAXT); return; }
    const int ch = a.K / 64;
    const bool chunked = a.K % 64 == 0 && aligned16(a.x) && a.xs % 4 == 0 && (a.ws != NULL || (aligned16(a.w0.p[0]) && aligned16(a.w0.p[1])));
    if (chunked && ch > 0 && (ch & (ch - 1)) == 0 && ch <= 32) {
        launch(mv_pair_kernel<MODE, 3>, sm_count() * 2, MV_THREADS, 0, s, a, kconst(), log2_floor(ch), RouteFuse{});
        count_launch();
        return;
    }
    launch(mv_generic_kernel<MODE, 3>, sm_count() * 2, MV_THREADS, 0, s, a, kconst(), a.sel ? 1 : T);
    count_launch();
}

// The decode step in one launch; false (nothing launched) when a size is outside what the pair kernel serves.
static bool launch_mv_step(cudaStream_t s, const StepParams& p) {
    const int cd = p.d / 64, cf = p.ff / 64;
    if (p.T < 1 || p.T > MV_MAXT || p.top_k < 1 || p.top_k > 32 || p.T * p.top_k > 256 || p.n_exp < p.top_k || p.n_exp > 32 * ROUTE_PER_LANE) return false;
    if (p.d % 64 || p.ff % 64 || cd < 1 || cf < 1 || (cd & (cd - 1)) || (cf & (cf - 1)) || cd > 32 || cf > 32) return false;
    if (!aligned16(p.x) || p.xs % 4 || !aligned16(p.A) || !aligned16(p.D)) return false;
    launch(mv_step_kernel, sm_count() * 2, MV_THREADS, 0, s, p, kconst(), log2_floor(cd), log2_floor(cf));
    count_launch();
    return true;
}

bool launch_q4_mv(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add);
void launch_bf16_mv(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add);
bool launch_bf16_mm_skinny(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add);

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
    if (fmt == MF_BF16) {      // stored BF16 weights (dense_bf16.cu): the tensor-core kernel where its shape rules allow, else a warp per row
        if (!launch_bf16_mm_skinny(s, w, K, R, x, xs, y, ys, T, add)) launch_bf16_mv(s, w, K, R, x, xs, y, ys, T, add);
        return;
    }
    if (!seed_fmt(fmt, "kc_mv")) return;
    MvParams a = {NULL, NULL, w, NULL, x, y, G, K, R, T, 1, xs, ys, add, 0, NULL, NULL, 0};
    if (fmt == MF_SEED4) launch_mv3<MODE_ROUND>(s, a, T);
    else launch_mv<MODE_ROUND>(s, a, T);
}

void kc_mv_sel(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
               const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    if (!seed_fmt(fmt, "kc_mv_sel")) return;
    MvParams a = {ws, NULL, WSlice{}, sel, x, y, G, K, R, P, xdiv, xs, ys, 0, 0, NULL, NULL, 0};
    if (fmt == MF_SEED4) launch_mv3<MODE_ROUND>(s, a, 1);
    else launch_mv<MODE_ROUND>(s, a, 1);
}

void kc_mv_gu(cudaStream_t s, int fmt, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* out,
              int ys, const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    if (!seed_fmt(fmt, "kc_mv_gu")) return;
    MvParams a = {wg, wu, WSlice{}, sel, x, out, G, K, R, P, xdiv, xs, ys, 0, 0, NULL, NULL, 0};
    if (fmt == MF_SEED4) launch_mv3<MODE_GU>(s, a, 1);
    else launch_mv<MODE_GU>(s, a, 1);
}

void nsl_mv_raw(cudaStream_t s, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    MvParams a = {sel ? ws : NULL, NULL, WSlice{}, sel, x, y, G, K, R, P, xdiv > 0 ? xdiv : 1, xs, ys, 0, 1, NULL, NULL, 0};
    if (!sel) a.w0 = *ws;   // dense: ws is a host pointer to the one slice
    launch_mv<MODE_ROUND>(s, a, sel ? 1 : P);
}

void nsl_mv_gu_raw(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* out,
                   int ys, const int32_t* sel, int P, int xdiv, const uint32_t* G) {
    MvParams a = {wg, wu, WSlice{}, sel, x, out, G, K, R, P, xdiv, xs, ys, 0, 1, NULL, NULL, 0};
    launch_mv<MODE_GU>(s, a, 1);
}

// kc_mv_gu with the router folded into its prologue: T <= MV_MAXT rows of logits -> ind / wt [T][top_k] and
// a [T * top_k][R]; pair t * top_k + j uses expert ind[t][j] and input row t.
void nsl_mv_gu_routed(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* out, int ys,
                      int n_exp, int top_k, const float* logits, int ld, int T, int32_t* ind, float* wt, int raw, const uint32_t* G) {
    if (T <= 0) return;
    if (T > MV_MAXT || n_exp < 1 || n_exp > 32 * ROUTE_PER_LANE || top_k < 1 || top_k > 32 || top_k > n_exp) {
        set_error("nsl_mv_gu_routed: %d rows (at most %d), %d experts (at most %d), top %d (at most 32)", T, MV_MAXT, n_exp,
                  32 * ROUTE_PER_LANE, top_k);
        return;
    }
    MvParams a = {wg, wu, WSlice{}, NULL, x, out, G, K, R, T * top_k, top_k, xs, ys, 0, raw, NULL, NULL, 0};
    const RouteFuse rf = {logits, ld, n_exp, top_k, T, ind, wt};
    launch_mv<MODE_GU>(s, a, 1, rf);
}

// The whole decode step of an expert layer (router, gate + up + SwiGLU, down, combine) as one launch: 1 = launched, 0 = a
// size is outside what it serves (nothing launched: the caller issues the three launches).  sync: 4 * (2 + T + T * top_k)
// bytes of device memory, zero before the first call; every call leaves its counters zero.  sync[0] is the status word:
// 1 after a launch in which a bounded wait ran out (its output is not valid), for the caller to read and clear.
// A and D are the caller's work buffers [T * top_k][ff] and [T * top_k][d].
int nsl_mv_step(cudaStream_t s, const WSlice* wg, const WSlice* wu, const WSlice* wd, int d, int ff, const float* x, int xs, int n_exp,
                int top_k, const float* logits, int ld, int T, int32_t* ind, float* wt, float* A, float* D, float* out, int raw,
                unsigned* sync, const uint32_t* G) {
    if (!sync || T < 1 || top_k < 1) return 0;
    StepParams p = {wg, wu, wd, x, logits, A, D, out, ind, wt, G, xs, ld, n_exp, top_k, T, d, ff, raw,
                    {sync + 2 + T, sync + 2, sync + 1, (int*) sync}};
    return launch_mv_step(s, p) ? 1 : 0;
}

// Expert-parallel forms: a compacted pair list whose length lives on the device.  Pair p uses slice sel[p] and input
// row xrow[p] of x, which holds packed bf16 rows when x_bf16 is set; at most max_pairs pairs, *count of them valid.
void nsl_mv_gu_rows(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const void* x, int xs, int x_bf16,
                    float* out, int ys, const int32_t* sel, const int32_t* xrow, int max_pairs, const int32_t* count,
                    int raw, const uint32_t* G) {
    MvParams a = {wg, wu, WSlice{}, sel, (const float*) x, out, G, K, R, max_pairs, 1, xs, ys, 0, raw, xrow, count, x_bf16};
    launch_mv<MODE_GU>(s, a, 1);
}
void nsl_mv_sel_rows(cudaStream_t s, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                     const int32_t* sel, int max_pairs, const int32_t* count, int raw, const uint32_t* G) {
    MvParams a = {ws, NULL, WSlice{}, sel, x, y, G, K, R, max_pairs, 1, xs, ys, 0, raw, NULL, count, 0};
    launch_mv<MODE_ROUND>(s, a, 1);
}


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
