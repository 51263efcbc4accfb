// Decode attention over a BF16 KV cache with grouped query heads: split-key partial passes and their reduction with the
// softplus output gate (engine/kernels_moe.cu:887-952, 2421-2426; engine/kernels_cuda.h:56-72, 130-131).
//
// One block per (split, KV head, row); one warp per query head of the KV head (any group size up to 16, where the
// reference fixes 4).  The two halves of a step of 32 keys use two thread layouts, so that neither needs a reduction
// per key:
//   scores   lane = key: a lane walks its own key's 128 values against the head's scaled query in shared memory;
//   values   lane = 4 dims: the 32 weights are broadcast by shuffle and every V row is one 256-byte read.
// The step's K and V rows are copied into shared memory once for the group (cp.async, the next step's rows in flight
// while this one is computed); K rows sit 272 bytes apart there so that 32 lanes walking 32 rows touch distinct banks
// (read straight from global memory the same walk costs 32 L1 wavefronts per load: 326 us against 134 MB per layer).
// The online softmax rescales once per step.  Partials and the reduction have the reference's layout and rounding
// points: part[row][head][split] = (m, l, acc[128]); o = bf16(bf16(acc / l) * bf16(softplus(g))).
#include <math.h>

#include "common.cuh"
#include "seed_block.cuh"

namespace nsl {

constexpr int ATT_HD = 128, ATT_MAX_GROUP = 16;

__device__ __forceinline__ const uint16_t* kv_row(const KvView& kv, int is_v, int abs_pos, int n_kv, int kvh) {
    const bool first = abs_pos < kv.nv;
    const KvSeg& sg = first ? kv.a : kv.b;
    const int row = first ? abs_pos : abs_pos - kv.nv;
    return (const uint16_t*) (is_v ? sg.v : sg.k) + ((size_t) row * n_kv + kvh) * ATT_HD;
}
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

constexpr int ATT_TILE = 32, ATT_KROW = 272;      // keys per step; bytes of a staged K row (256 + 16: conflict-free row walks)

__device__ __forceinline__ void attn_cp16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}

__global__ void __launch_bounds__(32 * ATT_MAX_GROUP) attn_split_kernel(AttnArgs a, const float* __restrict__ q, KvView kv,
                                                                        const RowInfo* __restrict__ ri, float* __restrict__ part) {
    __shared__ __align__(16) float qs[ATT_MAX_GROUP][ATT_HD];
    __shared__ __align__(16) unsigned char kt[2][ATT_TILE * ATT_KROW];      // the step's K rows, shared by the group's warps
    __shared__ __align__(16) unsigned char vt[2][ATT_TILE * 256];           // and its V rows
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = a.n_head / a.n_kv, qh = kvh * group + warp;
    grid_dependents_go();
    grid_dependency_wait();
    {
        const float4 v = *(const float4*) (q + ((size_t) t * a.n_head + qh) * ATT_HD + lane * 4);
        *(float4*) &qs[warp][lane * 4] = make_float4(v.x * a.scale, v.y * a.scale, v.z * a.scale, v.w * a.scale);
    }
    const int pos = ri[t].pos, kv0 = ri[t].kv0;
    const int nsr = a.chunk > 0 ? min(a.n_splits, (pos + a.chunk) / a.chunk) : 1;   // this row's split count, whatever rows share the call
    const int chunk = (pos + nsr) / nsr;                          // ceil((pos + 1) / nsr)
    const int p0 = split * chunk, p1 = min(pos + 1, p0 + chunk);  // splits >= nsr are empty
    // the block's threads copy a step's 32 K rows and 32 V rows (16 pieces of 16 bytes each) into a stage
    auto stage_in = [&](int st, int p) {
        for (int i = threadIdx.x; i < 2 * ATT_TILE * 16; i += blockDim.x) {
            const int is_v = i >= ATT_TILE * 16, r = (i >> 4) & (ATT_TILE - 1), piece = i & 15;
            const uint16_t* src = kv_row(kv, is_v, kv0 + min(p + r, p1 - 1), a.n_kv, kvh) + piece * 8;
            attn_cp16(is_v ? vt[st] + r * 256 + piece * 16 : kt[st] + r * ATT_KROW + piece * 16, src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float m = -INFINITY, l = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (p0 < p1) stage_in(0, p0);
    int st = 0;
    for (int p = p0; p < p1; p += ATT_TILE, st ^= 1) {
        if (p + ATT_TILE < p1) {
            stage_in(st ^ 1, p + ATT_TILE);      // the next step's rows fly while this one is computed
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const bool valid = p + lane < p1;
        const unsigned char* kr = kt[st] + lane * ATT_KROW;
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint4 k8 = *(const uint4*) (kr + j * 16);
            const float4 qa = *(const float4*) &qs[warp][8 * j], qb = *(const float4*) &qs[warp][8 * j + 4];
            s = fmaf(qa.x, bf_lo(k8.x), s); s = fmaf(qa.y, bf_hi(k8.x), s);
            s = fmaf(qa.z, bf_lo(k8.y), s); s = fmaf(qa.w, bf_hi(k8.y), s);
            s = fmaf(qb.x, bf_lo(k8.z), s); s = fmaf(qb.y, bf_hi(k8.z), s);
            s = fmaf(qb.z, bf_lo(k8.w), s); s = fmaf(qb.w, bf_hi(k8.w), s);
        }
        if (!valid) s = -INFINITY;
        float mx = s;
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        mx = fmaxf(mx, m);
        const float cor = expf(m - mx), e = valid ? expf(s - mx) : 0.0f;
        l = fmaf(l, cor, e);      // per lane: the lanes' sums meet once, after the last step
        acc.x *= cor; acc.y *= cor; acc.z *= cor; acc.w *= cor;
        m = mx;
        const int nk = min(ATT_TILE, p1 - p);
        const uint2* vr = (const uint2*) vt[st] + lane;
        for (int kk = 0; kk < nk; ++kk) {
            const float pk = __shfl_sync(0xFFFFFFFFu, e, kk);
            const uint2 v4 = vr[kk * 32];
            acc.x = fmaf(pk, bf_lo(v4.x), acc.x); acc.y = fmaf(pk, bf_hi(v4.x), acc.y);
            acc.z = fmaf(pk, bf_lo(v4.y), acc.z); acc.w = fmaf(pk, bf_hi(v4.y), acc.w);
        }
        __syncthreads();      // the stage may be refilled by the step after next
    }
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, o);
    float* pp = part + (((size_t) t * a.n_head + qh) * a.n_splits + split) * (ATT_HD + 2);
    if (lane == 0) { pp[0] = m; pp[1] = l; }
    pp[2 + lane * 4 + 0] = acc.x; pp[2 + lane * 4 + 1] = acc.y; pp[2 + lane * 4 + 2] = acc.z; pp[2 + lane * 4 + 3] = acc.w;
}

__device__ __forceinline__ float softplus_ln2(float g) {   // softplus with beta = ln 2 in f32, then BF16
    const float gx = g * 0.69314718055994531f;
    return bf16_round((fmaxf(gx, 0.0f) + logf(1.0f + expf(-fabsf(gx)))) / 0.69314718055994531f);
}

__global__ void __launch_bounds__(ATT_HD) attn_reduce_kernel(AttnArgs a, const float* __restrict__ part, const float* __restrict__ g,
                                                             float* __restrict__ o) {
    const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
    grid_dependents_go();
    grid_dependency_wait();
    const float* pp = part + ((size_t) t * a.n_head + h) * a.n_splits * (ATT_HD + 2);
    float m = -INFINITY;
    for (int s = 0; s < a.n_splits; ++s) m = fmaxf(m, pp[s * (ATT_HD + 2)]);
    float l = 0.0f, acc = 0.0f;
    for (int s = 0; s < a.n_splits; ++s) {
        const float ms = pp[s * (ATT_HD + 2)];
        if (ms == -INFINITY) continue;
        const float c = expf(ms - m);
        l = fmaf(pp[s * (ATT_HD + 2) + 1], c, l);
        acc = fmaf(pp[s * (ATT_HD + 2) + 2 + d], c, acc);
    }
    const float att = bf16_round(acc / l);
    const size_t i = ((size_t) t * a.n_head + h) * ATT_HD + d;
    o[i] = g ? bf16_round(att * softplus_ln2(g[i])) : att;
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void kc_attn(cudaStream_t s, AttnArgs a, const float* q, KvView kv, const RowInfo* ri, float* part, const float* g, float* o, int T) {
    if (T < 1) return;
    if (kv.fmt != KV_BF16) { set_error("kc_attn: KV cache format %d is not served by this library (BF16 = %d only)", kv.fmt, (int) KV_BF16); return; }
    const int group = a.n_kv > 0 ? a.n_head / a.n_kv : 0;
    if (a.n_kv < 1 || a.n_head % a.n_kv || group < 1 || group > ATT_MAX_GROUP || a.n_splits < 1 || a.chunk < 0 || (a.chunk == 0 && a.n_splits > 1) || !aligned16(q) ||
        !aligned16(kv.a.k) || !aligned16(kv.a.v) || (kv.b.k && (!aligned16(kv.b.k) || !aligned16(kv.b.v)))) {
        set_error("kc_attn: %d query heads over %d KV heads (groups of 1..%d), %d splits of %d keys, or unaligned buffers", a.n_head,
                  a.n_kv, (int) ATT_MAX_GROUP, a.n_splits, a.chunk);
        return;
    }
    launch(attn_split_kernel, dim3((unsigned) a.n_splits, (unsigned) a.n_kv, (unsigned) T), 32 * group, 0, s, a, q, kv, ri, part);
    PdlScope chain(true);      // the reduction's blocks come in while the split pass drains
    launch(attn_reduce_kernel, dim3((unsigned) a.n_head, (unsigned) T), ATT_HD, 0, s, a, (const float*) part, g, o);
    count_launch(2);
}

}   // extern "C"
