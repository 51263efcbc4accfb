// The small kernels a decoder layer needs around the seed mat-vecs and the attention: embedding rows, the grouped RMSNorm,
// RoPE with the KV-cache write, and the residual add.  Behaviour (engine/kernels_moe.cu:676-713, 837-885):
//   kc_embed    x[t] = BF16 row ids[t] of the table
//   kc_gnorm    y = bf16(w * (x * rsqrt(mean over the element's half of the row of x^2 + eps))), w in BF16
//   kc_rope_kv  non-interleaved rotary embedding (pairs p, p + 64 of a 128-wide head, angle pos * inv[p]) on q in place
//               (rounded to bf16) and on k into the cache; v into the cache; a BF16 cache or the 8-bit one (one f32 scale per
//               row and KV head = max |bf16 value| / 127, codes rounded to nearest even)
#include <math.h>

#include "common.cuh"
#include "seed_block.cuh"

namespace nsl {

constexpr int HD = 128;      // head width of the attention kernels

__device__ __forceinline__ float bf16_to_f32(uint16_t b) { return __uint_as_float((uint32_t) b << 16); }

__global__ void __launch_bounds__(256) embed_bf16_kernel(const uint16_t* __restrict__ table, int d, const int32_t* __restrict__ ids,
                                                         float* __restrict__ x) {
    const int t = blockIdx.y;
    const uint16_t* row = table + (size_t) ids[t] * d;
    for (int c = blockIdx.x * 256 + threadIdx.x; c < d; c += gridDim.x * 256) x[(size_t) t * d + c] = bf16_to_f32(row[c]);
}

// One block per row; threads 0..127 own the first half of the row, 128..255 the second, so each half's mean square is a
// reduction over four warps and no element asks which group it is in.
__global__ void __launch_bounds__(256) gnorm_kernel(int d, float eps, const float* __restrict__ x, const uint16_t* __restrict__ w,
                                                    float* __restrict__ y) {
    __shared__ float part[8];
    grid_dependents_go();
    grid_dependency_wait();
    const int t = blockIdx.x, half = threadIdx.x >> 7, i0 = threadIdx.x & 127, hw = d / 2;
    const float* xr = x + (size_t) t * d + (size_t) half * hw;
    float s = 0.0f;
    for (int c = i0; c < hw; c += 128) { const float v = xr[c]; s = fmaf(v, v, s); }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    const float tot = ((part[4 * half] + part[4 * half + 1]) + part[4 * half + 2]) + part[4 * half + 3];
    const float r = rsqrtf(tot / (float) hw + eps);
    const uint16_t* wr = w + (size_t) half * hw;
    float* yr = y + (size_t) t * d + (size_t) half * hw;
    for (int c = i0; c < hw; c += 128) yr[c] = bf16_round(bf16_to_f32(wr[c]) * (xr[c] * r));
}

// One warp per (row, head): lane l rotates the pairs (l, l + 64) and (l + 32, l + 96).  Heads below n_head are query heads
// (rotated in place); heads below n_kv also carry that KV head's key and value into the cache.
__global__ void __launch_bounds__(128) rope_kv_kernel(float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, KvView kv,
                                                      const RowInfo* __restrict__ ri, const float* __restrict__ inv, int n_head, int n_kv, int heads) {
    grid_dependents_go();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, head = blockIdx.x * 4 + (threadIdx.x >> 5), t = blockIdx.y;
    if (head >= heads) return;
    const int pos = ri[t].pos;
    float sn[2], cs[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) sincosf((float) pos * inv[lane + 32 * j], &sn[j], &cs[j]);
    if (head < n_head) {
        float* qh = q + ((size_t) t * n_head + head) * HD;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int p = lane + 32 * j;
            const float a = qh[p], b = qh[p + 64];
            qh[p] = bf16_round(a * cs[j] - b * sn[j]);
            qh[p + 64] = bf16_round(b * cs[j] + a * sn[j]);
        }
    }
    if (head >= n_kv) return;      // uniform over the warp
    const float* kh = k + ((size_t) t * n_kv + head) * HD;
    const float* vh = v + ((size_t) t * n_kv + head) * HD;
    float kr[4], vr[4];      // dims lane, lane + 64, lane + 32, lane + 96
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int p = lane + 32 * j;
        const float a = kh[p], b = kh[p + 64];
        kr[2 * j] = a * cs[j] - b * sn[j];
        kr[2 * j + 1] = b * cs[j] + a * sn[j];
        vr[2 * j] = vh[p];
        vr[2 * j + 1] = vh[p + 64];
    }
    int row = ri[t].kv0 + pos;      // the sequence slot's cache row: positions below nv in segment a, the rest in b
    const KvSeg sg = row < kv.nv ? kv.a : kv.b;
    if (row >= kv.nv) row -= kv.nv;
    const size_t off = ((size_t) row * n_kv + head) * HD;
    if (kv.fmt == KV_BF16) {
        uint16_t* kc = (uint16_t*) sg.k + off;
        uint16_t* vc = (uint16_t*) sg.v + off;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int p = lane + 32 * j;
            kc[p] = bf16_bits(kr[2 * j]); kc[p + 64] = bf16_bits(kr[2 * j + 1]);
            vc[p] = bf16_bits(vr[2 * j]); vc[p + 64] = bf16_bits(vr[2 * j + 1]);
        }
        return;
    }
    float mk = 0.0f, mv = 0.0f;      // the 8-bit cache quantizes the values the BF16 cache would hold
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        kr[i] = bf16_round(kr[i]); vr[i] = bf16_round(vr[i]);
        mk = fmaxf(mk, fabsf(kr[i])); mv = fmaxf(mv, fabsf(vr[i]));
    }
    for (int o = 16; o > 0; o >>= 1) { mk = fmaxf(mk, __shfl_xor_sync(0xFFFFFFFFu, mk, o)); mv = fmaxf(mv, __shfl_xor_sync(0xFFFFFFFFu, mv, o)); }
    const float sk = mk > 0.0f ? mk / 127.0f : 1.0f, sv = mv > 0.0f ? mv / 127.0f : 1.0f;
    int8_t* kc = (int8_t*) sg.k + off;
    int8_t* vc = (int8_t*) sg.v + off;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int p = lane + 32 * j;
        kc[p] = (int8_t) __float2int_rn(kr[2 * j] / sk); kc[p + 64] = (int8_t) __float2int_rn(kr[2 * j + 1] / sk);
        vc[p] = (int8_t) __float2int_rn(vr[2 * j] / sv); vc[p + 64] = (int8_t) __float2int_rn(vr[2 * j + 1] / sv);
    }
    if (lane == 0) {
        sg.ks[(size_t) row * n_kv + head] = sk;
        sg.vs[(size_t) row * n_kv + head] = sv;
    }
}

// x[i] = bf16(x[i] + y[i]): the residual stream holds bf16-valued numbers.
__global__ void residual_add_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
    grid_dependents_go();
    grid_dependency_wait();
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t) gridDim.x * blockDim.x) x[i] = bf16_round(x[i] + y[i]);
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void kc_embed(cudaStream_t s, int fmt, WSlice w, int d, const int32_t* ids, float* x, int T) {
    if (T <= 0 || d <= 0) return;
    if (fmt != MF_BF16) { set_error("kc_embed: table format %d is not served by this library (BF16 = %d only)", fmt, (int) MF_BF16); return; }
    embed_bf16_kernel<<<dim3((unsigned) ((d + 255) / 256 < 8 ? (d + 255) / 256 : 8), (unsigned) T), 256, 0, s>>>((const uint16_t*) w.p[0], d, ids, x);
    count_launch();
}

void kc_gnorm(cudaStream_t s, int d, float eps, const float* x, const uint16_t* w, float* y, int T) {
    if (T <= 0) return;
    if (d < 2 || d % 2) { set_error("kc_gnorm: width %d must be even (two groups)", d); return; }
    launch(gnorm_kernel, (unsigned) T, 256, 0, s, d, eps, x, w, y);
    count_launch();
}

void kc_rope_kv(cudaStream_t s, float* q, const float* k, const float* v, KvView kv, const RowInfo* ri, const float* inv, int n_head,
                int n_kv, int T) {
    if (T <= 0) return;
    if (kv.fmt != KV_BF16 && kv.fmt != KV_Q8) { set_error("kc_rope_kv: KV cache format %d is not served (BF16 and Q8 only)", kv.fmt); return; }
    if (n_head < 1 || n_kv < 1 || (kv.fmt == KV_Q8 && (!kv.a.ks || !kv.a.vs))) { set_error("kc_rope_kv: %d query / %d KV heads, or an 8-bit cache without scales", n_head, n_kv); return; }
    const int heads = n_head > n_kv ? n_head : n_kv;
    launch(rope_kv_kernel, dim3((unsigned) (heads + 3) / 4, (unsigned) T), 128, 0, s, q, k, v, kv, ri, inv, n_head, n_kv, heads);
    count_launch();
}

void nsl_residual_add(cudaStream_t s, float* x, const float* y, size_t n) {
    if (!n) return;
    const size_t blocks = (n + 255) / 256;
    launch(residual_add_kernel, (unsigned) (blocks < (size_t) sm_count() * 8 ? blocks : (size_t) sm_count() * 8), 256, 0, s, x, y, n);
    count_launch();
}

}   // extern "C"
