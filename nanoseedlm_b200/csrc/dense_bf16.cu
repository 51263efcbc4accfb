// Dense mat-vec over stored BF16 weights (kc_mv with MF_BF16; engine/kernels_moe.cu:92, 596: y[t][r] = bf16(W[r] . x[t]), f32
// sums, optional residual add as store_y).  An HBM-bound kernel: a warp owns a row at a time and reads it as 16-byte
// pieces (8 weights a lane, 512 contiguous bytes a warp), the tokens' inputs come from L1; a token's sum is formed in the
// same order whatever the number of tokens in the call.
#include "common.cuh"
#include "seed_block.cuh"

namespace nsl {

template <int NT>
__global__ void __launch_bounds__(256) bf16_mv_kernel(const uint16_t* __restrict__ W, int K, int R, const float* __restrict__ x, int xs,
                                                      float* __restrict__ y, int ys, int T, int add) {
    grid_dependents_go();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int nchunk = K / 8;
    for (int r = blockIdx.x * 8 + (threadIdx.x >> 5); r < R; r += gridDim.x * 8) {
        const uint4* wr = (const uint4*) (W + (size_t) r * K);
        float acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.0f;
        for (int c = lane; c < nchunk; c += 32) {
            const uint4 q = __ldg(wr + c);
            const uint32_t u[4] = {q.x, q.y, q.z, q.w};
            float w[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) { w[2 * i] = __uint_as_float(u[i] << 16); w[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u); }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                if (t >= T) break;
                const float4* xp = (const float4*) (x + (size_t) t * xs + 8 * c);
                const float4 a = __ldg(xp), b = __ldg(xp + 1);
                float s = acc[t];
                s = fmaf(w[0], a.x, s); s = fmaf(w[1], a.y, s); s = fmaf(w[2], a.z, s); s = fmaf(w[3], a.w, s);
                s = fmaf(w[4], b.x, s); s = fmaf(w[5], b.y, s); s = fmaf(w[6], b.z, s); s = fmaf(w[7], b.w, s);
                acc[t] = s;
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            if (t >= T) break;
            float s = acc[t];
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
            if (lane == 0) {
                float* yo = y + (size_t) t * ys + r;
                *yo = add ? bf16_round(*yo + bf16_round(s)) : bf16_round(s);      // engine/kernels_moe.cu:214
            }
        }
    }
}

void launch_bf16_mv(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add) {
    if (R <= 0 || T <= 0) return;
    if (T > MV_MAXT || K <= 0 || K % 8 || !aligned16(w.p[0]) || !aligned16(x) || xs % 4) {
        set_error("kc_mv (BF16): %d tokens (at most %d), K = %d (a multiple of 8), weights and inputs 16-byte aligned", T, MV_MAXT, K);
        return;
    }
    const int blocks = (R + 7) / 8 < sm_count() * 8 ? (R + 7) / 8 : sm_count() * 8;
    if (T <= 2) launch(bf16_mv_kernel<2>, blocks, 256, 0, s, (const uint16_t*) w.p[0], K, R, x, xs, y, ys, T, add);
    else if (T <= 4) launch(bf16_mv_kernel<4>, blocks, 256, 0, s, (const uint16_t*) w.p[0], K, R, x, xs, y, ys, T, add);
    else launch(bf16_mv_kernel<8>, blocks, 256, 0, s, (const uint16_t*) w.p[0], K, R, x, xs, y, ys, T, add);
    count_launch();
}

}   // namespace nsl
