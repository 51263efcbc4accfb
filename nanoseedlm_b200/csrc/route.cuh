// The softmax top-k router of one row by one warp (engine/kernels_qwen4.cu:385-422, nslm/lib_qwen4_ops.c:107-122).
#pragma once
#include <math.h>
#include <stdint.h>

namespace nsl {

constexpr uint32_t FULL = 0xFFFFFFFFu;
constexpr int ROUTE_PER_LANE = 32;   // experts <= 1024

// Lane l holds experts l, l+32, ..; k rounds of a warp arg-max where equal logits go to the higher expert id, best first;
// weights exp(l - max) renormalised over the k picked.  E <= 32 * PER, k <= 32.  ind_row / wt_row: k entries, global or
// shared memory, written by lane 0 and lanes 0..k-1.
template <int PER>
__device__ __forceinline__ void route_row(int E, int k, const float* __restrict__ l, int lane, int32_t* ind_row, float* wt_row) {
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? l[e] : -INFINITY;
        mx = fmaxf(mx, v[j]);
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
    float top = 0.0f, mine = 0.0f;   // lane r keeps round r's unnormalised weight
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = -1;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int e = lane + 32 * j;
            if (e < E && (v[j] > bv || (v[j] == bv && e > bi))) { bv = v[j]; bi = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(FULL, bv, o);
            const int oi = __shfl_xor_sync(FULL, bi, o);
            if (ov > bv || (ov == bv && oi > bi)) { bv = ov; bi = oi; }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (lane + 32 * j == bi) v[j] = -INFINITY;
        const float w = expf(bv - mx);
        top += w;
        if (lane == r) mine = w;
        if (lane == 0) ind_row[r] = bi;
    }
    if (lane < k) wt_row[lane] = mine / top;
}

}   // namespace nsl
