// Softmax top-k routing of one row by one warp (behaviour: nslm/lib_qwen4_ops.c:107-122 -- the k largest logits, equal
// logits to the higher expert id, best first, weights exp(l - max) renormalised over the k picked).
//
// Selection by ordered integer keys.  A logit becomes a 32-bit key whose unsigned order is the float order, so "largest
// value, then largest id" is two warp-wide integer maxima (redux.sync): first over the lanes' best keys, then over the ids
// of the lanes that hold that key.  Each lane keeps the best of its own experts cached; after a round only the lane that
// owned the winner retires it (key 0 sorts below every float, -inf included) and rescans its registers.
#pragma once
#include <math.h>
#include <stdint.h>

namespace nsl {

constexpr uint32_t FULL = 0xFFFFFFFFu;
constexpr int ROUTE_PER_LANE = 32;   // experts <= 1024

__device__ __forceinline__ uint32_t route_key(float f) {       // monotone: a < b  <=>  key(a) < key(b)
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float route_unkey(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// Lane l holds experts l, l + 32, ...  E <= 32 * PER, k <= 32, k <= E.  ind_row / wt_row: k entries in global or shared
// memory; ind_row is written by lane 0, wt_row by lanes 0..k-1.
template <int PER>
__device__ __forceinline__ void route_row(int E, int k, const float* __restrict__ l, int lane, int32_t* ind_row, float* wt_row) {
    uint32_t key[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        key[j] = e < E ? route_key(l[e]) : 0u;
    }
    uint32_t best = 0u;      // this lane's largest key and the slot that holds it (the later slot on equal keys: higher id)
    int slot = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j)
        if (key[j] >= best && key[j] != 0u) { best = key[j]; slot = j; }
    float mx = 0.0f, total = 0.0f, mine = 0.0f;
    for (int r = 0; r < k; ++r) {
        const uint32_t top = __reduce_max_sync(FULL, best);
        const uint32_t id1 = __reduce_max_sync(FULL, best == top ? (uint32_t) (lane + 32 * slot + 1) : 0u);   // id + 1 of the winner
        const int win = (int) id1 - 1;
        const float v = route_unkey(top);
        if (r == 0) mx = v;
        const float w = expf(v - mx);
        total += w;
        if (lane == r) mine = w;
        if (lane == 0) ind_row[r] = win;
        if ((win & 31) == lane) {       // the owner retires the winner and finds its next best
            best = 0u;
            slot = 0;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                if (j == (win >> 5)) key[j] = 0u;
                if (key[j] >= best && key[j] != 0u) { best = key[j]; slot = j; }
            }
        }
    }
    if (lane < k) wt_row[lane] = mine / total;
}

}   // namespace nsl
