// The affine int4 dense mat-vec (the LM head's format: engine/kernels_moe.cu:171-189, MLX's qmv form) and the greedy
// arg-max over its logits (engine/kernels_moe.cu:2115-2151).
//
// Format MF_Q4: codes u32 [R][K/8], eight 4-bit values q in [0, 15] per word (value i in bits 4i..4i+3); per group of
// 64 weights along K a bf16 scale s and a bf16 bias b; weight = s q + b.  Per group and token the reference adds
// s * sum(q x) + b * sum(x) in f32.
//
// This kernel is bound by HBM (0.5625 B per weight: 4 bits + 2 x 16 bits per 64), not by the logic pipe, because eight
// codes cost seven logic operations: (w >> 4i) & 0x000F000F | 0x43004300 is the bf16 PAIR {128 + q_i, 128 + q_(i+4)},
// and one packed subtract gives {q_i - 8, q_(i+4) - 8} exactly.  Those registers ARE the A fragments of
// mma.sync.m16n8k16 (bf16 in, f32 accumulate): 16 rows x 16 weights per instruction against up to 8 tokens' inputs
// (bf16-valued f32 activations convert exactly), whose order along K is permuted once, when they are staged in shared
// memory, to match the order the unpacking produces.  Per group: result += s * acc + (b + 8 s) * sum(x).
// A token's column of the MMA does not depend on the other columns, so its rows are the same bits for every T.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "seed_block.cuh"

namespace nsl {

constexpr int Q4_THREADS = 256, Q4_WARPS = Q4_THREADS / 32, Q4_GROUP = 64;

__device__ __forceinline__ void mma_bf16_16x8x16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One code word -> four bf16 pairs {q_i - 8, q_(i+4) - 8}, i = 0..3.  (w >> 4i) & mask | bias is ONE three-input logic
// operation when mask and bias are register (or constant-bank) operands; written with immediates the compiler emits an
// AND and an OR (the instruction takes one immediate), which doubled the logic-pipe work of the whole kernel.  The two
// words therefore live in constant memory, where the compiler cannot see their values.
static __constant__ uint32_t q4_nib_mask = 0x000F000Fu, q4_nib_bias = 0x43004300u;
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t* r) {
    const uint32_t mask = q4_nib_mask, bias = q4_nib_bias;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t v;      // {128 + q_i, 128 + q_(i+4)}
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(w >> (4 * i)), "r"(mask), "r"(bias));
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(r[i]) : "r"(v), "r"(0x43084308u));   // - 136
    }
}

// The first product of a group: the accumulator starts from zero (no registers to clear).
__device__ __forceinline__ void mma_bf16_16x8x16_first(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t) h << 16); }
__device__ __forceinline__ bool aligned16_dev(const void* p) { return ((unsigned long long) p & 15ull) == 0; }

// Shared memory: xb[g][q][n][8] u32 (the B fragments of group g's four MMAs for thread (n, q)), then xsum[g][8] f32.
__global__ void __launch_bounds__(Q4_THREADS) q4_mv_kernel(const uint32_t* __restrict__ codes, const uint16_t* __restrict__ S,
                                                          const uint16_t* __restrict__ B, int K, int R, const float* __restrict__ x,
                                                          int xs, float* __restrict__ y, int ys, int T, int add) {
    extern __shared__ __align__(16) uint32_t q4_smem[];
    const int G = K / Q4_GROUP;
    uint32_t* xb = q4_smem;
    float* xsum = (float*) (q4_smem + (size_t) G * 4 * 8 * 8);
    grid_dependents_go();
    grid_dependency_wait();
    // stage the inputs: thread (n, q) of group g gets x_n[64 g + 16 q + {m, m + 4}] and [.. + {8 + m, 12 + m}], m = 0..3;
    // one warp pass covers one group (32 threads = 4 q x 8 n), so the group's input sums are two shuffles away
    const bool vec = (xs & 3) == 0 && aligned16_dev(x);
    for (int i = threadIdx.x; i < G * 32; i += Q4_THREADS) {
        const int g = i >> 5, q = (i >> 3) & 3, n = i & 7;
        uint32_t* dst = xb + (size_t) i * 8;
        float v[16];
        if (n < T) {
            const float* xp = x + (size_t) n * xs + g * 64 + q * 16;
            if (vec) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 t = __ldg((const float4*) xp + j);
                    v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __ldg(xp + j);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
        }
        float part = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { v[j] = bf16_round(v[j]); part += v[j]; }
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            dst[2 * m] = bf16_bits(v[m]) | ((uint32_t) bf16_bits(v[m + 4]) << 16);
            dst[2 * m + 1] = bf16_bits(v[8 + m]) | ((uint32_t) bf16_bits(v[12 + m]) << 16);
        }
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 8);      // over q (lanes 8 apart)
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 16);
        if (q == 0) xsum[g * 8 + n] = part;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, q = lane & 3, rr = lane >> 2;
    const int tiles = (R + 15) / 16;
    for (int tile = blockIdx.x * Q4_WARPS + warp; tile < tiles; tile += gridDim.x * Q4_WARPS) {
        const int r0 = min(tile * 16 + rr, R - 1), r1 = min(tile * 16 + rr + 8, R - 1);     // clamped: stores are guarded
        const uint2* c0p = (const uint2*) (codes + (size_t) r0 * (K / 8)) + q;
        const uint2* c1p = (const uint2*) (codes + (size_t) r1 * (K / 8)) + q;
        float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint16_t* S0 = S + (size_t) r0 * G, *S1 = S + (size_t) r1 * G, *B0 = B + (size_t) r0 * G, *B1 = B + (size_t) r1 * G;
        auto group = [&](int g, uint2 w0, uint2 w1, float s0, float s1, float bb0, float bb1) {
            uint32_t a0[8], a1[8];
            unpack8(w0.x, a0); unpack8(w0.y, a0 + 4);
            unpack8(w1.x, a1); unpack8(w1.y, a1 + 4);
            const uint4 b01 = *(const uint4*) (xb + ((size_t) (g * 4 + q) * 8 + rr) * 8);
            const uint4 b23 = *(const uint4*) (xb + ((size_t) (g * 4 + q) * 8 + rr) * 8 + 4);
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint32_t f0[4] = {a0[0], a1[0], a0[4], a1[4]}, f1[4] = {a0[1], a1[1], a0[5], a1[5]};
            const uint32_t f2[4] = {a0[2], a1[2], a0[6], a1[6]}, f3[4] = {a0[3], a1[3], a0[7], a1[7]};
            mma_bf16_16x8x16(c, f0, b01.x, b01.y);
            mma_bf16_16x8x16(c, f1, b01.z, b01.w);
            mma_bf16_16x8x16(c, f2, b23.x, b23.y);
            mma_bf16_16x8x16(c, f3, b23.z, b23.w);
            const float e0 = fmaf(8.0f, s0, bb0), e1 = fmaf(8.0f, s1, bb1);
            const float2 xg = *(const float2*) (xsum + g * 8 + 2 * q);
            out[0] += fmaf(s0, c[0], e0 * xg.x);
            out[1] += fmaf(s0, c[1], e0 * xg.y);
            out[2] += fmaf(s1, c[2], e1 * xg.x);
            out[3] += fmaf(s1, c[3], e1 * xg.y);
        };
        int g = 0;
        if ((G & 7) == 0) {      // eight groups per pass: one 16-byte load of scales and of biases per row, 16 code loads in flight
            for (; g < G; g += 8) {
                const uint4 sv0 = __ldg((const uint4*) (S0 + g)), sv1 = __ldg((const uint4*) (S1 + g));
                const uint4 bv0 = __ldg((const uint4*) (B0 + g)), bv1 = __ldg((const uint4*) (B1 + g));
                uint2 w0[8], w1[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) { w0[j] = __ldg(c0p + 4 * (g + j)); w1[j] = __ldg(c1p + 4 * (g + j)); }
                const uint32_t sa0[4] = {sv0.x, sv0.y, sv0.z, sv0.w}, sa1[4] = {sv1.x, sv1.y, sv1.z, sv1.w};
                const uint32_t ba0[4] = {bv0.x, bv0.y, bv0.z, bv0.w}, ba1[4] = {bv1.x, bv1.y, bv1.z, bv1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int sh = (j & 1) * 16;
                    group(g + j, w0[j], w1[j], bf16_to_f32((uint16_t) (sa0[j >> 1] >> sh)), bf16_to_f32((uint16_t) (sa1[j >> 1] >> sh)),
                          bf16_to_f32((uint16_t) (ba0[j >> 1] >> sh)), bf16_to_f32((uint16_t) (ba1[j >> 1] >> sh)));
                }
            }
        }
        for (; g < G; ++g)
            group(g, __ldg(c0p + 4 * g), __ldg(c1p + 4 * g), bf16_to_f32(__ldg(S0 + g)), bf16_to_f32(__ldg(S1 + g)),
                  bf16_to_f32(__ldg(B0 + g)), bf16_to_f32(__ldg(B1 + g)));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = tile * 16 + rr + (i >> 1) * 8, t = 2 * q + (i & 1);
            if (row < R && t < T) {
                float* yo = y + (size_t) t * ys + row;
                *yo = add ? bf16_round(*yo + bf16_round(out[i])) : bf16_round(out[i]);
            }
        }
    }
}

// The same arithmetic with the streams prefetched through shared memory.  The plain kernel above is latency-bound (ncu:
// 5.5 long-scoreboard stalls per issued instruction at 27 % of the DRAM peak): its loads are only in flight while a warp
// waits for them.  Here every warp owns a ring of NST stages; a stage holds one PASS = eight groups of a 16-row tile:
// per row 256 bytes of codes, then the eight scales and the eight biases (16 + 16 bytes), 288 bytes in all, which also
// makes the 8-byte reads of a half warp conflict-free.  cp.async fills the stages NST - 1 passes ahead, no registers
// held, so a warp keeps (NST - 1) x 4.5 KB in flight while it computes.  K must be a multiple of 512.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((unsigned) __cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}

// GPP groups per pass (8 or 4).  A stage row: GPP * 32 bytes of codes, GPP scales, GPP biases, padded to a stride of
// 32 (mod 128) bytes so that the 8-byte reads of a half warp (four rows x four 8-byte pieces) touch distinct banks.
template <int GPP> struct Q4Ring {
    static constexpr int CODES = GPP * 32, ROW = CODES + 32, STAGE = 16 * ROW;      // 288 / 160 bytes per row
};

template <int NST, int WARPS, int GPP>
__global__ void __launch_bounds__(32 * WARPS, 1) q4_mv_ring_kernel(const uint32_t* __restrict__ codes, const uint16_t* __restrict__ S,
                                                                   const uint16_t* __restrict__ B, int K, int R,
                                                                   const float* __restrict__ x, int xs, float* __restrict__ y, int ys,
                                                                   int T, int add) {
    constexpr int ROW = Q4Ring<GPP>::ROW, STAGE = Q4Ring<GPP>::STAGE, CODES = Q4Ring<GPP>::CODES;
    extern __shared__ __align__(16) uint32_t q4_smem[];
    const int G = K / Q4_GROUP, PPT = G / GPP;      // passes per tile
    uint32_t* xb = q4_smem;
    float* xsum = (float*) (q4_smem + (size_t) G * 256);
    unsigned char* ring = (unsigned char*) (xsum + G * 8) + (size_t) (threadIdx.x >> 5) * NST * STAGE;
    grid_dependents_go();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, q = lane & 3, rr = lane >> 2;
    const int tiles = (R + 15) / 16;
    const int tile0 = blockIdx.x * WARPS + warp, tstride = gridDim.x * WARPS;
    const int my_tiles = tile0 < tiles ? (tiles - tile0 + tstride - 1) / tstride : 0;
    const int my_passes = my_tiles * PPT;

    auto issue = [&](int idx) {
        if (idx < my_passes) {
            const int tile = tile0 + (idx / PPT) * tstride, p = idx % PPT;
            unsigned char* st = ring + (size_t) (idx % NST) * STAGE;
            constexpr int PIECES = CODES / 16, RPI = 32 / PIECES;      // 16-byte pieces per row; rows per warp instruction
#pragma unroll
            for (int i = 0; i < 16 / RPI; ++i) {
                const int lr = RPI * i + lane / PIECES, piece = lane % PIECES, row = min(tile * 16 + lr, R - 1);
                cp_async16(st + lr * ROW + piece * 16, (const unsigned char*) (codes + (size_t) row * (K / 8) + p * (GPP * 8)) + piece * 16);
            }
            const int lr = lane & 15, row = min(tile * 16 + lr, R - 1);
            const uint16_t* src = (lane >> 4 ? B : S) + (size_t) row * G + p * GPP;
            if (GPP == 8) cp_async16(st + lr * ROW + CODES + (lane >> 4) * 16, src);
            else cp_async8(st + lr * ROW + CODES + (lane >> 4) * 8, src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int i = 0; i < NST - 1; ++i) issue(i);      // the streams start before the inputs are staged

    const bool vec = (xs & 3) == 0 && aligned16_dev(x);
    for (int i = threadIdx.x; i < G * 32; i += 32 * WARPS) {
        const int g = i >> 5, sq = (i >> 3) & 3, n = i & 7;
        uint32_t* dst = xb + (size_t) i * 8;
        float v[16];
        if (n < T) {
            const float* xp = x + (size_t) n * xs + g * 64 + sq * 16;
            if (vec) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 t = __ldg((const float4*) xp + j);
                    v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __ldg(xp + j);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
        }
        float part = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { v[j] = bf16_round(v[j]); part += v[j]; }
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            dst[2 * m] = bf16_bits(v[m]) | ((uint32_t) bf16_bits(v[m + 4]) << 16);
            dst[2 * m + 1] = bf16_bits(v[8 + m]) | ((uint32_t) bf16_bits(v[12 + m]) << 16);
        }
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 8);
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 16);
        if (sq == 0) xsum[g * 8 + n] = part;
    }
    __syncthreads();

    float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int idx = 0; idx < my_passes; ++idx) {
        asm volatile("cp.async.wait_group %0;" ::"n"(NST - 2) : "memory");
        __syncwarp();      // every lane's pieces of this stage have landed
        const int tile = tile0 + (idx / PPT) * tstride, p = idx % PPT;
        const unsigned char* st = ring + (size_t) (idx % NST) * STAGE;
        const unsigned char* row0 = st + rr * ROW, *row1 = st + (rr + 8) * ROW;
        // the pass's scales and biases of both rows: GPP bf16 each, two per word
        uint32_t sa0[GPP / 2], sa1[GPP / 2], ba0[GPP / 2], ba1[GPP / 2];
        if (GPP == 8) {
            const uint4 t0 = *(const uint4*) (row0 + CODES), t1 = *(const uint4*) (row0 + CODES + 16);
            const uint4 t2 = *(const uint4*) (row1 + CODES), t3 = *(const uint4*) (row1 + CODES + 16);
            sa0[0] = t0.x; sa0[1] = t0.y; sa0[GPP / 2 - 2] = t0.z; sa0[GPP / 2 - 1] = t0.w;
            ba0[0] = t1.x; ba0[1] = t1.y; ba0[GPP / 2 - 2] = t1.z; ba0[GPP / 2 - 1] = t1.w;
            sa1[0] = t2.x; sa1[1] = t2.y; sa1[GPP / 2 - 2] = t2.z; sa1[GPP / 2 - 1] = t2.w;
            ba1[0] = t3.x; ba1[1] = t3.y; ba1[GPP / 2 - 2] = t3.z; ba1[GPP / 2 - 1] = t3.w;
        } else {
            const uint4 t0 = *(const uint4*) (row0 + CODES), t2 = *(const uint4*) (row1 + CODES);      // {scales, biases}
            sa0[0] = t0.x; sa0[1] = t0.y; ba0[0] = t0.z; ba0[1] = t0.w;
            sa1[0] = t2.x; sa1[1] = t2.y; ba1[0] = t2.z; ba1[1] = t2.w;
        }
#pragma unroll
        for (int j = 0; j < GPP; ++j) {
            const int g = p * GPP + j, sh = (j & 1) * 16;
            const uint2 w0 = *(const uint2*) (row0 + j * 32 + q * 8), w1 = *(const uint2*) (row1 + j * 32 + q * 8);
            uint32_t a0[8], a1[8];
            unpack8(w0.x, a0); unpack8(w0.y, a0 + 4);
            unpack8(w1.x, a1); unpack8(w1.y, a1 + 4);
            const uint4 b01 = *(const uint4*) (xb + ((size_t) (g * 4 + q) * 8 + rr) * 8);
            const uint4 b23 = *(const uint4*) (xb + ((size_t) (g * 4 + q) * 8 + rr) * 8 + 4);
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint32_t f0[4] = {a0[0], a1[0], a0[4], a1[4]}, f1[4] = {a0[1], a1[1], a0[5], a1[5]};
            const uint32_t f2[4] = {a0[2], a1[2], a0[6], a1[6]}, f3[4] = {a0[3], a1[3], a0[7], a1[7]};
            mma_bf16_16x8x16(c, f0, b01.x, b01.y);
            mma_bf16_16x8x16(c, f1, b01.z, b01.w);
            mma_bf16_16x8x16(c, f2, b23.x, b23.y);
            mma_bf16_16x8x16(c, f3, b23.z, b23.w);
            const float s0 = bf16_to_f32((uint16_t) (sa0[j >> 1] >> sh)), s1 = bf16_to_f32((uint16_t) (sa1[j >> 1] >> sh));
            const float e0 = fmaf(8.0f, s0, bf16_to_f32((uint16_t) (ba0[j >> 1] >> sh)));
            const float e1 = fmaf(8.0f, s1, bf16_to_f32((uint16_t) (ba1[j >> 1] >> sh)));
            const float2 xg = *(const float2*) (xsum + g * 8 + 2 * q);
            out[0] += fmaf(s0, c[0], e0 * xg.x);
            out[1] += fmaf(s0, c[1], e0 * xg.y);
            out[2] += fmaf(s1, c[2], e1 * xg.x);
            out[3] += fmaf(s1, c[3], e1 * xg.y);
        }
        __syncwarp();      // a stage read one pass ago is refilled NST - 1 passes ahead
        issue(idx + NST - 1);
        if (p == PPT - 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = tile * 16 + rr + (i >> 1) * 8, t = 2 * q + (i & 1);
                if (row < R && t < T) {
                    float* yo = y + (size_t) t * ys + row;
                    *yo = add ? bf16_round(*yo + bf16_round(out[i])) : bf16_round(out[i]);
                }
                out[i] = 0.0f;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// The ring kernel is bound by the shared-memory pipe (ncu: l1tex 87 % busy, DRAM 34 %): per 16-row tile it moves 72 KB
// through shared memory, 32 KB of it the inputs' MMA fragments that every warp re-reads for every tile.  Here the K
// dimension is split over the block's warps instead: warp w owns groups 4 w .. 4 w + 3 for EVERY tile of its block,
// so its 32 fragment registers and 8 input sums are loaded once and stay in registers; per tile a warp streams
// 16 rows x 128 bytes of codes (+ 8 scales, 8 biases per row) through its cp.async ring, runs 16 MMAs, and the warps'
// partial sums meet in shared memory (8 KB per tile), where they are added in warp order.  K = 256 x WARPS.
// BPS blocks share an SM (16 warps in all): a block's barrier per tile then overlaps another block's work.  Shared
// memory: the partial sums, then the staged inputs, whose place the rings take once every warp holds its fragments.
template <int WARPS, int NST, int BPS>
__global__ void __launch_bounds__(32 * WARPS, BPS) q4_mv_ksplit_kernel(const uint32_t* __restrict__ codes, const uint16_t* __restrict__ S,
                                                                     const uint16_t* __restrict__ B, int K, int R,
                                                                     const float* __restrict__ x, int xs, float* __restrict__ y,
                                                                     int ys, int T, int add) {
    constexpr int ROW = Q4Ring<4>::ROW, STAGE = Q4Ring<4>::STAGE;
    constexpr int G = 4 * WARPS, KB = 128 * WARPS;      // groups and bytes of codes per row (K = 256 x WARPS)
    extern __shared__ __align__(16) uint32_t q4_smem[];
    float* part = (float*) q4_smem;                                              // [2][WARPS][32][4]
    uint32_t* xb = q4_smem + 2 * WARPS * 128;
    float* xsum = (float*) (xb + (size_t) G * 256);
    // the rings take the place of the staged inputs once those sit in the warps' registers
    unsigned char* ring = (unsigned char*) xb + (size_t) (threadIdx.x >> 5) * NST * STAGE;
    grid_dependents_go();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, q = lane & 3, rr = lane >> 2;
    const int tiles = (R + 15) / 16;
    const int my_tiles = (int) blockIdx.x < tiles ? (tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x : 0;

    // the copies of the next tile to fetch: running source pointers (a tile further = gridDim.x x 16 rows) and stage
    int nidx = 0, nstage = 0, ntile = blockIdx.x;
    const unsigned char* csrc = (const unsigned char*) codes + ((size_t) blockIdx.x * 16 + (lane >> 3)) * KB + warp * 128 + (lane & 7) * 16;
    const uint16_t* ssrc = (lane >> 4 ? B : S) + ((size_t) blockIdx.x * 16 + (lane & 15)) * G + warp * 4;
    const size_t cstep = (size_t) gridDim.x * 16 * KB, sstep = (size_t) gridDim.x * 16 * G;
    const unsigned cdst = (unsigned) __cvta_generic_to_shared(ring) + (lane >> 3) * ROW + (lane & 7) * 16;
    const unsigned sdst = (unsigned) __cvta_generic_to_shared(ring) + (lane & 15) * ROW + 128 + (lane >> 4) * 8;
    auto issue = [&]() {      // this warp's 128-byte slice of the 16 rows of its block's next tile
        if (nidx < my_tiles) {
            const unsigned so = (unsigned) nstage * STAGE;
            if (ntile * 16 + 16 <= R) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(cdst + so + i * 4 * ROW), "l"(csrc + (size_t) i * 4 * KB) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(sdst + so), "l"(ssrc) : "memory");
            } else {      // the last, partial tile: rows beyond R - 1 read row R - 1 (their results are not stored)
                unsigned char* st = ring + so;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int lr = 4 * i + (lane >> 3), piece = lane & 7, row = min(ntile * 16 + lr, R - 1);
                    cp_async16(st + lr * ROW + piece * 16, (const unsigned char*) codes + (size_t) row * KB + warp * 128 + piece * 16);
                }
                const int lr = lane & 15, row = min(ntile * 16 + lr, R - 1);
                cp_async8(st + lr * ROW + 128 + (lane >> 4) * 8, (lane >> 4 ? B : S) + (size_t) row * G + warp * 4);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        ++nidx;
        ntile += gridDim.x;
        csrc += cstep;
        ssrc += sstep;
        nstage = nstage + 1 == NST ? 0 : nstage + 1;
    };
    const bool vec = (xs & 3) == 0 && aligned16_dev(x);
    for (int i = threadIdx.x; i < G * 32; i += 32 * WARPS) {
        const int g = i >> 5, sq = (i >> 3) & 3, n = i & 7;
        uint32_t* dst = xb + (size_t) i * 8;
        float v[16];
        if (n < T) {
            const float* xp = x + (size_t) n * xs + g * 64 + sq * 16;
            if (vec) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 t = __ldg((const float4*) xp + j);
                    v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __ldg(xp + j);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
        }
        float psum = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { v[j] = bf16_round(v[j]); psum += v[j]; }
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            dst[2 * m] = bf16_bits(v[m]) | ((uint32_t) bf16_bits(v[m + 4]) << 16);
            dst[2 * m + 1] = bf16_bits(v[8 + m]) | ((uint32_t) bf16_bits(v[12 + m]) << 16);
        }
        psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 8);
        psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 16);
        if (sq == 0) xsum[g * 8 + n] = psum;
    }
    __syncthreads();
    // this warp's four groups of inputs: fragments and sums, in registers for the whole kernel
    uint32_t breg[4][8];
    float xg[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int g = warp * 4 + j;
        const uint4 lo = *(const uint4*) (xb + ((size_t) (g * 4 + q) * 8 + rr) * 8), hi = *(const uint4*) (xb + ((size_t) (g * 4 + q) * 8 + rr) * 8 + 4);
        breg[j][0] = lo.x; breg[j][1] = lo.y; breg[j][2] = lo.z; breg[j][3] = lo.w;
        breg[j][4] = hi.x; breg[j][5] = hi.y; breg[j][6] = hi.z; breg[j][7] = hi.w;
        xg[j][0] = xsum[g * 8 + 2 * q];
        xg[j][1] = xsum[g * 8 + 2 * q + 1];
    }
    __syncthreads();      // every warp has its inputs: their place is the rings' now
#pragma unroll
    for (int i = 0; i < NST - 1; ++i) issue();

    int stage = 0;
    for (int idx = 0; idx < my_tiles; ++idx) {
        asm volatile("cp.async.wait_group %0;" ::"n"(NST - 2) : "memory");
        __syncwarp();
        const int tile = blockIdx.x + idx * gridDim.x;
        const unsigned char* st = ring + (size_t) stage * STAGE;
        stage = stage + 1 == NST ? 0 : stage + 1;
        const unsigned char* row0 = st + rr * ROW, *row1 = st + (rr + 8) * ROW;
        const uint4 t0 = *(const uint4*) (row0 + 128), t2 = *(const uint4*) (row1 + 128);      // {4 scales, 4 biases}
        const uint32_t sa0[2] = {t0.x, t0.y}, ba0[2] = {t0.z, t0.w}, sa1[2] = {t2.x, t2.y}, ba1[2] = {t2.z, t2.w};
        float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int sh = (j & 1) * 16;
            const uint2 w0 = *(const uint2*) (row0 + j * 32 + q * 8), w1 = *(const uint2*) (row1 + j * 32 + q * 8);
            uint32_t a0[8], a1[8];
            unpack8(w0.x, a0); unpack8(w0.y, a0 + 4);
            unpack8(w1.x, a1); unpack8(w1.y, a1 + 4);
            float c[4];
            const uint32_t f0[4] = {a0[0], a1[0], a0[4], a1[4]}, f1[4] = {a0[1], a1[1], a0[5], a1[5]};
            const uint32_t f2[4] = {a0[2], a1[2], a0[6], a1[6]}, f3[4] = {a0[3], a1[3], a0[7], a1[7]};
            mma_bf16_16x8x16_first(c, f0, breg[j][0], breg[j][1]);
            mma_bf16_16x8x16(c, f1, breg[j][2], breg[j][3]);
            mma_bf16_16x8x16(c, f2, breg[j][4], breg[j][5]);
            mma_bf16_16x8x16(c, f3, breg[j][6], breg[j][7]);
            const float s0 = bf16_to_f32((uint16_t) (sa0[j >> 1] >> sh)), s1 = bf16_to_f32((uint16_t) (sa1[j >> 1] >> sh));
            const float e0 = fmaf(8.0f, s0, bf16_to_f32((uint16_t) (ba0[j >> 1] >> sh)));
            const float e1 = fmaf(8.0f, s1, bf16_to_f32((uint16_t) (ba1[j >> 1] >> sh)));
            out[0] = fmaf(s0, c[0], fmaf(e0, xg[j][0], out[0]));
            out[1] = fmaf(s0, c[1], fmaf(e0, xg[j][1], out[1]));
            out[2] = fmaf(s1, c[2], fmaf(e1, xg[j][0], out[2]));
            out[3] = fmaf(s1, c[3], fmaf(e1, xg[j][1], out[3]));
        }
        __syncwarp();
        issue();
        float* pb = part + (size_t) (idx & 1) * WARPS * 128;
        *(float4*) (pb + (warp * 32 + lane) * 4) = make_float4(out[0], out[1], out[2], out[3]);
        __syncthreads();      // the block's partial sums of this tile are in; the other buffer is free for the next tile
        // the tile's 128 outputs (32 lane slots x 4) are shared out over the warps; each is the warps' sum in warp order
        for (int e = warp * 32 + lane; e < 128; e += 32 * WARPS) {
            float acc = pb[e];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) acc += pb[w * 128 + e];
            const int sl = e >> 2, i = e & 3;      // the lane slot (rr, q) and its output i
            const int row = tile * 16 + (sl >> 2) + (i >> 1) * 8, t = 2 * (sl & 3) + (i & 1);
            if (row < R && t < T) {
                float* yo = y + (size_t) t * ys + row;
                *yo = add ? bf16_round(*yo + bf16_round(acc)) : bf16_round(acc);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int WARPS, int NST, int BPS>
static void launch_q4_ksplit(cudaStream_t s, size_t total, int blocks, const WSlice& w, int K, int R, const float* x, int xs, float* y,
                             int ys, int T, int add) {
    static bool attr_set[16];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 15]) {
        cudaFuncSetAttribute(q4_mv_ksplit_kernel<WARPS, NST, BPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin() - 1024);
        attr_set[dev & 15] = true;
    }
    launch(q4_mv_ksplit_kernel<WARPS, NST, BPS>, (unsigned) blocks, 32 * WARPS, total, s, (const uint32_t*) w.p[0], (const uint16_t*) w.p[1],
           (const uint16_t*) w.p[2], K, R, x, xs, y, ys, T, add);
}

template <int NST, int WARPS, int GPP>
static void launch_q4_ring(cudaStream_t s, size_t total, int blocks, const WSlice& w, int K, int R, const float* x, int xs, float* y,
                           int ys, int T, int add) {
    static bool attr_set[16];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 15]) {
        cudaFuncSetAttribute(q4_mv_ring_kernel<NST, WARPS, GPP>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin() - 1024);
        attr_set[dev & 15] = true;
    }
    launch(q4_mv_ring_kernel<NST, WARPS, GPP>, (unsigned) blocks, 32 * WARPS, total, s, (const uint32_t*) w.p[0],
           (const uint16_t*) w.p[1], (const uint16_t*) w.p[2], K, R, x, xs, y, ys, T, add);
}

// Greedy arg-max of each row (ties: the lowest id) and, optionally, its softmax probability 1 / sum exp(l - max).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, float* __restrict__ prob,
                                                      int V) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const float* l = logits + (size_t) blockIdx.x * V;
    float best = -INFINITY;
    int idx = 0x7FFFFFFF;
    for (int i = tid; i < V; i += 1024) {
        const float v = l[i];
        if (v > best) { best = v; idx = i; }      // ascending i: the first of equal values stays
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float b2 = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int i2 = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
        if (b2 > best || (b2 == best && i2 < idx)) { best = b2; idx = i2; }
    }
    if (lane == 0) { bv[w] = best; bi[w] = idx; }
    __syncthreads();
    if (w == 0) {
        best = bv[lane]; idx = bi[lane];
        for (int o = 16; o > 0; o >>= 1) {
            const float b2 = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int i2 = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
            if (b2 > best || (b2 == best && i2 < idx)) { best = b2; idx = i2; }
        }
        if (lane == 0) { out[blockIdx.x] = idx == 0x7FFFFFFF ? 0 : idx; bv[0] = best; }
    }
    if (!prob) return;
    __syncthreads();
    const float mx = bv[0];
    float s = 0.0f;
    for (int i = tid; i < V; i += 1024) s += expf(l[i] - mx);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    __syncthreads();      // every thread has read bv[0]
    if (lane == 0) bv[w] = s;
    __syncthreads();
    if (tid == 0) {
        float tot = 0.0f;
        for (int i = 0; i < 32; ++i) tot += bv[i];
        prob[blockIdx.x] = 1.0f / tot;
    }
}

// Called by kc_mv for fmt == MF_Q4.  Returns false (with the error recorded) when the shape is not served.
bool launch_q4_mv(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add) {
    if (K < Q4_GROUP || K % Q4_GROUP || R < 1 || T < 1 || T > MV_MAXT || (w.gs != 0 && w.gs != 6)) {
        set_error("kc_mv (Q4): K = %d must be a multiple of 64, 1..%d tokens, groups of 64 (gs %d)", K, (int) MV_MAXT, w.gs);
        return false;
    }
    if (((uintptr_t) w.p[0] & 7u) || !aligned16(w.p[1]) || !aligned16(w.p[2])) {
        set_error("kc_mv (Q4): codes must be 8-byte aligned, scales and biases 16-byte aligned");
        return false;
    }
    const size_t smem = (size_t) (K / Q4_GROUP) * (4 * 8 * 8 * 4 + 8 * 4);
    const int tiles = (R + 15) / 16;
    static bool attr_set[16];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 15]) {
        cudaFuncSetAttribute(q4_mv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin() - 1024);
        attr_set[dev & 15] = true;
    }
    const size_t budget = (size_t) max_smem_optin() - 1024;
    if (aligned16(w.p[0]) && (K == 1024 || K == 2048 || K == 4096)) {      // K split over the block's warps
        // 16 warps an SM in blocks of K / 256 warps, four stages per warp in the place of the staged inputs: with two
        // blocks an SM one block's barrier per tile overlaps the other's work (151936 x 2048: 51.9 us with one block of
        // 8 warps and 6 stages, 49.2 us with two blocks of 4 stages)
        const int warps = K / 256, bps = 16 / warps;
        const size_t rings = (size_t) warps * 4 * Q4Ring<4>::STAGE;
        const size_t total = (size_t) 2 * warps * 512 + (rings > smem ? rings : smem);
        const int blocks = tiles < bps * sm_count() ? tiles : bps * sm_count();
        if (warps == 4) launch_q4_ksplit<4, 4, 4>(s, total, blocks, w, K, R, x, xs, y, ys, T, add);
        else if (warps == 8) launch_q4_ksplit<8, 4, 2>(s, total, blocks, w, K, R, x, xs, y, ys, T, add);
        else launch_q4_ksplit<16, 4, 1>(s, total, blocks, w, K, R, x, xs, y, ys, T, add);
        count_launch();
        return true;
    }
    if (K % 512 == 0 && aligned16(w.p[0]) && smem + (size_t) 8 * 2 * Q4Ring<8>::STAGE <= budget) {      // streams through shared memory
        // 8 warps with three passes of eight groups in flight each (measured faster than 16 warps with three passes of four:
        // 66.9 against 77.2 us on the 151936 x 2048 head), or 8 warps with one pass in flight when shared memory is short
        const bool deep = smem + (size_t) 8 * 4 * Q4Ring<8>::STAGE <= budget;
        int blocks = (tiles + 7) / 8;
        if (blocks > sm_count()) blocks = sm_count();
        if (deep) launch_q4_ring<4, 8, 8>(s, smem + (size_t) 8 * 4 * Q4Ring<8>::STAGE, blocks, w, K, R, x, xs, y, ys, T, add);
        else launch_q4_ring<2, 8, 8>(s, smem + (size_t) 8 * 2 * Q4Ring<8>::STAGE, blocks, w, K, R, x, xs, y, ys, T, add);
        count_launch();
        return true;
    }
    if (smem > budget) {
        set_error("kc_mv (Q4): K = %d does not fit the inputs of 8 tokens in shared memory", K);
        return false;
    }
    const int per_sm = smem > 100 * 1024 ? 1 : 2;      // 106 registers: two blocks of 8 warps per SM
    int blocks = (tiles + Q4_WARPS - 1) / Q4_WARPS;
    if (blocks > sm_count() * per_sm) blocks = sm_count() * per_sm;
    launch(q4_mv_kernel, (unsigned) blocks, Q4_THREADS, smem, s, (const uint32_t*) w.p[0], (const uint16_t*) w.p[1],
           (const uint16_t*) w.p[2], K, R, x, xs, y, ys, T, add);
    count_launch();
    return true;
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void kc_argmax_p(cudaStream_t s, const float* logits, int32_t* out, float* prob, int V, int n) {
    if (V < 1 || n < 1) return;
    argmax_kernel<<<(unsigned) n, 1024, 0, s>>>(logits, out, prob, V);
    count_launch();
}

void kc_argmax(cudaStream_t s, const float* logits, int32_t* out, int V, int n) { kc_argmax_p(s, logits, out, NULL, V, n); }

}   // extern "C"
