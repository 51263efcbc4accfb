// Dense products over stored BF16 weights.  First the mat-vec for shapes the tensor-core kernel below does not take (K not a
// multiple of 256; kc_mv with MF_BF16; engine/kernels_moe.cu:92, 596: y[t][r] = bf16(W[r] . x[t]), f32
// sums, optional residual add as store_y).  A warp owns a row at a time and reads it as 16-byte
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

// ---- 1..64 rows of inputs on the tensor cores ---------------------------------------------------------------------
// kc_mv and kc_mm with MF_BF16 for a decode batch (engine/qwen4_cuda.c: mv()): at 8 rows a 2048 x 2048 product takes 6 us here
// against 34 us for the warp-per-row kernel above, whose 16 input loads per weight load bind it to the load-store pipe.  A block owns 16 weight rows and
// 8 tokens; its 8 warps split K and each runs mma.sync.m16n8k16 (bf16 in, f32 accumulate) over its range with the 8
// tokens as the columns.  The weights are not staged: a lane's 16-byte load of a weight row IS its A fragments of two
// MMAs, because the products' k index is free to be permuted as long as the B fragments use the same permutation: lane
// (g, t) loads weights k0 + 8 t .. + 7 of rows g and g + 8, and reads the same 8 inputs of token g; MMA 1 takes elements
// 0-3, MMA 2 elements 4-7.  The block's 8 input rows are staged once in shared memory as bf16 (exact: the inputs are
// bf16-valued f32, engine/kernels_moe.cu:1-3; row stride K * 2 + 64 bytes, so the 8 lanes of a quarter warp read 128
// consecutive bytes).  Everything a thread reads from global memory -- its weights of up to 8 steps and its share of the
// inputs -- is requested before anything is used: one memory latency per block, not one per step (a version that loaded
// step by step took 15.5 us per 2048 x 2048 product at 32 tokens, whatever the grid).  The warps' partial sums meet in
// shared memory and are added in warp order; a token's result does not depend on the other tokens of the call.
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256) bf16_mm_skinny_kernel(const uint16_t* __restrict__ W, int K, int R, const float* __restrict__ x, int xs,
                                                             float* __restrict__ y, int ys, int T, int add) {
    extern __shared__ __align__(16) unsigned char xsm[];      // 8 rows of K bf16 inputs
    __shared__ float part[8][16][9];
    grid_dependents_go();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t4 = lane & 3;
    const int r0 = blockIdx.x * 16, tok0 = blockIdx.y * 8;
    const uint16_t* wa = W + (size_t) min(r0 + g, R - 1) * K + 8 * t4;
    const uint16_t* wb = W + (size_t) min(r0 + g + 8, R - 1) * K + 8 * t4;
    const int kw = K / 8, k0 = warp * kw, stride = K * 2 + 64;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int kb = k0; kb < k0 + kw; kb += 256) {
        const int ns = min(8, (k0 + kw - kb) / 32);
        uint4 a[8], b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < ns) { a[i] = __ldg((const uint4*) (wa + kb + 32 * i)); b[i] = __ldg((const uint4*) (wb + kb + 32 * i)); }      // weights never change
        if (kb == k0) {      // the inputs, once: they may come from the previous kernel in the stream
            grid_dependency_wait();
            const int kc8 = K / 8;
#pragma unroll 8
            for (int c = threadIdx.x; c < 8 * kc8; c += 256) {
                const int n = c / kc8, kc = c - n * kc8;
                const float4* xp = (const float4*) (x + (size_t) min(tok0 + n, T - 1) * xs + 8 * kc);
                const float4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                *(uint4*) (xsm + (size_t) n * stride + 16 * kc) =
                    make_uint4(bf16x2_bits(x0.x, x0.y), bf16x2_bits(x0.z, x0.w), bf16x2_bits(x1.x, x1.y), bf16x2_bits(x1.z, x1.w));
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < ns) {
                const uint4 xq = *(const uint4*) (xsm + (size_t) g * stride + 2 * (kb + 32 * i + 8 * t4));
                mma_bf16_16816(acc, a[i].x, b[i].x, a[i].y, b[i].y, xq.x, xq.y);
                mma_bf16_16816(acc, a[i].z, b[i].z, a[i].w, b[i].w, xq.z, xq.w);
            }
        }
    }
    part[warp][g][2 * t4] = acc[0];
    part[warp][g][2 * t4 + 1] = acc[1];
    part[warp][g + 8][2 * t4] = acc[2];
    part[warp][g + 8][2 * t4 + 1] = acc[3];
    __syncthreads();
    if (threadIdx.x < 128) {
        const int row = threadIdx.x & 15, col = threadIdx.x >> 4;
        if (r0 + row < R && tok0 + col < T) {
            float s = part[0][row][col];
#pragma unroll
            for (int w = 1; w < 8; ++w) s += part[w][row][col];
            float* yo = y + (size_t) (tok0 + col) * ys + r0 + row;
            *yo = add ? bf16_round(*yo + bf16_round(s)) : bf16_round(s);      // engine/kernels_moe.cu:214
        }
    }
}

// Serves kc_mm for stored BF16 weights when the batch is a decode batch; false: the caller runs the tile GEMM.
bool launch_bf16_mm_skinny(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add) {
    const size_t smem = 8 * ((size_t) K * 2 + 64);
    if (T < 1 || T > 64 || K < 256 || K % 256 || R < 1 || smem > 160 * 1024 || !aligned16(w.p[0]) || !aligned16(x) || xs % 4) return false;
    static bool done[16];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!done[dev & 15]) {
        cudaFuncSetAttribute(bf16_mm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        done[dev & 15] = true;
    }
    launch(bf16_mm_skinny_kernel, dim3((unsigned) ((R + 15) / 16), (unsigned) ((T + 7) / 8)), 256, smem, s, (const uint16_t*) w.p[0], K, R, x, xs, y, ys,
           T, add);
    count_launch();
    return true;
}

}   // namespace nsl
