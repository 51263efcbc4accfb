// Prompt-row GEMM over seed weights on the 5th-generation tensor cores (tcgen05 + TMEM), dense and grouped by expert.
// Replaces the SEED4P4 paths of the reference's k_mm / k_mm3 / k_mm_packed and their grouped forms
// (engine/kernels_moe.cu:405-525, 2354-2395), which stage one 64 x 32 weight tile per K step for mma.sync.
//
// Y[n][r] = sum_k W[r][k] X[n][k] for a tile of 128 weight rows x up to 128 tokens (one entry of the tile table: one
// expert's run of pairs, or 128 consecutive tokens of a dense call).
//
// One block = 8 producer warps + 1 MMA warp.  Per K step of 64 the producers regenerate the 128 x 64 weight tile from
// its seeds (one 8-weight block per 16-byte row chunk, written bf16 in the 128-byte swizzled K-major layout the MMA
// reads) and convert the tokens' inputs to the same layout; one elected thread issues tcgen05.mma (M 128, N = the
// tile's pair count rounded up to 16, K 16, bf16 x bf16 -> f32 in TMEM) and commits the stage back to the producers
// through an mbarrier.  Three stages of shared memory overlap the expansion of step k+1, k+2 with the MMAs of step k.
// The expansion is the cost (about a hundred integer/FP operations per 8 weights against 2 x 8 x N flops of tensor
// work), so a weight tile is expanded once per tile entry and serves all of its tokens; the tensor pipe idles most of
// the time by construction.  The accumulator is read back with tcgen05.ld by the producer warps (TMEM lane = weight
// row, column = token), rounded as the reference's store_y does and written so that a warp stores 32 consecutive rows
// of one token.
//
// Weight precision: default, seed weights rounded to bf16 (one term); kc_seed_gemm_f32(1), three bf16 terms whose sum is
// the f32 weight exactly (three MMAs per step), as the reference's two modes (engine/kernels_moe.cu:405-412).
//
// Every wait on an mbarrier is bounded: after the limit the block records a status word, stops issuing work, frees its
// TMEM and returns.
#include "common.cuh"
#include "seed_block.cuh"

namespace nsl {

constexpr int GM_BM = 128, GM_BN = 128, GM_BK = 64, GM_STAGES = 3;
constexpr int GM_PRODUCERS = 256, GM_THREADS = GM_PRODUCERS + 32;
constexpr int GM_TILE_BYTES = GM_BM * GM_BK * 2;   // 16 KB: one bf16 operand tile
constexpr uint32_t GM_WAIT_LIMIT = 1u << 22;

struct MmParams {
    const WSlice* ws;        // grouped: device table; dense: NULL
    WSlice w0;
    const void* X;           // f32, or packed bf16
    float* Y;
    const int32_t* perm;
    const MmTile* tiles;
    const int32_t* ntiles;   // device tile count, or NULL
    const uint32_t* G;
    int* status;             // device status word (0 = ok)
    int K, R, T, xs, ys, xdiv, add, grouped, packed;
};

__device__ int g_mm_status;   // 0, or the code of the first bounded wait that ran out

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false after GM_WAIT_LIMIT polls (the caller records the code and stops).  Polling on purpose: the suspended
// form (mbarrier.try_wait) saved the polls' instructions but cost 3 us per 174 us launch in wake-up latency; short sleeps
// between a waiting producer's polls measured the same as bare polls (158.2 -> 157.5 us) and are kept for the issue slots.
// EAGER: false for the producers' wait for a free stage: a producer that is ahead sleeps between polls from the first
// miss on, so that its polls do not take issue slots from the warps the stage is waiting for.
template <bool EAGER = true>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < GM_WAIT_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (!EAGER) __nanosleep(i < 8 ? 48 : 96);
        if ((i & 15u) == 15u && *abort_flag) return false;
        if (EAGER && i > 64) __nanosleep(64);
    }
    return false;
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    // K-major operand tile, 128-byte swizzle: start address >> 4; leading byte offset (unused with swizzle) 1;
    // stride byte offset 1024 (8 rows of 128 bytes) >> 4; descriptor version 1; layout type 2 = SWIZZLE_128B
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | ((uint64_t) 1 << 16) | ((uint64_t) (1024 >> 4) << 32) | ((uint64_t) 1 << 46) |
           ((uint64_t) 2 << 61);
}
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    // D f32 (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (GM_BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// A thread's share of one K step: 4 consecutive blocks of its row = two block pairs (seed / coefficient words packed
// two per 32-bit word, even block low) and their 4 exponent codes (one nibble each, block j at bits 4j).  P = 3 (SEED4)
// has no code stream: a block's code is the low nibble of its nibble word, read where the weights are formed.
struct QuadIn { uint32_t sw[2], cw[2], codes; bool live; };

template <bool P3>
__device__ __forceinline__ QuadIn load_quad(const WSlice& w, int row, int kb, int R, int NB, bool vec) {
    QuadIn q = {{0u, 0u}, {0u, 0u}, 0u, false};
    if (row >= R || kb >= NB) return q;
    q.live = true;
    const size_t g = (size_t) row * NB + kb;
    if (vec) {   // NB % 4 == 0: the four blocks are one aligned 8-byte load per stream and two code bytes
        const uint2 s2 = __ldg((const uint2*) ((const uint16_t*) w.p[0] + g));
        const uint2 c2 = __ldg((const uint2*) ((const uint16_t*) w.p[1] + g));
        q.sw[0] = s2.x; q.sw[1] = s2.y; q.cw[0] = c2.x; q.cw[1] = c2.y;
        if (!P3) q.codes = __ldg((const uint16_t*) ((const uint8_t*) w.p[3] + (g >> 1)));
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (kb + j >= NB) break;   // (a missing block keeps seed 0: its weights are forced to zero below)
            const uint32_t sd = __ldg((const uint16_t*) w.p[0] + g + j), cf = __ldg((const uint16_t*) w.p[1] + g + j);
            const uint32_t cd = P3 ? 0u : (__ldg((const uint8_t*) w.p[3] + ((g + j) >> 1)) >> (((g + j) & 1) * 4)) & 15u;
            q.sw[j >> 1] |= sd << (16 * (j & 1));
            q.cw[j >> 1] |= cf << (16 * (j & 1));
            q.codes |= cd << (4 * j);
        }
    }
    return q;
}

// WF: the weights' form.  0: SEED4P4 blocks; 1: stored BF16 values; 2: SEED4 (P = 3) blocks.
// VEC: rows are whole quads of blocks (K a multiple of 32), so a thread's four blocks are one aligned load per stream and no
// row ends inside a quad.
template <int NT, int WF, bool VEC>
__global__ void __launch_bounds__(GM_THREADS, 2) seed_gemm_kernel(MmParams a, KConst kc) {
    constexpr bool BF16W = WF == 1, P3 = WF == 2;
    // A launch that follows this one and does not depend on it (the up projection after the gate projection) may be made
    // a programmatic dependent launch: its blocks then fill the SMs this grid's last wave leaves idle.
    grid_dependents_go();
    if (a.ntiles && (int) blockIdx.y >= *a.ntiles) return;
    extern __shared__ uint8_t smem_raw[];
    __shared__ StreamTab tab;
    __shared__ __align__(8) uint64_t bars[2 * GM_STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ int srow[GM_BN], drow[GM_BN];
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t* smem = (uint8_t*) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    constexpr int STAGE_BYTES = (NT + 1) * GM_TILE_BYTES;   // NT weight tiles + the input tile
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[GM_STAGES]), bar_done = smem_u32(&bars[2 * GM_STAGES]);

    int start, count;
    WSlice w;
    if (a.grouped) {
        const MmTile tl = a.tiles[blockIdx.y];
        w = a.ws[tl.slice];
        start = tl.start;
        count = tl.count < GM_BN ? tl.count : GM_BN;
    } else {
        w = a.w0;
        start = (int) blockIdx.y * GM_BN;
        count = a.T - start < GM_BN ? a.T - start : GM_BN;
    }
    if (count <= 0) return;
    const int n_eff = (count + 15) & ~15;
    const int r0 = (int) blockIdx.x * GM_BM;
    const int NB = a.K / 8, KT = (a.K + GM_BK - 1) / GM_BK;

    if (!BF16W) load_stream_tab(tab, a.G, tid, GM_THREADS);
    if (tid < GM_BN) {
        const bool ok = tid < count;
        srow[tid] = !ok ? -1 : a.grouped ? a.perm[start + tid] / a.xdiv : start + tid;
        drow[tid] = !ok ? -1 : a.grouped ? a.perm[start + tid] : start + tid;
    }
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < GM_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, GM_PRODUCERS / 32);      // one arrival per producer warp
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == GM_PRODUCERS / 32) {   // the MMA warp owns the TMEM allocation: 128 f32 columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(GM_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = tmem_slot;

    if (warp < GM_PRODUCERS / 32) {
        // ---- producers: weight tile (thread = row, half of the 8 blocks) and input tile (thread = token, half of 64 k) --
        const int prow = tid >> 1, half = tid & 1;
        const int grow = r0 + prow;
        constexpr bool vec = VEC;
        QuadIn cur = {{0u, 0u}, {0u, 0u}, 0u, false}, nxt = cur;
        uint4 bcur[4], bnxt[4];      // BF16 weights: this thread's 32 values of the K step, as stored
        auto load_bf16 = [&](int kt, uint4* o) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = kt * GM_BK + half * 32 + 8 * i;
                o[i] = grow < a.R && k < a.K ? __ldg((const uint4*) ((const uint16_t*) w.p[0] + (size_t) grow * a.K + k)) : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        if (BF16W) load_bf16(0, bcur);
        else cur = load_quad<P3>(w, grow, half * 4, a.R, NB, vec);
        nxt = cur;
        // packed inputs: this thread's 16-byte chunks of the K step's n_eff x 64 tile (chunk ci = tid + 256 i), requested one
        // K step ahead so that they land during the expansion
        uint4 xq[4];
        const int nx = (n_eff * 8 + GM_PRODUCERS - 1) / GM_PRODUCERS;      // chunks per thread: 1 for tiles of up to 32 pairs
        auto load_x = [&](int kt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int ci = tid + i * GM_PRODUCERS;
                if (i < nx) xq[i] = make_uint4(0u, 0u, 0u, 0u);
                if (i < nx && ci < n_eff * 8) {
                    const int src = srow[ci >> 3], k = kt * GM_BK + 8 * (ci & 7);
                    if (src >= 0 && k < a.K) xq[i] = __ldg((const uint4*) ((const uint16_t*) a.X + (size_t) src * a.xs + k));
                }
            }
        };
        // f32 inputs: the thread's first two chunks (tiles of up to 64 pairs whole) travel the same way as raw values, two
        // float4 a chunk in the same registers (xq[2 c], xq[2 c + 1]); further chunks are loaded and converted in place
        auto load_xf = [&](int kt) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int ci = tid + c * GM_PRODUCERS;
                xq[2 * c] = xq[2 * c + 1] = make_uint4(0u, 0u, 0u, 0u);
                if (c < nx && ci < n_eff * 8) {
                    const int src = srow[ci >> 3], k = kt * GM_BK + 8 * (ci & 7);
                    if (src >= 0 && k < a.K) {
                        const uint4* xp = (const uint4*) ((const float*) a.X + (size_t) src * a.xs + k);
                        xq[2 * c] = __ldg(xp);
                        xq[2 * c + 1] = __ldg(xp + 1);
                    }
                }
            }
        };
        if (a.packed) load_x(0); else load_xf(0);
        bool live = true;
        for (int kt = 0; kt < KT && live; ++kt) {
            const int s = kt % GM_STAGES;
            if (kt + 1 < KT) {
                if (BF16W) load_bf16(kt + 1, bnxt);
                else nxt = load_quad<P3>(w, grow, (kt + 1) * 8 + half * 4, a.R, NB, vec);
            }
            if (kt >= GM_STAGES && !mbar_wait<false>(bar_empty + 8 * s, ((kt / GM_STAGES) - 1) & 1, &abort_flag)) {
                abort_flag = 1;
                atomicCAS(&g_mm_status, 0, 1);
                live = false;
                break;
            }
            uint8_t* stage = smem + (size_t) s * STAGE_BYTES;
            if (BF16W) {      // stored weights: the row's four 16-byte chunks of this half, as they are
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int chunk = half * 4 + i;
                    *(uint4*) (stage + (uint32_t) prow * 128u + (uint32_t) ((chunk ^ (prow & 7)) << 4)) = bcur[i];
                }
            }
            if (a.packed) {      // this K step's inputs (requested a step ago), then the next step's request
                uint8_t* bt = stage + (size_t) NT * GM_TILE_BYTES;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int ci = tid + i * GM_PRODUCERS, n = ci >> 3, chunk = ci & 7;
                    if (i < nx && ci < n_eff * 8) *(uint4*) (bt + (uint32_t) n * 128u + (uint32_t) ((chunk ^ (n & 7)) << 4)) = xq[i];
                }
                if (kt + 1 < KT) load_x(kt + 1);
            } else {
                uint8_t* bt = stage + (size_t) NT * GM_TILE_BYTES;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int ci = tid + c * GM_PRODUCERS, n = ci >> 3, chunk = ci & 7;
                    if (c < nx && ci < n_eff * 8) {
                        const uint4 lo = xq[2 * c], hi = xq[2 * c + 1];
                        *(uint4*) (bt + (uint32_t) n * 128u + (uint32_t) ((chunk ^ (n & 7)) << 4)) =
                            make_uint4(bf16x2_bits(__uint_as_float(lo.x), __uint_as_float(lo.y)), bf16x2_bits(__uint_as_float(lo.z), __uint_as_float(lo.w)),
                                       bf16x2_bits(__uint_as_float(hi.x), __uint_as_float(hi.y)), bf16x2_bits(__uint_as_float(hi.z), __uint_as_float(hi.w)));
                    }
                }
                if (kt + 1 < KT) load_xf(kt + 1);
            }
            // seed weights: two block pairs, expanded side by side
#pragma unroll
            for (int bp = 0; bp < (BF16W ? 0 : 2); ++bp) {
                float wa[8], wb[8];
                if (cur.live && P3) {      // two P = 3 blocks, each bit for bit as nsl_decode3_f32 gives it
                    const uint32_t sa = cur.sw[bp] & 0xFFFFu, sb = cur.sw[bp] >> 16, na = cur.cw[bp] & 0xFFFFu, nb = cur.cw[bp] >> 16;
                    const uint32_t ga = stream_bits(tab, sa), gb = stream_bits(tab, sb);
                    block_weights3(sa | (ga << 16), ga, na, exact_scale45(w.eb + (int) (na & 15u) + 1), kc, wa);
                    block_weights3(sb | (gb << 16), gb, nb, exact_scale45(w.eb + (int) (nb & 15u) + 1), kc, wb);
                } else if (cur.live) {
                    const uint32_t cd = cur.codes >> (8 * bp);
                    const u64 sc2 = pack2(exact_scale45(w.eb + (int) (cd & 15u)), exact_scale45(w.eb + (int) ((cd >> 4) & 15u)));
                    u64 w2[8];
                    pair_weights(tab, cur.sw[bp], cur.cw[bp], sc2, kc, w2);
#pragma unroll
                    for (int i = 0; i < 8; ++i) unpack2(w2[i], wa[i], wb[i]);
                }
                if (cur.live) {
                    if (!vec) {   // a row whose block count is not a multiple of 4 ends inside a quad: blocks past it are zero
                        const bool has_a = (cur.sw[bp] & 0xFFFFu) != 0u, has_b = (cur.sw[bp] >> 16) != 0u;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            if (!has_a) wa[i] = 0.0f;
                            if (!has_b) wb[i] = 0.0f;
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) wa[i] = wb[i] = 0.0f;
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float* wv = e ? wb : wa;
                    const int chunk = half * 4 + 2 * bp + e;
                    const uint32_t off = (uint32_t) prow * 128u + (uint32_t) ((chunk ^ (prow & 7)) << 4);
#pragma unroll
                    for (int q = 0; q < NT; ++q) {   // term q = the bf16 value of what remains (exact subtraction)
                        const uint4 o = make_uint4(bf16x2_bits(wv[0], wv[1]), bf16x2_bits(wv[2], wv[3]),
                                                   bf16x2_bits(wv[4], wv[5]), bf16x2_bits(wv[6], wv[7]));
                        *(uint4*) (stage + (size_t) q * GM_TILE_BYTES + off) = o;
                        if (q + 1 < NT) {
                            wv[0] -= __uint_as_float(o.x << 16); wv[1] -= __uint_as_float(o.x & 0xFFFF0000u);
                            wv[2] -= __uint_as_float(o.y << 16); wv[3] -= __uint_as_float(o.y & 0xFFFF0000u);
                            wv[4] -= __uint_as_float(o.z << 16); wv[5] -= __uint_as_float(o.z & 0xFFFF0000u);
                            wv[6] -= __uint_as_float(o.w << 16); wv[7] -= __uint_as_float(o.w & 0xFFFF0000u);
                        }
                    }
                }
            }
            // f32 inputs: the n_eff x 64 tile as 16-byte chunks (8 values) dealt round-robin to the producer threads
            if (!a.packed) {
                uint8_t* bt = stage + (size_t) NT * GM_TILE_BYTES;
                for (int ci = tid + 2 * GM_PRODUCERS; ci < n_eff * 8; ci += GM_PRODUCERS) {      // chunks beyond the two that were requested ahead
                    const int n = ci >> 3, chunk = ci & 7, src = srow[n], k = kt * GM_BK + 8 * chunk;
                    uint4 o = make_uint4(0u, 0u, 0u, 0u);
                    if (src >= 0 && k < a.K) {
                        const float4* xp = (const float4*) ((const float*) a.X + (size_t) src * a.xs + k);
                        const float4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
                        o = make_uint4(bf16x2_bits(x0.x, x0.y), bf16x2_bits(x0.z, x0.w), bf16x2_bits(x1.x, x1.y),
                                       bf16x2_bits(x1.z, x1.w));
                    }
                    *(uint4*) (bt + (uint32_t) n * 128u + (uint32_t) ((chunk ^ (n & 7)) << 4)) = o;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA's reads
            __syncwarp();                                                  // the warp's 32 lanes have written and fenced:
            if (lane == 0) mbar_arrive(bar_full + 8 * s);                  // one arrival for all of them (not 32 on one word)
            cur = nxt;
            if (BF16W) {
#pragma unroll
                for (int i = 0; i < 4; ++i) bcur[i] = bnxt[i];
            }
        }
        // ---- epilogue: TMEM lane = weight row, column = token ----------------------------------------------------------
        if (live && !mbar_wait(bar_done, 0, &abort_flag)) {
            abort_flag = 1;
            atomicCAS(&g_mm_status, 0, 2);
            live = false;
        }
        if (live) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int lq = warp & 3, chalf = warp >> 2;
            const int row = r0 + lq * 32 + lane;
            for (int c0 = chalf * 64; c0 < chalf * 64 + 64 && c0 < n_eff; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_acc + ((uint32_t) (lq * 32) << 16) + (uint32_t) c0, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int dst = drow[c0 + j];
                    if (dst < 0 || row >= a.R) continue;
                    float* yo = a.Y + (size_t) dst * a.ys + row;
                    const float acc = __uint_as_float(v[j]);
                    *yo = a.add ? bf16_round(*yo + bf16_round(acc)) : bf16_round(acc);   // engine/kernels_moe.cu:214
                }
            }
        }
    } else if (lane == 0) {
        // ---- the MMA issuer --------------------------------------------------------------------------------------------
        const uint32_t idesc = umma_idesc(n_eff);
        bool live = true;
        for (int kt = 0; kt < KT; ++kt) {
            const int s = kt % GM_STAGES;
            if (!mbar_wait(bar_full + 8 * s, (kt / GM_STAGES) & 1, &abort_flag)) {
                abort_flag = 1;
                atomicCAS(&g_mm_status, 0, 3);
                live = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = smem_base + (uint32_t) s * STAGE_BYTES, sb = sa + NT * GM_TILE_BYTES;
#pragma unroll
            for (int q = 0; q < NT; ++q)
#pragma unroll
                for (int k4 = 0; k4 < GM_BK / 16; ++k4)
                    umma(tmem_acc, umma_desc(sa + q * GM_TILE_BYTES + k4 * 32), umma_desc(sb + k4 * 32), idesc,
                         (kt | q | k4) != 0);
            umma_commit(bar_empty + 8 * s);   // the stage is free when these MMAs have read it
        }
        if (live) umma_commit(bar_done);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == GM_PRODUCERS / 32) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(GM_BN) : "memory");
    }
}

bool launch_bf16_mm_skinny(cudaStream_t s, const WSlice& w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add);

thread_local bool tl_mm_overlap = false;

static int g_exact;   // kc_seed_gemm_f32: process-wide, as the reference's switch (engine/kernels_moe.cu:2354)

template <int NT, int WF, bool VEC>
static void launch_gemm_v(cudaStream_t s, const MmParams& a, dim3 grid) {
    const size_t smem = (size_t) GM_STAGES * (NT + 1) * GM_TILE_BYTES + 1024;
    static bool attr_set[16];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 15]) {
        cudaFuncSetAttribute(seed_gemm_kernel<NT, WF, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        attr_set[dev & 15] = true;
    }
    // tl_mm_overlap: the caller says this launch reads nothing its predecessor in the stream writes
    PdlScope pdl(tl_mm_overlap);
    launch(seed_gemm_kernel<NT, WF, VEC>, grid, GM_THREADS, smem, s, a, kconst());
    count_launch();
}
template <int NT, int WF>
static void launch_gemm_nt(cudaStream_t s, const MmParams& a, dim3 grid) {
    if (WF == 1 || a.K % 32 == 0) launch_gemm_v<NT, WF, true>(s, a, grid);      // stored BF16 weights have no quads
    else launch_gemm_v<NT, WF, false>(s, a, grid);
}

static void launch_gemm(cudaStream_t s, int fmt, const char* who, MmParams a, int tiles_y) {
    if (fmt != MF_SEED4P4 && fmt != MF_SEED4 && fmt != MF_BF16) {
        set_error("%s: weight format %d is not served by this library (SEED4P4 = %d, SEED4 = %d and BF16 = %d only)", who, fmt, (int) MF_SEED4P4,
                  (int) MF_SEED4, (int) MF_BF16);
        return;
    }
    if (a.K <= 0 || a.K % 8 || a.R <= 0) { set_error("%s: K = %d (a multiple of 8), R = %d", who, a.K, a.R); return; }
    if (fmt == MF_BF16 && ((a.ws == NULL && !aligned16(a.w0.p[0])))) { set_error("%s: BF16 weights must be 16-byte aligned", who); return; }
    if (tiles_y <= 0) return;
    if (!aligned16(a.X) || (a.packed ? a.xs % 8 : a.xs % 4)) {
        set_error("%s: inputs must be 16-byte aligned with a row stride that is a multiple of 16 bytes", who);
        return;
    }
    const dim3 grid((unsigned) ((a.R + GM_BM - 1) / GM_BM), (unsigned) tiles_y);
    if (fmt == MF_BF16) launch_gemm_nt<1, 1>(s, a, grid);      // stored BF16 weights (p[0] = [R][K]): no expansion, one term
    else if (fmt == MF_SEED4) { if (g_exact) launch_gemm_nt<3, 2>(s, a, grid); else launch_gemm_nt<1, 2>(s, a, grid); }      // P = 3
    else if (g_exact) launch_gemm_nt<3, 0>(s, a, grid);
    else launch_gemm_nt<1, 0>(s, a, grid);
}

}   // namespace nsl

using namespace nsl;

extern "C" {

void kc_seed_gemm_f32(int on) { g_exact = on; }

void kc_mm(cudaStream_t s, int fmt, WSlice w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add,
           const uint32_t* G) {
    if (fmt == MF_BF16 && launch_bf16_mm_skinny(s, w, K, R, x, xs, y, ys, T, add)) return;      // a decode batch (dense_bf16.cu)
    MmParams a = {NULL, w, x, y, NULL, NULL, NULL, G, NULL, K, R, T, xs, ys, 1, add, 0, 0};
    launch_gemm(s, fmt, "kc_mm", a, (T + GM_BN - 1) / GM_BN);
}
void kc_mm_packed(cudaStream_t s, int fmt, WSlice w, int K, int R, const uint16_t* x, int xs, float* y, int ys, int T, int add,
                  const uint32_t* G) {
    MmParams a = {NULL, w, x, y, NULL, NULL, NULL, G, NULL, K, R, T, xs, ys, 1, add, 0, 1};
    launch_gemm(s, fmt, "kc_mm_packed", a, (T + GM_BN - 1) / GM_BN);
}
void kc_mm_grouped(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                   int xdiv, const int32_t* perm, const MmTile* tiles, int ntiles, const uint32_t* G) {
    MmParams a = {ws, WSlice{}, x, y, perm, tiles, NULL, G, NULL, K, R, 0, xs, ys, xdiv, 0, 1, 0};
    launch_gemm(s, fmt, "kc_mm_grouped", a, ntiles);
}
void kc_mm_grouped_dev(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                       int xdiv, const int32_t* perm, const MmTile* tiles, const int32_t* ntiles, int max_tiles,
                       const uint32_t* G) {
    MmParams a = {ws, WSlice{}, x, y, perm, tiles, ntiles, G, NULL, K, R, 0, xs, ys, xdiv, 0, 1, 0};
    launch_gemm(s, fmt, "kc_mm_grouped_dev", a, max_tiles);
}
void kc_mm_grouped_packed(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const uint16_t* x, int xs, float* y, int ys,
                          int xdiv, const int32_t* perm, const MmTile* tiles, const int32_t* nt, int max_tiles,
                          const uint32_t* G) {
    MmParams a = {ws, WSlice{}, x, y, perm, tiles, nt, G, NULL, K, R, 0, xs, ys, xdiv, 0, 1, 1};
    launch_gemm(s, fmt, "kc_mm_grouped_packed", a, max_tiles);
}

// 0, or the code of the first bounded wait that ran out in a GEMM block since the last call (1 producer waiting for a
// free stage, 2 epilogue waiting for the accumulator, 3 MMA issuer waiting for a full stage).  Reads device memory: call
// it after the stream has been synchronised.
int nsl_mm_status(void) {
    int v = 0, zero = 0;
    cudaMemcpyFromSymbol(&v, g_mm_status, sizeof v);
    if (v) cudaMemcpyToSymbol(g_mm_status, &zero, sizeof zero);
    return v;
}

}   // extern "C"
