// Decode attention over a BF16 or 8-bit KV cache with grouped query heads: split-key partial passes on the tensor cores
// and their reduction with the softplus output gate (engine/kernels_moe.cu:887-952, 2421-2426; engine/kernels_cuda.h:56-72,
// 130-131).  Two forms of the first pass: the step's keys dealt evenly to the blocks (the default), and a block per caller
// split (a row's result then never depends on the rows it shares a call with).
// Partials and the reduction have the reference's layout and rounding points: part[row][head][split] = (m, l, acc[128]);
// o = bf16(bf16(acc / l) * bf16(softplus(g))).
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

constexpr int ATT_KROW = 272;      // bytes of a staged K row (256 + 16: ldmatrix then touches distinct banks)

// ---- the first pass on the tensor cores -----------------------------------------------------------------------------------
// One warp serves ALL query heads of the KV head: they are the columns of mma.sync.m16n8k16 products (bf16 in, f32
// accumulate; 8 heads a tile, columns beyond the group are zero; see attn_keys for the two products).  Queries are
// bf16-valued, so the score products are exact and the softmax scale is applied to the f32 sums; the weights enter the
// second product as two bf16 terms (hi + lo: 16 significant bits; their sum l is kept in f32).  Per step of 16 keys a warp
// issues 8 MMAs for the scores and 16 for the values of a tile instead of ~2500 scalar instructions for the group.  The
// warps of a block take a key range's steps in turn, each with its own running (m, l, acc) and its own ring of K / V rows
// in shared memory (the next step's rows fly while this one is computed; rows 272 bytes apart: ldmatrix touches distinct
// banks); at the end the warps' states are merged through the same shared memory.
constexpr int ATT_MMA_WARPS = 4, ATT_VROW = 272, ATT_MT = 16, ATT_SLOT = ATT_MT * (ATT_KROW + ATT_VROW);
constexpr int ATT_MAX_ROWS = 1024;      // rows of a step in the balanced form (the reference's rows x splits <= 1024)
static_assert(2 * ATT_SLOT >= ATT_MAX_GROUP * 130 * 4, "a warp's ring holds its final state");
static_assert(32 * ATT_MMA_WARPS == ATT_HD && ATT_MMA_WARPS == 4, "the merge gives a thread one dim; ring_sync numbers four rings");

__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Two f32 to a bf16 pair, round to nearest even (lo in bits 0-15).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {      // 2^x, relative error 2^-22; 2^-inf = 0
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void attn_cp16s(unsigned smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gmem) : "memory");
}

// The 16 K rows and 16 V rows of the step at key p into a slot: 32 lanes x 8 pieces of 16 bytes each (rows beyond the range
// repeat its last row; their scores are masked).  Always one cp.async group, empty when the step lies beyond the range.
__device__ __forceinline__ void attn_fill_slot(unsigned char* slot, const KvView& kv, int n_kv, int kvh, int kv0, int p, int p1, int lane) {
    constexpr int N = ATT_MT / 2;
    if (p < p1) {
        const int rl = lane >> 4, piece = lane & 15;
        const unsigned sk = (unsigned) __cvta_generic_to_shared(slot) + rl * ATT_KROW + piece * 16, sv = sk + ATT_MT * ATT_KROW;
        const int row0 = kv0 + p;
        if (p + ATT_MT <= p1 && (row0 + ATT_MT <= kv.nv || row0 >= kv.nv)) {      // 16 whole rows of one segment: one address, strides
            const unsigned char* kb = (const unsigned char*) (kv_row(kv, 0, row0 + rl, n_kv, kvh) + piece * 8);
            const unsigned char* vb = (const unsigned char*) (kv_row(kv, 1, row0 + rl, n_kv, kvh) + piece * 8);
            const size_t two_rows = (size_t) n_kv * (2 * ATT_HD * 2);
#pragma unroll
            for (int i = 0; i < N; ++i) {
                attn_cp16s(sk + i * 2 * ATT_KROW, kb + i * two_rows);
                attn_cp16s(sv + i * 2 * ATT_VROW, vb + i * two_rows);
            }
        } else {
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const int row = kv0 + min(p + 2 * i + rl, p1 - 1);
                attn_cp16s(sk + i * 2 * ATT_KROW, kv_row(kv, 0, row, n_kv, kvh) + piece * 8);
                attn_cp16s(sv + i * 2 * ATT_VROW, kv_row(kv, 1, row, n_kv, kvh) + piece * 8);
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned) __cvta_generic_to_shared(p); }

// ---- the 8-bit cache (KV_Q8: int8 codes, one f32 scale per row and KV head; engine/kernels_cuda.h:58-59) ------------------
// A warp's ring holds the raw rows of two steps (16 K rows and 16 V rows of 128 bytes, then their 32 scales); before a step
// is used its rows are expanded into the one BF16 slot the products read: bf16(code * scale), the value the reference's
// kernels read (engine/kernels_moe.cu:807-824).
constexpr int ATT_RAW_V = ATT_MT * ATT_HD, ATT_RAW_SCALES = 2 * ATT_RAW_V, ATT_RAW = ATT_RAW_SCALES + 2 * ATT_MT * 4;
static_assert(ATT_SLOT + 2 * ATT_RAW <= 2 * ATT_SLOT, "the BF16 slot and two raw slots fit a two-slot ring");

__device__ __forceinline__ void attn_cp4s(unsigned smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem), "l"(gmem) : "memory");
}
__device__ __forceinline__ const KvSeg& kv_seg_of(const KvView& kv, int abs_pos, int& row) {
    const bool first = abs_pos < kv.nv;
    row = first ? abs_pos : abs_pos - kv.nv;
    return first ? kv.a : kv.b;
}
// The step at key p, raw: 256 pieces of 16 bytes (8 rounds of 32) and 32 scales.
// Always one cp.async group.
__device__ __forceinline__ void attn_fill_raw(unsigned char* raw, const KvView& kv, int n_kv, int kvh, int kv0, int p, int p1, int lane) {
    if (p < p1) {
        const unsigned base = smem_u32(raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int id = i * 32 + lane, is_v = id >> 7, r = (id >> 3) & 15, piece = id & 7;
            int row;
            const KvSeg& sg = kv_seg_of(kv, kv0 + min(p + r, p1 - 1), row);
            attn_cp16s(base + is_v * ATT_RAW_V + r * ATT_HD + piece * 16,
                       (const unsigned char*) (is_v ? sg.v : sg.k) + ((size_t) row * n_kv + kvh) * ATT_HD + piece * 16);
        }
        {
            const int is_v = lane >> 4, r = lane & 15;
            int row;
            const KvSeg& sg = kv_seg_of(kv, kv0 + min(p + r, p1 - 1), row);
            attn_cp4s(base + ATT_RAW_SCALES + lane * 4, (is_v ? sg.vs : sg.ks) + (size_t) row * n_kv + kvh);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ uint32_t q8_pair(uint32_t u, int i, float s) {      // codes i and i + 1 of a word as a bf16 pair
    const float a = (float) (int) (signed char) ((u >> (8 * i)) & 255u) * s, b = (float) (int) (signed char) ((u >> (8 * i + 8)) & 255u) * s;
    return pack_bf16x2(a, b);
}
// Raw rows -> the BF16 slot (rows 272 bytes apart, K then V).
__device__ __forceinline__ void attn_expand_raw(unsigned char* slot, const unsigned char* raw, int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int id = i * 32 + lane, is_v = id >> 7, r = (id >> 3) & 15, piece = id & 7;
        const uint4 u = *(const uint4*) (raw + is_v * ATT_RAW_V + r * ATT_HD + piece * 16);
        const float sc = *(const float*) (raw + ATT_RAW_SCALES + (is_v * ATT_MT + r) * 4);
        uint4 lo, hi;
        lo.x = q8_pair(u.x, 0, sc); lo.y = q8_pair(u.x, 2, sc); lo.z = q8_pair(u.y, 0, sc); lo.w = q8_pair(u.y, 2, sc);
        hi.x = q8_pair(u.z, 0, sc); hi.y = q8_pair(u.z, 2, sc); hi.z = q8_pair(u.w, 0, sc); hi.w = q8_pair(u.w, 2, sc);
        uint4* dst = (uint4*) (slot + is_v * ATT_MT * ATT_KROW + r * ATT_KROW + piece * 32);
        dst[0] = lo;
        dst[1] = hi;
    }
}

__device__ __forceinline__ void ldsm_x4(uint32_t* r, const unsigned char* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned) __cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, const unsigned char* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned) __cvta_generic_to_shared(p)));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {      // an 8 x 8 tile of 16-bit values, transposed across the warp
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

// Keys [p0, p1) of row t's cache for the query heads of KV head kvh, by the whole block: the warps take the steps of 16 keys
// in turn, merge their states and write the group's partials (m, l, acc[128]) at pp, pp + head_stride, ...
// NSLOT = slots of a warp's ring (steps in flight + the one in use); NT = tiles of 8 heads (1: groups of <= 8; 2: <= 16).
// The products are the transposed ones, so that the 8 columns of a tile are heads and nothing is computed for absent rows:
//   S^T [16 keys][8 heads]   = K [16 keys][128] . Q^T      A = K rows by ldmatrix, B = Q^T in registers (16 per tile)
//   O^T [128 dims][8 heads] += V^T [dims][16 keys] . P^T   A = V rows by ldmatrix.trans, B = P^T: the C fragments of S^T
//                                                          as bf16 pairs, transposed across the warp by movmatrix
// A lane holds keys r0 and r0 + 8 of heads 2 q4 and 2 q4 + 1 of each tile: the maxima and sums of a head run over the 8
// lanes of equal q4.  Ends with the block in step (shared memory reusable).
// SRC: how the rows come.  ATT_SRC_ASYNC: BF16 rows by cp.async; ATT_SRC_Q8: the 8-bit cache (one BF16 slot and two raw slots).
enum { ATT_SRC_ASYNC = 0, ATT_SRC_Q8 = 2 };
template <int NSLOT, int NT, int SRC>
__device__ __forceinline__ void attn_keys(const AttnArgs& a, const float* __restrict__ q, const KvView& kv, int t, int kvh, int kv0,
                                          int p0, int p1, unsigned char* att_smem, float* pp, size_t head_stride) {
    constexpr int STAGE = NSLOT * ATT_SLOT, STRIDE = ATT_MMA_WARPS * ATT_MT;
    const int lane = threadIdx.x & 31, ring_id = threadIdx.x >> 5, q4 = lane & 3, r0 = lane >> 2;
    const int group = a.n_head / a.n_kv;
    unsigned char* stage = att_smem + (size_t) ring_id * STAGE;
    constexpr bool Q8 = SRC == ATT_SRC_Q8;
    constexpr int DT = 8;      // tiles of 16 dims of the value product
    static_assert(!Q8 || NSLOT == 2, "the 8-bit cache's ring has two raw slots");
    unsigned char* raw = stage + ATT_SLOT;      // Q8: the two raw slots behind the BF16 slot
    int p = p0 + ring_id * ATT_MT;
    if (Q8) {
        attn_fill_raw(raw, kv, a.n_kv, kvh, kv0, p, p1, lane);
    } else {
#pragma unroll
        for (int i = 0; i < NSLOT - 1; ++i)
            attn_fill_slot(stage + i * ATT_SLOT, kv, a.n_kv, kvh, kv0, p + i * STRIDE, p1, lane);
    }
    // Q^T as the B fragments of the 8 steps over the 128 dims: column r0 of a tile = head 8 nt + r0 (zero beyond the group);
    // the first rows of K and V fly meanwhile
    uint32_t qb[NT][8][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int head = 8 * nt + r0;
        const float* qh = q + ((size_t) t * a.n_head + kvh * group + head) * ATT_HD;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = 16 * j + 2 * q4;
            const float2 z = make_float2(0.0f, 0.0f);
            const float2 x = head < group ? *(const float2*) (qh + d) : z, y = head < group ? *(const float2*) (qh + d + 8) : z;
            qb[nt][j][0] = pack_bf16x2(x.x, x.y);
            qb[nt][j][1] = pack_bf16x2(y.x, y.y);
        }
    }
    float m[NT][2], l[NT][2], ot[NT][DT][4];      // [.][0]: head 2 q4 of the tile, [.][1]: head 2 q4 + 1; m in base-2 units
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        m[nt][0] = m[nt][1] = -INFINITY;
        l[nt][0] = l[nt][1] = 0.0f;
#pragma unroll
        for (int i = 0; i < DT; ++i) ot[nt][i][0] = ot[nt][i][1] = ot[nt][i][2] = ot[nt][i][3] = 0.0f;
    }
    const float scale2 = a.scale * 1.4426950408889634f;
    // lane -> the row it addresses of the four 8 x 8 tiles of an ldmatrix.x4:
    //   K (A = keys x dims):   tiles (keys 0-7 | 8-15) x (dims +0 | +8) in the order a0 a1 a2 a3 = (k lo, d lo) (k hi, d lo) (k lo, d hi) (k hi, d hi)
    //   V (A = dims x keys, transposed on load): (d lo, k lo) (d hi, k lo) (d lo, k hi) (d hi, k hi)
    const int k_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * ATT_KROW + (lane >> 4) * 16;
    const int v_off = ATT_MT * ATT_KROW + ((lane & 7) + (lane >> 4) * 8) * ATT_VROW + ((lane >> 3) & 1) * 16;
    int cur = 0, nxt = NSLOT - 1;      // the slot in use; the slot the step NSLOT - 1 ahead goes to (its reads ended with the
                                       // previous step's closing ring_sync)
    for (; p < p1; p += STRIDE) {
        if (Q8) {
            attn_fill_raw(raw + nxt * ATT_RAW, kv, a.n_kv, kvh, kv0, p + STRIDE, p1, lane);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
            __syncwarp();
            // the BF16 slot's reads ended with the previous step's closing ring_sync
            attn_expand_raw(stage, raw + cur * ATT_RAW, lane);
        } else {
            attn_fill_slot(stage + nxt * ATT_SLOT, kv, a.n_kv, kvh, kv0, p + (NSLOT - 1) * STRIDE, p1, lane);
            asm volatile("cp.async.wait_group %0;" ::"n"(NSLOT - 1) : "memory");
        }
        __syncwarp();
        const unsigned char* slot = Q8 ? stage : stage + cur * ATT_SLOT;
        nxt = cur;
        cur = cur + 1 == NSLOT ? 0 : cur + 1;
        // scores: two accumulation chains a tile (even and odd dim steps)
        float s[NT][4], s2[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = s2[nt][0] = s2[nt][1] = s2[nt][2] = s2[nt][3] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t ka[4];
            ldsm_x4(ka, slot + k_off + 32 * j);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma_bf16((j & 1) ? s2[nt] : s[nt], ka, qb[nt][j][0], qb[nt][j][1]);
        }
        // softmax in the base-2 domain: x = score * scale * log2(e); keys r0 (elements 0, 1) and r0 + 8 (2, 3)
        const bool v0 = p + r0 < p1, v1 = p + r0 + 8 < p1;
        uint32_t ph[NT][2], pl[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            s[nt][0] = v0 ? (s[nt][0] + s2[nt][0]) * scale2 : -INFINITY; s[nt][1] = v0 ? (s[nt][1] + s2[nt][1]) * scale2 : -INFINITY;
            s[nt][2] = v1 ? (s[nt][2] + s2[nt][2]) * scale2 : -INFINITY; s[nt][3] = v1 ? (s[nt][3] + s2[nt][3]) * scale2 : -INFINITY;
            float mxa = fmaxf(s[nt][0], s[nt][2]), mxb = fmaxf(s[nt][1], s[nt][3]);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                mxa = fmaxf(mxa, __shfl_xor_sync(0xFFFFFFFFu, mxa, off));
                mxb = fmaxf(mxb, __shfl_xor_sync(0xFFFFFFFFu, mxb, off));
            }
            mxa = fmaxf(mxa, m[nt][0]); mxb = fmaxf(mxb, m[nt][1]);      // finite: a step's first key is always valid
            const float cora = ex2_approx(m[nt][0] - mxa), corb = ex2_approx(m[nt][1] - mxb);
            m[nt][0] = mxa; m[nt][1] = mxb;
            s[nt][0] = ex2_approx(s[nt][0] - mxa); s[nt][2] = ex2_approx(s[nt][2] - mxa);
            s[nt][1] = ex2_approx(s[nt][1] - mxb); s[nt][3] = ex2_approx(s[nt][3] - mxb);
            l[nt][0] = fmaf(l[nt][0], cora, s[nt][0] + s[nt][2]);
            l[nt][1] = fmaf(l[nt][1], corb, s[nt][1] + s[nt][3]);
            if (cora != 1.0f || corb != 1.0f) {      // the running maxima rarely move after a range's first steps
#pragma unroll
                for (int i = 0; i < DT; ++i) { ot[nt][i][0] *= cora; ot[nt][i][1] *= corb; ot[nt][i][2] *= cora; ot[nt][i][3] *= corb; }
            }
            // the weights as two bf16 terms, hi + lo (16 significant bits): one bf16 term alone moves an output by up to a third
            // of its own bf16 unit, which after the two roundings of the gate shows as two-unit differences
            const uint32_t h01 = pack_bf16x2(s[nt][0], s[nt][1]), h23 = pack_bf16x2(s[nt][2], s[nt][3]);
            const uint32_t l01 = pack_bf16x2(s[nt][0] - bf_lo(h01), s[nt][1] - bf_hi(h01));
            const uint32_t l23 = pack_bf16x2(s[nt][2] - bf_lo(h23), s[nt][3] - bf_hi(h23));
            ph[nt][0] = movmatrix_trans(h01); ph[nt][1] = movmatrix_trans(h23);
            pl[nt][0] = movmatrix_trans(l01); pl[nt][1] = movmatrix_trans(l23);
        }
        // values: this warp's tiles of 16 dims
#pragma unroll
        for (int i = 0; i < DT; ++i) {
            uint32_t va[4];
            ldsm_x4_trans(va, slot + v_off + 32 * i);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mma_bf16(ot[nt][i], va, ph[nt][0], ph[nt][1]);
                mma_bf16(ot[nt][i], va, pl[nt][0], pl[nt][1]);
            }
        }
        __syncwarp();      // this slot's reads are done before a later step refills it
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");      // only empty groups are left
    // the ring's state into the ring: [16 heads][130] = m (natural units; -inf stays -inf), l, acc (each warp its dims)
    __syncwarp();
    float* mine = (float*) stage;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l[nt][0] += __shfl_xor_sync(0xFFFFFFFFu, l[nt][0], off);
            l[nt][1] += __shfl_xor_sync(0xFFFFFFFFu, l[nt][1], off);
        }
        float* ha = mine + (8 * nt + 2 * q4) * 130, *hb = ha + 130;
        if (r0 == 0) {
            ha[0] = m[nt][0] * 0.69314718055994531f; ha[1] = l[nt][0];
            hb[0] = m[nt][1] * 0.69314718055994531f; hb[1] = l[nt][1];
        }
#pragma unroll
        for (int i = 0; i < DT; ++i) {
            const int d = 2 + 16 * i + r0;
            ha[d] = ot[nt][i][0]; hb[d] = ot[nt][i][1]; ha[d + 8] = ot[nt][i][2]; hb[d + 8] = ot[nt][i][3];
        }
    }
    __syncthreads();
    // merge the rings' states.  A head's four weights exp(m_ring - max) are the same for all 128 dims: thread h computes
    // them once (and the head's m and l), then thread d handles dim d of every head.
    __shared__ float merge_c[ATT_MMA_WARPS][ATT_MAX_GROUP], merge_m[ATT_MAX_GROUP], merge_l[ATT_MAX_GROUP];
    if (threadIdx.x < group) {
        const int h = threadIdx.x;
        float mm = -INFINITY;
        for (int w = 0; w < ATT_MMA_WARPS; ++w) mm = fmaxf(mm, ((const float*) (att_smem + (size_t) w * STAGE))[h * 130]);
        float ll = 0.0f;
        for (int w = 0; w < ATT_MMA_WARPS; ++w) {
            const float* st = (const float*) (att_smem + (size_t) w * STAGE) + h * 130;
            const float c = st[0] == -INFINITY ? 0.0f : expf(st[0] - mm);      // a ring without keys: weight 0 (its l and acc are 0)
            merge_c[w][h] = c;
            ll = fmaf(st[1], c, ll);
        }
        merge_m[h] = mm;
        merge_l[h] = ll;
    }
    __syncthreads();
    const int d = threadIdx.x;
    for (int h = 0; h < group; ++h) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_MMA_WARPS; ++w) acc = fmaf(((const float*) (att_smem + (size_t) w * STAGE))[h * 130 + 2 + d], merge_c[w][h], acc);
        float* ph = pp + h * head_stride;
        if (d == 0) { ph[0] = merge_m[h]; ph[1] = merge_l[h]; }
        ph[2 + d] = acc;
    }
    __syncthreads();
}

// One block per (split, KV head, row): the split's keys as the reference cuts them.
template <int NSLOT, int NT, int SRC>
__global__ void __launch_bounds__(32 * ATT_MMA_WARPS) attn_split_mma_kernel(AttnArgs a, const float* __restrict__ q, KvView kv,
                                                                            const RowInfo* __restrict__ ri, float* __restrict__ part) {
    extern __shared__ __align__(16) unsigned char att_smem[];      // the warps' rings, later their states
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int group = a.n_head / a.n_kv;
    grid_dependency_wait();      // the rows' positions and q may come from the previous kernel in the stream
    grid_dependents_go();        // only now: the reduction reads the rows' positions as soon as it starts
    const int pos = ri[t].pos, kv0 = ri[t].kv0;
    const int nsr = a.chunk > 0 ? min(a.n_splits, (pos + a.chunk) / a.chunk) : 1;
    const int chunk = (pos + nsr) / nsr;
    const int p0 = split * chunk, p1 = min(pos + 1, p0 + chunk);
    attn_keys<NSLOT, NT, SRC>(a, q, kv, t, kvh, kv0, p0, p1, att_smem, part + (((size_t) t * a.n_head + kvh * group) * a.n_splits + split) * (ATT_HD + 2),
                                (size_t) a.n_splits * (ATT_HD + 2));
}

// ---- the balanced form ------------------------------------------------------------------------------------------------
// The step's work is cut into units of 16 keys, numbered row by row, KV head by KV head; block b takes units
// [b * per, (b + 1) * per), whichever rows they belong to, so every block reads the same number of bytes whatever the
// rows' lengths and the caller's split count.  A (row, KV head) pair's units lie in consecutive blocks; the j-th of them
// writes the pair's partial j, and `per` is raised until no pair has more partials than the caller's buffer holds
// (n_splits per head).  Both kernels derive the same plan from the rows' positions.
struct AttnPlan {
    int total;      // units of the step (all rows, all KV heads)
    int per;        // units per block
};

// u(t) = units of row t; pre[t] = u(0) + ... + u(t - 1), pre[T] = their sum.  Called by all threads of a block of NW warps.
template <int NW>
__device__ __forceinline__ AttnPlan attn_plan(const RowInfo* __restrict__ ri, int T, int n_kv, int n_splits, int n_blocks, int* pre) {
    __shared__ int wsum[NW], wmax[NW];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int each = (T + 32 * NW - 1) / (32 * NW);      // <= 8 rows a thread
    int sum = 0, mx = 0;
    for (int i = 0; i < each; ++i) {
        const int r = tid * each + i;
        const int u = r < T ? (max(ri[r].pos, 0) + ATT_MT) / ATT_MT : 0;
        sum += u;
        mx = max(mx, u);
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, off);
        if (lane >= off) incl += v;
        mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    }
    if (lane == 31) { wsum[warp] = incl; wmax[warp] = mx; }
    __syncthreads();
    int before = 0, rows_total = 0, max_u = 0;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        if (w < warp) before += wsum[w];
        rows_total += wsum[w];
        max_u = max(max_u, wmax[w]);
    }
    int run = before + incl - sum;
    for (int i = 0; i < each; ++i) {
        const int r = tid * each + i;
        if (r < T) {
            pre[r] = run;
            run += (max(ri[r].pos, 0) + ATT_MT) / ATT_MT;
        }
    }
    if (tid == 0) pre[T] = rows_total;
    __syncthreads();
    AttnPlan pl;
    pl.total = rows_total * n_kv;
    pl.per = max((pl.total + n_blocks - 1) / n_blocks, ATT_MMA_WARPS);                   // every warp of a block has a step
    pl.per = max(pl.per, (max_u - 1 + n_splits - 3) / (n_splits - 2));                    // a pair: <= (u - 1) / per + 2 partials
    return pl;
}

template <int NSLOT, int NT, int SRC>
__global__ void __launch_bounds__(32 * ATT_MMA_WARPS, NT == 2 && SRC == ATT_SRC_Q8 ? 2 : 3)      // three blocks an SM: <= 168 / 85 registers
attn_flat_mma_kernel(AttnArgs a, const float* __restrict__ q, KvView kv, const RowInfo* __restrict__ ri, float* __restrict__ part, int T) {
    extern __shared__ __align__(16) unsigned char att_smem[];
    __shared__ int pre[ATT_MAX_ROWS + 1];
    const int group = a.n_head / a.n_kv;
    grid_dependency_wait();      // the rows' positions and q may come from the previous kernel in the stream
    grid_dependents_go();        // only now: the reduction reads the rows' positions as soon as it starts
    const AttnPlan pl = attn_plan<ATT_MMA_WARPS>(ri, T, a.n_kv, a.n_splits, (int) gridDim.x, pre);
    int x = (int) blockIdx.x * pl.per;
    const int xe = min(pl.total, x + pl.per);
    while (x < xe) {
        // the row of unit x: the last t with n_kv * pre[t] <= x
        int lo = 0, hi = T - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (a.n_kv * pre[mid] <= x) lo = mid; else hi = mid - 1;
        }
        const int t = lo, u = pre[t + 1] - pre[t];
        const int kvh = (x - a.n_kv * pre[t]) / u;
        const int first = a.n_kv * pre[t] + kvh * u;      // the pair's first unit
        const int end = min(xe, first + u);
        const int pos = max(ri[t].pos, 0), kv0 = ri[t].kv0;
        const int slot = (int) blockIdx.x - first / pl.per;
        attn_keys<NSLOT, NT, SRC>(a, q, kv, t, kvh, kv0, (x - first) * ATT_MT, min(pos + 1, (end - first) * ATT_MT), att_smem,
                                  part + (((size_t) t * a.n_head + kvh * group) * a.n_splits + slot) * (ATT_HD + 2),
                                  (size_t) a.n_splits * (ATT_HD + 2));
        x = end;
    }
}

__device__ __forceinline__ float softplus_ln2(float g) {   // softplus with beta = ln 2 in f32, then BF16
    const float gx = g * 0.69314718055994531f;
    return bf16_round((fmaxf(gx, 0.0f) + logf(1.0f + expf(-fabsf(gx)))) / 0.69314718055994531f);
}

// Merges a head's partials and applies the gate.  n_blocks = 0: the split form's n_splits partials (unused ones carry
// m = -inf); otherwise the balanced form's, as many as the pair's units touch blocks.
__global__ void __launch_bounds__(ATT_HD) attn_reduce_kernel(AttnArgs a, const float* __restrict__ part, const float* __restrict__ g,
                                                             float* __restrict__ o, const RowInfo* __restrict__ ri, int T, int n_blocks) {
    __shared__ int pre[ATT_MAX_ROWS + 1];
    const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
    grid_dependents_go();
    // This kernel is always launched behind the first pass, whose blocks let their dependents go only AFTER their own wait
    // for the kernel before kc_attn: by the time a block runs here the rows' positions are final, and the plan can be made
    // while the first pass is still running.  The partials are read after the wait below.
    int n = a.n_splits;
    if (n_blocks > 0) {
        const AttnPlan pl = attn_plan<ATT_HD / 32>(ri, T, a.n_kv, a.n_splits, n_blocks, pre);
        const int u = pre[t + 1] - pre[t], first = a.n_kv * pre[t] + (h / (a.n_head / a.n_kv)) * u;
        n = (first + u - 1) / pl.per - first / pl.per + 1;
    }
    grid_dependency_wait();
    const float* pp = part + ((size_t) t * a.n_head + h) * a.n_splits * (ATT_HD + 2);
    __shared__ float pm[ATT_HD], pl[ATT_HD], pc[ATT_HD];      // the partials' (m, l): one load each, side by side; their weights
    float m = -INFINITY, l = 0.0f, acc = 0.0f;
    if (n <= ATT_HD) {
        if (d < n) { pm[d] = pp[d * (ATT_HD + 2)]; pl[d] = pp[d * (ATT_HD + 2) + 1]; }
        __syncthreads();
        for (int s = 0; s < n; ++s) m = fmaxf(m, pm[s]);
        if (d < n) pc[d] = pm[d] == -INFINITY ? 0.0f : expf(pm[d] - m);      // an unused partial carries m = -inf, l = 0, acc = 0
        __syncthreads();
#pragma unroll 4
        for (int s = 0; s < n; ++s) {
            l = fmaf(pl[s], pc[s], l);
            acc = fmaf(pp[s * (ATT_HD + 2) + 2 + d], pc[s], acc);
        }
    } else {
        for (int s = 0; s < n; ++s) m = fmaxf(m, pp[s * (ATT_HD + 2)]);
        for (int s = 0; s < n; ++s) {
            const float ms = pp[s * (ATT_HD + 2)];
            if (ms == -INFINITY) continue;
            const float c = expf(ms - m);
            l = fmaf(pp[s * (ATT_HD + 2) + 1], c, l);
            acc = fmaf(pp[s * (ATT_HD + 2) + 2 + d], c, acc);
        }
    }
    const float att = bf16_round(acc / l);
    const size_t i = ((size_t) t * a.n_head + h) * ATT_HD + d;
    o[i] = g ? bf16_round(att * softplus_ln2(g[i])) : att;
}

}   // namespace nsl

using namespace nsl;

static int g_attn_invariant = 0;   // 1: the first pass always runs a block per caller split (see nsl_attn_batch_invariant)

template <typename K>
static void attn_smem_attr(K kernel, int bytes, bool* done) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (!done[dev & 15]) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        done[dev & 15] = true;
    }
}

static int attn_sm_count() {
    static int n[16];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!n[dev & 15]) cudaDeviceGetAttribute(&n[dev & 15], cudaDevAttrMultiProcessorCount, dev);
    return n[dev & 15] > 0 ? n[dev & 15] : 148;
}

template <int NT, int SRC>
static void launch_attn_flat(cudaStream_t s, int n_blocks, const AttnArgs& a, const float* q, const KvView& kv, const RowInfo* ri, float* part, int T) {
    static bool done[16];
    constexpr int SMEM = ATT_MMA_WARPS * 2 * ATT_SLOT;
    attn_smem_attr(attn_flat_mma_kernel<2, NT, SRC>, SMEM, done);
    launch(attn_flat_mma_kernel<2, NT, SRC>, dim3((unsigned) n_blocks), 32 * ATT_MMA_WARPS, (size_t) SMEM, s, a, q, kv, ri, part, T);
}

template <int NT, int SRC>
static void launch_attn_split(cudaStream_t s, const AttnArgs& a, const float* q, const KvView& kv, const RowInfo* ri, float* part, int T) {
    static bool done[16];
    constexpr int SMEM = ATT_MMA_WARPS * 2 * ATT_SLOT;
    attn_smem_attr(attn_split_mma_kernel<2, NT, SRC>, SMEM, done);
    launch(attn_split_mma_kernel<2, NT, SRC>, dim3((unsigned) a.n_splits, (unsigned) a.n_kv, (unsigned) T), 32 * ATT_MMA_WARPS, (size_t) SMEM, s,
           a, q, kv, ri, part);
}

extern "C" {

// on = 1: the first pass always runs one block per (caller split, KV head, row), so a row's keys are cut by its own position
// alone and its output is bit-identical whatever rows share the call.  0 (default): the balanced form where it applies, whose
// cuts (and with them the order of the f32 sums, within the same bound) depend on all rows of the step.
void nsl_attn_batch_invariant(int on) { g_attn_invariant = on != 0; }

void kc_attn(cudaStream_t s, AttnArgs a, const float* q, KvView kv, const RowInfo* ri, float* part, const float* g, float* o, int T) {
    if (T < 1) return;
    if (kv.fmt != KV_BF16 && kv.fmt != KV_Q8) {
        set_error("kc_attn: KV cache format %d is not served by this library (BF16 = %d and Q8 = %d only)", kv.fmt, (int) KV_BF16, (int) KV_Q8);
        return;
    }
    const bool q8 = kv.fmt == KV_Q8;
    const int group = a.n_kv > 0 ? a.n_head / a.n_kv : 0;
    if (a.n_kv < 1 || a.n_head % a.n_kv || group < 1 || group > ATT_MAX_GROUP || a.n_splits < 1 || a.chunk < 0 || (a.chunk == 0 && a.n_splits > 1) || !aligned16(q) ||
        !aligned16(kv.a.k) || !aligned16(kv.a.v) || (kv.b.k && (!aligned16(kv.b.k) || !aligned16(kv.b.v))) ||
        (q8 && (!kv.a.ks || !kv.a.vs || (kv.b.k && (!kv.b.ks || !kv.b.vs))))) {
        set_error("kc_attn: %d query heads over %d KV heads (groups of 1..%d), %d splits of %d keys, unaligned buffers or an 8-bit cache without scales",
                  a.n_head, a.n_kv, (int) ATT_MAX_GROUP, a.n_splits, a.chunk);
        return;
    }
    const bool flat = !g_attn_invariant && a.n_splits >= 3 && a.chunk > 0 && T <= ATT_MAX_ROWS;
    int n_blocks = 0;
    if (flat) {
        n_blocks = 3 * attn_sm_count();      // three blocks with two-slot rings (70 KB of shared memory) fit an SM
        if (q8 && group <= 8) launch_attn_flat<1, ATT_SRC_Q8>(s, n_blocks, a, q, kv, ri, part, T);
        else if (q8) launch_attn_flat<2, ATT_SRC_Q8>(s, n_blocks, a, q, kv, ri, part, T);
        else if (group <= 8) launch_attn_flat<1, ATT_SRC_ASYNC>(s, n_blocks, a, q, kv, ri, part, T);
        else launch_attn_flat<2, ATT_SRC_ASYNC>(s, n_blocks, a, q, kv, ri, part, T);
    } else {
        if (q8 && group <= 8) launch_attn_split<1, ATT_SRC_Q8>(s, a, q, kv, ri, part, T);
        else if (q8) launch_attn_split<2, ATT_SRC_Q8>(s, a, q, kv, ri, part, T);
        else if (group <= 8) launch_attn_split<1, ATT_SRC_ASYNC>(s, a, q, kv, ri, part, T);
        else launch_attn_split<2, ATT_SRC_ASYNC>(s, a, q, kv, ri, part, T);
    }
    PdlScope chain(true);      // the reduction's blocks come in while the first pass drains
    launch(attn_reduce_kernel, dim3((unsigned) a.n_head, (unsigned) T), ATT_HD, 0, s, a, (const float*) part, g, o, ri, T, n_blocks);
    count_launch(2);
}

}   // extern "C"
