// Device primitives for SEED4P4 blocks on sm_100a: the LFSR stream table in shared memory and the per-block
// expansion, in the forms the kernels use.
//
// Format facts (reference: nslm/lfsr.h:6-10,52-59; nslm/search4.h:1-31; nslm/lib_rows.c:56-73): a block is 8 weights
// = a 16-bit seed + a coefficient word (four int4 q_p, two's complement, bits 4p..4p+3) + a 4-bit exponent code;
// state k (k = 1..32) is bits k..k+15 of the 48-bit window seed | G[seed] << 16 where G is the 32-bit stream table;
// weight c = fl((float) isum_c * fl(R32 2^e)), isum_c = sum_p (state_(4c+p+1) - 32768) q_p.
//
// How the expansion is laid out here.  On this part the integer/logic pipe issues at half the FP32 rate (measured:
// 63 LOP3/SHF/PRMT vs 119 FFMA lane-ops per clock per SM) and packed FP32 pairs (fma.rn.f32x2) halve the FP issue
// count again, so a block costs what its integer operations cost.  They are kept to one shift per weight and one
// logic operation per state:
//   Y_c  = the window shifted so that stream bit 4c+1 sits at bit 4            (one shift per weight)
//   v_cp = as_float((Y_c & (0xFFFF << (4+p))) | (130-p) << 23) = 2^(3-p) + state_(4c+p+1) / 2^16     (one LOP3, exact)
// The offsets 8, 4, 2, 1 and the centring (-32768 = -0.5 in these units) fold into per-block constants.  The window
// is held as two words, A = stream bits 0..31 (weights 0..3) and G = stream bits 16..47 (weights 4..7), so no shift
// crosses a word.  The second constant of every two-constant logic operation comes from a register that the compiler
// cannot see through (KConst, passed as a kernel argument): with two literals the assembler emits two instructions.
// Two adjacent blocks are expanded side by side and their state values packed as f32x2 pairs {block A, block B}, so
// the 32 multiply-adds of each block issue as 32 packed operations per block pair.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsl {

typedef unsigned long long u64;

struct StreamTab {
    uint32_t lo[256];   // G[s] for s = 0..255
    uint32_t hi[256];   // G[s << 8]
};

// G is linear over GF(2) (reference: tests/test_lfsr.c:87-93): G[s] = G[s & 0xFF] ^ G[s & 0xFF00], so 512 entries of
// the caller's 65536-entry table are all a kernel needs.
__device__ __forceinline__ void load_stream_tab(StreamTab& t, const uint32_t* __restrict__ G, int tid, int nthreads) {
    for (int i = tid; i < 256; i += nthreads) {
        t.lo[i] = __ldg(G + i);
        t.hi[i] = __ldg(G + (i << 8));
    }
}

__device__ __forceinline__ uint32_t stream_bits(const StreamTab& t, uint32_t seed) {
    return t.lo[seed & 0xFFu] ^ t.hi[(seed >> 8) & 0xFFu];
}

// Run-time constants of the expansion (see the header comment).  Filled by kconst() on the host.
struct KConst {
    uint32_t expo[4];   // (130 - p) << 23
    uint32_t cxor[4];   // (150 - 4p) << 23 | 8 << 4p
    uint32_t cor;       // 112 << 23
    float coff[4];      // -(2^(23 - 4p) + 8)
};
inline KConst kconst() {
    KConst k;
    for (int p = 0; p < 4; ++p) {
        k.expo[p] = (uint32_t) (130 - p) << 23;
        k.cxor[p] = ((uint32_t) (150 - 4 * p) << 23) | (8u << (4 * p));
        k.coff[p] = -((float) (1u << (23 - 4 * p)) + 8.0f);
    }
    k.cor = 112u << 23;
    return k;
}

__device__ __forceinline__ float bf16_round(float x) {   // round to nearest even, kept as f32 (nslm/lfsr.h:104-109)
    uint32_t u = __float_as_uint(x);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return __uint_as_float(u & 0xFFFF0000u);
}
__device__ __forceinline__ uint16_t bf16_bits(float x) {
    uint32_t u = __float_as_uint(x);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t) (u >> 16);
}

// (a & MASK) | c and (a & MASK) ^ c as single LOP3s: MASK a literal, c a register.
template <uint32_t MASK>
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "n"(MASK), "r"(c));
    return d;
}
template <uint32_t MASK>
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "n"(MASK), "r"(c));
    return d;
}

// The shifted copy for weight c: stream bit 4c+1 at bit 4.  a = stream bits 0..31, g = bits 16..47.
template <int C>
__device__ __forceinline__ uint32_t weight_word(uint32_t a, uint32_t g) {
    const uint32_t src = C < 4 ? a : g;
    constexpr int cc = C & 3;
    return cc == 0 ? src * 8u : src >> (4 * cc - 3);   // the left shift as a multiply: it issues on the FMA pipe
}
// v_cp = 2^(3-p) + state / 2^16
template <int P>
__device__ __forceinline__ float state_value(uint32_t y, const KConst& k) {
    return __uint_as_float(and_or<(0xFFFFu << (4 + P))>(y, k.expo[P]));
}
// Coefficient p as an exact float: nibble ^ 8 under a power of two chosen so the nibble's low bit weighs 1, before the
// subtraction of coff[p].  cw holds the coefficient word in bits 0..15 (higher bits are ignored).
template <int P>
__device__ __forceinline__ float coef_raw(uint32_t cw, const KConst& k) {
    return __uint_as_float(and_xor<(0xFu << (4 * P))>(cw, k.cxor[P]));
}
// 2^(code - 15) for block i (0..7) of a chunk whose eight codes are the nibbles of cd.
__device__ __forceinline__ float code_scale(uint32_t cd, int i, const KConst& k) {   // i: a constant after unrolling
    const int sh = 23 - 4 * i;
    const uint32_t f = sh >= 0 ? cd * (1u << (sh & 31)) : cd >> ((-sh) & 31);
    return __uint_as_float(and_or<0x07800000u>(f, k.cor));
}
// The factor that completes code_scale: R32 * 2^(eb + 31) (a power-of-two scaling of R32: exact).
__device__ __forceinline__ float slice_scale(int eb) {
    return __uint_as_float(__float_as_uint(1.0f / 32767.0f) + ((uint32_t) (eb + 31) << 23));
}

// Input-side constants of one block: xm[p] = -(2^(3-p) + 0.5) * sum(x), which centres the states.
__device__ __forceinline__ void block_offsets(const float* x, float* xm) {
    const float s = ((x[0] + x[4]) + (x[1] + x[5])) + ((x[2] + x[6]) + (x[3] + x[7]));
    xm[0] = -8.5f * s;
    xm[1] = -4.5f * s;
    xm[2] = -2.5f * s;
    xm[3] = -1.5f * s;
}

// ---- single block (the any-shape mat-vec, the decode, the GEMM tiles) -----------------------------------------------
// The 32 state values: v[4c+p].
__device__ __forceinline__ void block_states(uint32_t a, uint32_t g, const KConst& k, float* v) {
#define NSL_V(C)                                         \
    {                                                    \
        const uint32_t y = weight_word<C>(a, g);         \
        v[4 * C + 0] = state_value<0>(y, k);             \
        v[4 * C + 1] = state_value<1>(y, k);             \
        v[4 * C + 2] = state_value<2>(y, k);             \
        v[4 * C + 3] = state_value<3>(y, k);             \
    }
    NSL_V(0) NSL_V(1) NSL_V(2) NSL_V(3) NSL_V(4) NSL_V(5) NSL_V(6) NSL_V(7)
#undef NSL_V
}
__device__ __forceinline__ void block_coefs(uint32_t cw, const KConst& k, float* q) {
    q[0] = coef_raw<0>(cw, k) + k.coff[0];
    q[1] = coef_raw<1>(cw, k) + k.coff[1];
    q[2] = coef_raw<2>(cw, k) + k.coff[2];
    q[3] = coef_raw<3>(cw, k) + k.coff[3];
}
// Dot form: sum_c x_c isum_c / 2^16.  d_p = xm_p + sum_c x_c v_cp (c ascending); result = ((q0 d0 + q1 d1) + q2 d2) + q3 d3
__device__ __forceinline__ float states_dot(const float* v, const float* q, const float* x, const float* xm) {
    float d0 = xm[0], d1 = xm[1], d2 = xm[2], d3 = xm[3];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        d0 = fmaf(x[c], v[4 * c + 0], d0);
        d1 = fmaf(x[c], v[4 * c + 1], d1);
        d2 = fmaf(x[c], v[4 * c + 2], d2);
        d3 = fmaf(x[c], v[4 * c + 3], d3);
    }
    return fmaf(q[3], d3, fmaf(q[2], d2, fmaf(q[1], d1, q[0] * d0)));
}
// Exact form: the eight weights bit for bit.  sum_p q_p v_cp stays below 2^8 in units of 2^-16, so every partial sum is
// exact in f32; adding kq = -sum_p q_p (2^(3-p) + 0.5) leaves isum_c / 2^16 exactly, and one multiply by
// sc16 = fl(R32 2^e) * 2^16 is the spec's single rounding.
__device__ __forceinline__ void block_weights(uint32_t a, uint32_t g, uint32_t cw, float sc16, const KConst& k, float* w) {
    float v[32], q[4];
    block_states(a, g, k, v);
    block_coefs(cw, k, q);
    const float kq = __fmaf_rn(q[3], -1.5f, __fmaf_rn(q[2], -2.5f, __fmaf_rn(q[1], -4.5f, __fmul_rn(q[0], -8.5f))));
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float t = __fmaf_rn(q[3], v[4 * c + 3],
                                  __fmaf_rn(q[2], v[4 * c + 2], __fmaf_rn(q[1], v[4 * c + 1], __fmul_rn(q[0], v[4 * c]))));
        w[c] = __fmul_rn(__fadd_rn(t, kq), sc16);
    }
}
// fl(R32 2^e) * 2^16 from exponent bits.
__device__ __forceinline__ float exact_scale16(int e) {
    return __uint_as_float(__float_as_uint(1.0f / 32767.0f) + ((uint32_t) (e + 16) << 23));
}

// ---- two adjacent blocks as f32x2 pairs {even block, odd block} ----------------------------------------------------
__device__ __forceinline__ u64 pack2(float lo, float hi) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
    u64 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
    u64 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
    u64 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// The 32 state-value pairs of the blocks whose seeds are the two halves of sw: v[4c+p] = {even, odd}.
__device__ __forceinline__ void pair_states(const StreamTab& tab, uint32_t sw, const KConst& k, u64* v) {
    const uint32_t s0 = sw & 0xFFFFu, s1 = sw >> 16;
    const uint32_t g0 = stream_bits(tab, s0), g1 = stream_bits(tab, s1);
    const uint32_t a0 = g0 * 65536u + s0, a1 = g1 * 65536u + s1;
#define NSL_V2(C)                                                                  \
    {                                                                              \
        const uint32_t y0 = weight_word<C>(a0, g0), y1 = weight_word<C>(a1, g1);   \
        v[4 * C + 0] = pack2(state_value<0>(y0, k), state_value<0>(y1, k));        \
        v[4 * C + 1] = pack2(state_value<1>(y0, k), state_value<1>(y1, k));        \
        v[4 * C + 2] = pack2(state_value<2>(y0, k), state_value<2>(y1, k));        \
        v[4 * C + 3] = pack2(state_value<3>(y0, k), state_value<3>(y1, k));        \
    }
    NSL_V2(0) NSL_V2(1) NSL_V2(2) NSL_V2(3) NSL_V2(4) NSL_V2(5) NSL_V2(6) NSL_V2(7)
#undef NSL_V2
}
// The four coefficient pairs of the two words packed in cw.
__device__ __forceinline__ void pair_coefs(uint32_t cw, const KConst& k, u64* q) {
    const uint32_t c1 = cw >> 16;
    q[0] = add2(pack2(coef_raw<0>(cw, k), coef_raw<0>(c1, k)), pack2(k.coff[0], k.coff[0]));
    q[1] = add2(pack2(coef_raw<1>(cw, k), coef_raw<1>(c1, k)), pack2(k.coff[1], k.coff[1]));
    q[2] = add2(pack2(coef_raw<2>(cw, k), coef_raw<2>(c1, k)), pack2(k.coff[2], k.coff[2]));
    q[3] = add2(pack2(coef_raw<3>(cw, k), coef_raw<3>(c1, k)), pack2(k.coff[3], k.coff[3]));
}
// Both blocks' dot forms at once: x2[c] = {x of the even block, x of the odd block}, xm2[p] likewise.
__device__ __forceinline__ u64 pair_dot(const u64* v, const u64* q, const u64* x2, const u64* xm2) {
    u64 d0 = xm2[0], d1 = xm2[1], d2 = xm2[2], d3 = xm2[3];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        d0 = fma2(x2[c], v[4 * c + 0], d0);
        d1 = fma2(x2[c], v[4 * c + 1], d1);
        d2 = fma2(x2[c], v[4 * c + 2], d2);
        d3 = fma2(x2[c], v[4 * c + 3], d3);
    }
    return fma2(q[3], d3, fma2(q[2], d2, fma2(q[1], d1, mul2(q[0], d0))));
}

}   // namespace nsl
