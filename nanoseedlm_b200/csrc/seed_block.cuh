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
// AND per state:
//   Y_c  = the window shifted so that stream bit 4c+1 sits at bit 4            (one shift per weight)
//   v_cp = as_float(Y_c & (0xFFFF << (4+p))) = state_(4c+p+1) * 2^(p-145)      (one AND with a literal; a subnormal float)
// FP32 subnormals are exact multiples of 2^-149 and this GPU's FMA takes them at full rate, so no exponent has to be
// merged in (a second constant per logic operation costs a second instruction or a register move).  The mat-vec
// kernels scale their inputs by 2^64 when they load them, so every product is a normal number; the powers of two and
// the centring (-32768 per state) fold into per-block constants.  The window is held as two words, A = stream bits
// 0..31 (weights 0..3) and G = stream bits 16..47 (weights 4..7), so no shift crosses a word.
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

// Run-time constants of the coefficient and exponent-code conversions (kernel arguments, so that they stay register
// or constant-bank operands).  Coefficient p becomes an exact float by placing nibble ^ 8 under an exponent chosen so
// that the nibble's low bit has the wanted weight, then subtracting the offset:
//   dot form   q'_p = q_p 2^(65-p):  exponent field 215 - 5p, offset 2^(88-5p) + 2^(68-p)
//   exact form q"_p = q_p 2^(100-p): exponent field 250 - 5p, offset 2^(123-5p) + 2^(103-p)
struct KConst {
    uint32_t cxor[4];
    float coff[4];
    uint32_t cxor_x[4];
    float coff_x[4];
    uint32_t cor;       // 112 << 23: 2^(code - 15) from a code placed at bits 23..26
};
inline KConst kconst() {
    KConst k;
    for (int p = 0; p < 4; ++p) {
        k.cxor[p] = ((uint32_t) (215 - 5 * p) << 23) | (8u << (4 * p));
        k.coff[p] = -(ldexpf(1.0f, 88 - 5 * p) + ldexpf(1.0f, 68 - p));
        k.cxor_x[p] = ((uint32_t) (250 - 5 * p) << 23) | (8u << (4 * p));
        k.coff_x[p] = -(ldexpf(1.0f, 123 - 5 * p) + ldexpf(1.0f, 103 - p));
    }
    k.cor = 112u << 23;
    return k;
}
#define NSL_XSCALE 18446744073709551616.0f   // 2^64: the mat-vec kernels' input scaling

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

// The same on two words at once, the results packed as a 64-bit pair {lo, hi}: written as one unit so the assembler
// places each result directly in its half of the pair (packing two separately produced values costs a move each).
template <uint32_t MASK>
__device__ __forceinline__ unsigned long long and_or_pair(uint32_t a0, uint32_t a1, uint32_t c) {
    unsigned long long d;
    asm("{\n\t.reg .b32 lo, hi;\n\tlop3.b32 lo, %1, %3, %4, 0xEA;\n\tlop3.b32 hi, %2, %3, %4, 0xEA;\n\tmov.b64 %0, {lo, hi};\n\t}"
        : "=l"(d) : "r"(a0), "r"(a1), "n"(MASK), "r"(c));
    return d;
}
template <uint32_t MASK>
__device__ __forceinline__ unsigned long long and_xor_pair(uint32_t a0, uint32_t a1, uint32_t c) {
    unsigned long long d;
    asm("{\n\t.reg .b32 lo, hi;\n\tlop3.b32 lo, %1, %3, %4, 0x6A;\n\tlop3.b32 hi, %2, %3, %4, 0x6A;\n\tmov.b64 %0, {lo, hi};\n\t}"
        : "=l"(d) : "r"(a0), "r"(a1), "n"(MASK), "r"(c));
    return d;
}

// The shifted copy for weight c: stream bit 4c+1 at bit 4.  a = stream bits 0..31, g = bits 16..47.
template <int C>
__device__ __forceinline__ uint32_t weight_word(uint32_t a, uint32_t g) {
    const uint32_t src = C < 4 ? a : g;
    constexpr int cc = C & 3;
    return cc == 0 ? src * 8u : src >> (4 * cc - 3);   // the left shift as a multiply: it issues on the FMA pipe
}
// v_cp = state_(4c+p+1) * 2^(p-145), a subnormal
template <int P>
__device__ __forceinline__ float state_value(uint32_t y) {
    return __uint_as_float(y & (0xFFFFu << (4 + P)));
}
// Coefficient p before the subtraction of its offset.  cw holds the coefficient word in bits 0..15 (higher bits are
// ignored).
template <int P>
__device__ __forceinline__ float coef_raw(uint32_t cw, uint32_t cx) {
    return __uint_as_float(and_xor<(0xFu << (4 * P))>(cw, cx));
}
// 2^(code - 15) for block i (0..7) of a chunk whose eight codes are the nibbles of cd.
__device__ __forceinline__ float code_scale(uint32_t cd, int i, const KConst& k) {   // i: a constant after unrolling
    const int sh = 23 - 4 * i;
    const uint32_t f = sh >= 0 ? cd * (1u << (sh & 31)) : cd >> ((-sh) & 31);
    return __uint_as_float(and_or<0x07800000u>(f, k.cor));
}
// {2^(code - 15) of block 2 bp, of block 2 bp + 1} of the chunk.
__device__ __forceinline__ unsigned long long code_scale_pair(uint32_t cd, int bp, const KConst& k) {
    const int s0 = 23 - 8 * bp, s1 = 19 - 8 * bp;
    const uint32_t f0 = s0 >= 0 ? cd * (1u << (s0 & 31)) : cd >> ((-s0) & 31);
    const uint32_t f1 = s1 >= 0 ? cd * (1u << (s1 & 31)) : cd >> ((-s1) & 31);
    return and_or_pair<0x07800000u>(f0, f1, k.cor);
}
// The factor that completes code_scale: R32 * 2^(eb + 31) (a power-of-two scaling of R32: exact).
__device__ __forceinline__ float slice_scale(int eb) {
    return __uint_as_float(__float_as_uint(1.0f / 32767.0f) + ((uint32_t) (eb + 31) << 23));
}

// Input-side constants of one block of SCALED inputs x' = 2^64 x: xm[p] = -32768 * 2^(p-145) * sum(x') =
// -2^(p-130) sum(x'), which centres the states.  The sum is taken on the unscaled values' order of magnitude by the
// caller passing the scaled inputs; 2^-66 etc. keep every factor a normal number.
__device__ __forceinline__ void block_offsets(const float* xs, float* xm) {   // xs: the 8 scaled inputs
    const float s = (((xs[0] + xs[4]) + (xs[1] + xs[5])) + ((xs[2] + xs[6]) + (xs[3] + xs[7]))) * 5.421010862427522e-20f;   // 2^-64
    xm[0] = -1.3552527156068805e-20f * s;   // -2^-66
    xm[1] = -2.710505431213761e-20f * s;    // -2^-65
    xm[2] = -5.421010862427522e-20f * s;    // -2^-64
    xm[3] = -1.0842021724855044e-19f * s;   // -2^-63
}

// ---- single block (the any-shape mat-vec, the decode, the GEMM tiles) -----------------------------------------------
// The 32 state values: v[4c+p].
__device__ __forceinline__ void block_states(uint32_t a, uint32_t g, float* v) {
#define NSL_V(C)                                      \
    {                                                 \
        const uint32_t y = weight_word<C>(a, g);      \
        v[4 * C + 0] = state_value<0>(y);             \
        v[4 * C + 1] = state_value<1>(y);             \
        v[4 * C + 2] = state_value<2>(y);             \
        v[4 * C + 3] = state_value<3>(y);             \
    }
    NSL_V(0) NSL_V(1) NSL_V(2) NSL_V(3) NSL_V(4) NSL_V(5) NSL_V(6) NSL_V(7)
#undef NSL_V
}
__device__ __forceinline__ void block_coefs(uint32_t cw, const KConst& k, float* q) {   // q'_p = q_p 2^(65-p)
    q[0] = coef_raw<0>(cw, k.cxor[0]) + k.coff[0];
    q[1] = coef_raw<1>(cw, k.cxor[1]) + k.coff[1];
    q[2] = coef_raw<2>(cw, k.cxor[2]) + k.coff[2];
    q[3] = coef_raw<3>(cw, k.cxor[3]) + k.coff[3];
}
// Dot form: sum_c x_c isum_c / 2^16 from scaled inputs.  d_p = xm_p + sum_c x'_c v_cp (c ascending);
// result = ((q'0 d0 + q'1 d1) + q'2 d2) + q'3 d3
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
// Exact form: the eight weights bit for bit.  With q"_p = q_p 2^(100-p) every product q"_p v_cp is the integer
// q_p state in units of 2^-45 and every partial sum is exact in f32; adding kq = -2^-30 sum_p q_p (the centring)
// leaves isum_c 2^-45 exactly, and one multiply by sc45 = fl(R32 2^e) * 2^45 is the spec's single rounding.
__device__ __forceinline__ void block_weights(uint32_t a, uint32_t g, uint32_t cw, float sc45, const KConst& k, float* w) {
    float v[32], q[4];
    block_states(a, g, v);
    q[0] = coef_raw<0>(cw, k.cxor_x[0]) + k.coff_x[0];
    q[1] = coef_raw<1>(cw, k.cxor_x[1]) + k.coff_x[1];
    q[2] = coef_raw<2>(cw, k.cxor_x[2]) + k.coff_x[2];
    q[3] = coef_raw<3>(cw, k.cxor_x[3]) + k.coff_x[3];
    // -2^(p-130) q"_p = -2^-30 q_p; the four constants are subnormal or tiny but exact
    const float kq = __fmaf_rn(q[3], -5.877471754111438e-39f,
                               __fmaf_rn(q[2], -2.938735877055719e-39f,
                                         __fmaf_rn(q[1], -1.4693679385278594e-39f, __fmul_rn(q[0], -7.346839692639297e-40f))));
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float t = __fmaf_rn(q[3], v[4 * c + 3],
                                  __fmaf_rn(q[2], v[4 * c + 2], __fmaf_rn(q[1], v[4 * c + 1], __fmul_rn(q[0], v[4 * c]))));
        w[c] = __fmul_rn(__fadd_rn(t, kq), sc45);
    }
}
// fl(R32 2^e) * 2^45 from exponent bits.
__device__ __forceinline__ float exact_scale45(int e) {
    return __uint_as_float(__float_as_uint(1.0f / 32767.0f) + ((uint32_t) (e + 45) << 23));
}

// ---- P = 3 blocks (format SEED4: nslm/lfsr.h:82-124) ----------------------------------------------------------------------
// 24 states; weight c uses states 3c+1 .. 3c+3.  The nibble word holds the exponent code in bits 0-3 and coefficient p
// in bits 4p+4 .. 4p+7, i.e. where the P = 4 coefficient word holds coefficient p + 1: the same conversions apply with
// the constants of position p + 1, which leaves every product half as large as in the P = 4 forms; the callers
// fold the missing factor 2 into the block scale (an exponent increment: exact).
// The shifted copy for weight c: stream bit 3c+1 at bit 4.  a = stream bits 0..31, g = bits 16..47.
template <int C>
__device__ __forceinline__ uint32_t weight_word3(uint32_t a, uint32_t g) {
    if (C == 0) return a * 8u;
    if (C == 1) return a;
    if (C <= 4) return a >> (3 * C - 3);
    if (C == 5) return g * 16u;
    if (C == 6) return g * 2u;
    return g >> 2;
}
// The 24 state values v[3c+p] = state_(3c+p+1) * 2^(p-145).
__device__ __forceinline__ void block_states3(uint32_t a, uint32_t g, float* v) {
#define NSL_V3(C)                                     \
    {                                                 \
        const uint32_t y = weight_word3<C>(a, g);     \
        v[3 * C + 0] = state_value<0>(y);             \
        v[3 * C + 1] = state_value<1>(y);             \
        v[3 * C + 2] = state_value<2>(y);             \
    }
    NSL_V3(0) NSL_V3(1) NSL_V3(2) NSL_V3(3) NSL_V3(4) NSL_V3(5) NSL_V3(6) NSL_V3(7)
#undef NSL_V3
}
__device__ __forceinline__ void block_coefs3(uint32_t nib, const KConst& k, float* q) {   // q'_p = q_p 2^(64-p)
    q[0] = coef_raw<1>(nib, k.cxor[1]) + k.coff[1];
    q[1] = coef_raw<2>(nib, k.cxor[2]) + k.coff[2];
    q[2] = coef_raw<3>(nib, k.cxor[3]) + k.coff[3];
}
// sum_c x_c isum_c / 2^17 from scaled inputs (xm from block_offsets: its first three entries).
__device__ __forceinline__ float states_dot3(const float* v, const float* q, const float* x, const float* xm) {
    float d0 = xm[0], d1 = xm[1], d2 = xm[2];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        d0 = fmaf(x[c], v[3 * c + 0], d0);
        d1 = fmaf(x[c], v[3 * c + 1], d1);
        d2 = fmaf(x[c], v[3 * c + 2], d2);
    }
    return fmaf(q[2], d2, fmaf(q[1], d1, q[0] * d0));
}
// The eight weights bit for bit: q"_p = q_p 2^(99-p), products in units of 2^-46, sc46 = fl(R32 2^e) * 2^46.
__device__ __forceinline__ void block_weights3(uint32_t a, uint32_t g, uint32_t nib, float sc46, const KConst& k, float* w) {
    float q[3];
    q[0] = coef_raw<1>(nib, k.cxor_x[1]) + k.coff_x[1];
    q[1] = coef_raw<2>(nib, k.cxor_x[2]) + k.coff_x[2];
    q[2] = coef_raw<3>(nib, k.cxor_x[3]) + k.coff_x[3];
    const float kq = __fmaf_rn(q[2], -2.938735877055719e-39f, __fmaf_rn(q[1], -1.4693679385278594e-39f, __fmul_rn(q[0], -7.346839692639297e-40f)));
    // weight by weight: its shift and three ANDs, then its arithmetic, so that the two pipes alternate in program order
#define NSL_WX3(C)                                                                                                                        \
    {                                                                                                                                     \
        const uint32_t y = weight_word3<C>(a, g);                                                                                         \
        const float t = __fmaf_rn(q[2], state_value<2>(y), __fmaf_rn(q[1], state_value<1>(y), __fmul_rn(q[0], state_value<0>(y))));      \
        w[C] = __fmul_rn(__fadd_rn(t, kq), sc46);                                                                                         \
    }
    NSL_WX3(0) NSL_WX3(1) NSL_WX3(2) NSL_WX3(3) NSL_WX3(4) NSL_WX3(5) NSL_WX3(6) NSL_WX3(7)
#undef NSL_WX3
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

// t[idx] for a table in shared memory with the address formed by a multiply-add whose factor 4 comes from constant
// memory, so that it stays a multiply-add: it issues on the FMA pipe, where the logic pipe is the one that binds
// (measured on config 1: 115.4 -> 113.9 us per step; doing the right shifts as high products the same way lost 1 %).
static __constant__ uint32_t nsl_four = 4u;
__device__ __forceinline__ uint32_t lut_word(const uint32_t* t, uint32_t idx) {
    uint32_t addr, v;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(addr) : "r"(idx), "r"(nsl_four), "r"((unsigned) __cvta_generic_to_shared(t)));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// The 32 state-value pairs of the blocks whose seeds are the two halves of sw: v[4c+p] = {even, odd}.
__device__ __forceinline__ void pair_states(const StreamTab& tab, uint32_t sw, u64* v) {
    // table indices and the two windows by byte permutes: one logic-pipe operation each
    const uint32_t g0 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4440)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4441));
    const uint32_t g1 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4442)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4443));
    const uint32_t a0 = __byte_perm(sw, g0, 0x5410), a1 = __byte_perm(sw, g1, 0x5432);
#define NSL_V2(C)                                                                  \
    {                                                                              \
        const uint32_t y0 = weight_word<C>(a0, g0), y1 = weight_word<C>(a1, g1);   \
        v[4 * C + 0] = pack2(state_value<0>(y0), state_value<0>(y1));              \
        v[4 * C + 1] = pack2(state_value<1>(y0), state_value<1>(y1));              \
        v[4 * C + 2] = pack2(state_value<2>(y0), state_value<2>(y1));              \
        v[4 * C + 3] = pack2(state_value<3>(y0), state_value<3>(y1));              \
    }
    NSL_V2(0) NSL_V2(1) NSL_V2(2) NSL_V2(3) NSL_V2(4) NSL_V2(5) NSL_V2(6) NSL_V2(7)
#undef NSL_V2
}
// The four coefficient pairs of the two words packed in cw.
__device__ __forceinline__ void pair_coefs(uint32_t cw, const KConst& k, u64* q) {
    const uint32_t c1 = cw >> 16;
    q[0] = add2(and_xor_pair<0x000Fu>(cw, c1, k.cxor[0]), pack2(k.coff[0], k.coff[0]));
    q[1] = add2(and_xor_pair<0x00F0u>(cw, c1, k.cxor[1]), pack2(k.coff[1], k.coff[1]));
    q[2] = add2(and_xor_pair<0x0F00u>(cw, c1, k.cxor[2]), pack2(k.coff[2], k.coff[2]));
    q[3] = add2(and_xor_pair<0xF000u>(cw, c1, k.cxor[3]), pack2(k.coff[3], k.coff[3]));
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

// pair_states + pair_dot written weight by weight: the two shifts and eight ANDs of weight c, then its four packed
// multiply-adds, so that logic-pipe and FMA-pipe instructions alternate in program order.  Same operations, same order
// per accumulator: the same bits.  Measured on the config-1 step at 8 rows: 112.9 us against 114.2 us with all 32 state
// values formed first (by halves, 16 at a time: 114.2; gate and up side by side per weight: 114.4).
__device__ __forceinline__ u64 pair_expand_dot(const StreamTab& tab, uint32_t sw, const u64* q, const u64* x2, const u64* xm2) {
    const uint32_t g0 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4440)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4441));
    const uint32_t g1 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4442)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4443));
    const uint32_t a0 = __byte_perm(sw, g0, 0x5410), a1 = __byte_perm(sw, g1, 0x5432);
    u64 d0 = xm2[0], d1 = xm2[1], d2 = xm2[2], d3 = xm2[3];
#define NSL_W2(C)                                                                  \
    {                                                                              \
        const uint32_t y0 = weight_word<C>(a0, g0), y1 = weight_word<C>(a1, g1);   \
        d0 = fma2(x2[C], pack2(state_value<0>(y0), state_value<0>(y1)), d0);       \
        d1 = fma2(x2[C], pack2(state_value<1>(y0), state_value<1>(y1)), d1);       \
        d2 = fma2(x2[C], pack2(state_value<2>(y0), state_value<2>(y1)), d2);       \
        d3 = fma2(x2[C], pack2(state_value<3>(y0), state_value<3>(y1)), d3);       \
    }
    NSL_W2(0) NSL_W2(1) NSL_W2(2) NSL_W2(3) NSL_W2(4) NSL_W2(5) NSL_W2(6) NSL_W2(7)
#undef NSL_W2
    return fma2(q[3], d3, fma2(q[2], d2, fma2(q[1], d1, mul2(q[0], d0))));
}

// The same for two adjacent P = 3 blocks (see block_states3 / block_coefs3 / states_dot3): 24 state-value pairs, the three
// coefficient pairs of the two nibble words packed in nw, and {2^(code - 15) of the even block, of the odd block} from the
// words' low nibbles.
__device__ __forceinline__ void pair_coefs3(uint32_t nw, const KConst& k, u64* q) {
    const uint32_t n1 = nw >> 16;
    q[0] = add2(and_xor_pair<0x00F0u>(nw, n1, k.cxor[1]), pack2(k.coff[1], k.coff[1]));
    q[1] = add2(and_xor_pair<0x0F00u>(nw, n1, k.cxor[2]), pack2(k.coff[2], k.coff[2]));
    q[2] = add2(and_xor_pair<0xF000u>(nw, n1, k.cxor[3]), pack2(k.coff[3], k.coff[3]));
}
// The P = 3 form of pair_expand_dot: 24 state-value pairs, weight by weight; d_p = xm_p + sum_c x_c v_cp (c ascending),
// result = (q0 d0 + q1 d1) + q2 d2.
__device__ __forceinline__ u64 pair_expand_dot3(const StreamTab& tab, uint32_t sw, const u64* q, const u64* x2, const u64* xm2) {
    const uint32_t g0 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4440)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4441));
    const uint32_t g1 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4442)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4443));
    const uint32_t a0 = __byte_perm(sw, g0, 0x5410), a1 = __byte_perm(sw, g1, 0x5432);
    u64 d0 = xm2[0], d1 = xm2[1], d2 = xm2[2];
#define NSL_W23(C)                                                                   \
    {                                                                                \
        const uint32_t y0 = weight_word3<C>(a0, g0), y1 = weight_word3<C>(a1, g1);   \
        d0 = fma2(x2[C], pack2(state_value<0>(y0), state_value<0>(y1)), d0);         \
        d1 = fma2(x2[C], pack2(state_value<1>(y0), state_value<1>(y1)), d1);         \
        d2 = fma2(x2[C], pack2(state_value<2>(y0), state_value<2>(y1)), d2);         \
    }
    NSL_W23(0) NSL_W23(1) NSL_W23(2) NSL_W23(3) NSL_W23(4) NSL_W23(5) NSL_W23(6) NSL_W23(7)
#undef NSL_W23
    return fma2(q[2], d2, fma2(q[1], d1, mul2(q[0], d0)));
}
__device__ __forceinline__ u64 code_scale_pair3(uint32_t nw, const KConst& k) {
    return and_or_pair<0x07800000u>(nw * (1u << 23), nw * (1u << 7), k.cor);      // bits 0-3 and 16-19 to bits 23-26
}

// Exact form for two adjacent blocks at once (the GEMM's weight tiles): w2[c] = {weight c of the even block, of the odd
// block}, bit for bit as block_weights gives them.  sc2 = {exact_scale45 of the even block, of the odd block}.
__device__ __forceinline__ void pair_weights(const StreamTab& tab, uint32_t sw, uint32_t cw, u64 sc2, const KConst& k, u64* w2) {
    u64 q[4];
    const uint32_t g0 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4440)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4441));
    const uint32_t g1 = lut_word(tab.lo, __byte_perm(sw, 0, 0x4442)) ^ lut_word(tab.hi, __byte_perm(sw, 0, 0x4443));
    const uint32_t a0 = __byte_perm(sw, g0, 0x5410), a1 = __byte_perm(sw, g1, 0x5432);
    const uint32_t c1 = cw >> 16;
    q[0] = add2(and_xor_pair<0x000Fu>(cw, c1, k.cxor_x[0]), pack2(k.coff_x[0], k.coff_x[0]));
    q[1] = add2(and_xor_pair<0x00F0u>(cw, c1, k.cxor_x[1]), pack2(k.coff_x[1], k.coff_x[1]));
    q[2] = add2(and_xor_pair<0x0F00u>(cw, c1, k.cxor_x[2]), pack2(k.coff_x[2], k.coff_x[2]));
    q[3] = add2(and_xor_pair<0xF000u>(cw, c1, k.cxor_x[3]), pack2(k.coff_x[3], k.coff_x[3]));
    const u64 kq = fma2(q[3], pack2(-5.877471754111438e-39f, -5.877471754111438e-39f),
                        fma2(q[2], pack2(-2.938735877055719e-39f, -2.938735877055719e-39f),
                             fma2(q[1], pack2(-1.4693679385278594e-39f, -1.4693679385278594e-39f),
                                  mul2(q[0], pack2(-7.346839692639297e-40f, -7.346839692639297e-40f)))));
    // weight by weight (its shifts and ANDs, then its multiply-adds: the two pipes alternate in program order); the centring
    // term first: every partial sum stays an exact integer multiple of 2^-45 below 2^24
#define NSL_WX(C)                                                                                               \
    {                                                                                                           \
        const uint32_t y0 = weight_word<C>(a0, g0), y1 = weight_word<C>(a1, g1);                                \
        w2[C] = mul2(fma2(q[3], pack2(state_value<3>(y0), state_value<3>(y1)),                                  \
                          fma2(q[2], pack2(state_value<2>(y0), state_value<2>(y1)),                             \
                               fma2(q[1], pack2(state_value<1>(y0), state_value<1>(y1)),                        \
                                    fma2(q[0], pack2(state_value<0>(y0), state_value<0>(y1)), kq)))), sc2);     \
    }
    NSL_WX(0) NSL_WX(1) NSL_WX(2) NSL_WX(3) NSL_WX(4) NSL_WX(5) NSL_WX(6) NSL_WX(7)
#undef NSL_WX
}
// Two f32 -> one word of two bf16 (round to nearest even), low half = a.
__device__ __forceinline__ uint32_t bf16x2_bits(float a, float b) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
    return d;
}

}   // namespace nsl
