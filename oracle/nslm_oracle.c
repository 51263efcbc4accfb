/* CPU oracle for the seed-decode matmul path -- see nslm_oracle.h.  TEST INFRASTRUCTURE ONLY.
 * Build with -ffp-contract=off (the reference builds its C without contraction, CMakeLists.txt:7-8,49); the places
 * where the reference uses an explicit fused multiply-add call fmaf()/fma() by name. */
#include "nslm_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------------------------------
 * LFSR: 16-bit Fibonacci register, taps 0,1,3,12, shift right, feedback into bit 15 (nslm/lfsr.h:20-23).
 * The seed is state 0; the block uses the states that FOLLOW it (nslm/lfsr.h:6-7, 26-28). */
uint16_t orc_lfsr_step(uint16_t s) {
    unsigned fb = (s ^ (s >> 1) ^ (s >> 3) ^ (s >> 12)) & 1u;
    return (uint16_t) ((s >> 1) | (fb << 15));
}

void orc_lfsr_states(uint16_t s, int n, uint16_t* out) {
    for (int i = 0; i < n; ++i) {
        s = orc_lfsr_step(s);
        out[i] = s;
    }
}

/* The 32 stream bits that follow the seed: bit k is the top bit of state k+1 (nslm/lfsr.h:52-59).  With
 * window = seed | stream32 << 16, state k is bits k..k+15 of the window (nslm/lib_rows.c:59,71). */
uint32_t orc_stream32(uint16_t s) {
    uint32_t g = 0;
    for (int k = 0; k < 32; ++k) {
        s = orc_lfsr_step(s);
        g |= (uint32_t) (s >> 15) << k;
    }
    return g;
}

void orc_table32(uint32_t* table) {
    for (uint32_t s = 0; s < 65536; ++s) table[s] = orc_stream32((uint16_t) s);
}

/* FNV-1a over the first 24 states of every seed 1..65535: the reference's format lock (tests/test_lfsr.c:41-56). */
uint64_t orc_fnv24_all_seeds(void) {
    uint64_t h = 1469598103934665603ull;
    for (uint32_t s = 1; s <= 65535; ++s) {
        uint16_t st[24];
        orc_lfsr_states((uint16_t) s, 24, st);
        for (int k = 0; k < 24; ++k) h = (h ^ st[k]) * 1099511628211ull;
    }
    return h;
}

/* Cycle length from state 1 (tests/test_lfsr.c:15-22 expects 65535). */
int orc_period(void) {
    uint16_t s = 1;
    int n = 0;
    do {
        s = orc_lfsr_step(s);
        ++n;
    } while (s != 1 && n < 70000);
    return n;
}

/* ------------------------------------------------------------------------------------------------------------------
 * Scalar helpers. */
static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* bf16 round-to-nearest-even of a finite f32 (nslm/lfsr.h:104-109). */
uint16_t orc_f2bf(float f) {
    uint32_t u = f2u(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t) (u >> 16);
}
float orc_bf2f(uint16_t h) { return u2f((uint32_t) h << 16); }
float orc_bfr(float f) { return orc_bf2f(orc_f2bf(f)); }

/* fl(R32 * 2^e), R32 = fl(1/32767): the power of two comes from exponent bits (nslm/lfsr.h:97-102). */
float orc_scale(int e) {
    const float r32 = 1.0f / 32767.0f;
    return r32 * u2f((uint32_t) (e + 127) << 23);
}

/* Coefficient p: two's-complement int4 in bits 4p..4p+3 of the word (nslm/search4.h:27). */
int orc_q4(uint16_t coef, int p) {
    int v = (coef >> (4 * p)) & 15;
    return v >= 8 ? v - 16 : v;
}

/* ------------------------------------------------------------------------------------------------------------------
 * P=4 block: weight c = fl( (float) isum_c * fl(R32 2^e) ), isum_c = sum_p (state_(4c+p+1) - 32768) q_p, an exact
 * integer (nslm/search4.h:4-6; nslm/lib_search4.c:22-31; f32 form nslm/lib_rows.c:66-73). */
static void block_isum(uint16_t seed, uint16_t coef, int32_t isum[8]) {
    uint16_t st[32];
    orc_lfsr_states(seed, 32, st);
    int q[4];
    for (int p = 0; p < 4; ++p) q[p] = orc_q4(coef, p);
    for (int c = 0; c < 8; ++c) {
        int32_t v = 0;
        for (int p = 0; p < 4; ++p) v += ((int32_t) st[4 * c + p] - 32768) * q[p];
        isum[c] = v;
    }
}

void orc_decode_block_f32(uint16_t seed, uint16_t coef, int e, float out[8]) {
    int32_t isum[8];
    block_isum(seed, coef, isum);
    const float sc = orc_scale(e);
    for (int c = 0; c < 8; ++c) out[c] = (float) isum[c] * sc;
}

void orc_decode_block_bf16(uint16_t seed, uint16_t coef, int e, uint16_t out[8]) {
    float w[8];
    orc_decode_block_f32(seed, coef, e, w);
    for (int c = 0; c < 8; ++c) out[c] = orc_f2bf(w[c]);
}

/* Exponent code of global block g of a slice: nibble g&1 of byte g>>1, low nibble = even block
 * (nslm/cpu_seed4.h:4-5; nslm/lib_rows.c:62). */
static int block_code(const uint8_t* codes, size_t g) { return (codes[g >> 1] >> ((g & 1) * 4)) & 15; }

void orc_decode_rows_f32(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K,
                         float* out) {
    const int nb = K / 8;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const size_t g = (size_t) r * nb + b;
            orc_decode_block_f32(seeds[g], coefs[g], eb + block_code(codes, g), out + g * 8);
        }
}

void orc_decode_rows_bf16(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K,
                          uint16_t* out) {
    const int nb = K / 8;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const size_t g = (size_t) r * nb + b;
            orc_decode_block_bf16(seeds[g], coefs[g], eb + block_code(codes, g), out + g * 8);
        }
}

/* ------------------------------------------------------------------------------------------------------------------
 * Mat-vec in double over the exact f32 weights: the form the reference's tests and CPU forwards use
 * (tests/test_cpu_seed4.c:14-24; nslm/lib_qwen4_ref.c:46-60; tests/test_mova_kernels.c:196-200). */
void orc_matvec_f64(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K,
                    const float* x, int xs, int T, double* y, int ys, double* mag) {
    const int nb = K / 8;
    for (int r = 0; r < rows; ++r) {
        for (int t = 0; t < T; ++t) {
            y[(size_t) t * ys + r] = 0;
            if (mag) mag[(size_t) t * ys + r] = 0;
        }
        for (int b = 0; b < nb; ++b) {
            const size_t g = (size_t) r * nb + b;
            float w[8];
            orc_decode_block_f32(seeds[g], coefs[g], eb + block_code(codes, g), w);
            for (int t = 0; t < T; ++t) {
                const float* xb = x + (size_t) t * xs + 8 * b;
                double a = 0, m = 0;
                for (int c = 0; c < 8; ++c) {
                    const double v = (double) w[c] * (double) xb[c];
                    a += v;
                    m += fabs(v);
                }
                y[(size_t) t * ys + r] += a;
                if (mag) mag[(size_t) t * ys + r] += m;
            }
        }
    }
}

/* The engines' output rounding: y = bf16(acc), or residual y = bf16(y + bf16(acc))
 * (engine/kernels_moe.cu:214; nslm/lib_mova_ref.c:76-80). */
void orc_mv(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K, const float* x,
            int xs, int T, int add, float* y, int ys) {
    double* acc = (double*) malloc(sizeof(double) * (size_t) T * rows);
    orc_matvec_f64(seeds, coefs, codes, eb, rows, K, x, xs, T, acc, rows, NULL);
    for (int t = 0; t < T; ++t)
        for (int r = 0; r < rows; ++r) {
            float* yo = y + (size_t) t * ys + r;
            const float a = orc_bfr((float) acc[(size_t) t * rows + r]);
            *yo = add ? orc_bfr(*yo + a) : a;
        }
    free(acc);
}

/* silu on a bf16 tensor, each op rounded: bf16(g * bf16(1/(1+exp(-g)))) (engine/kernels_moe.cu:28-31). */
float orc_silu_bf(float g) {
    const float s = orc_bfr(1.0f / (1.0f + expf(-g)));
    return orc_bfr(g * s);
}

/* Fused gate+up: a = bf16(silu_bf(bf16 g) * bf16 u) (engine/kernels_moe.cu:338-348). */
void orc_mv_gu(const uint16_t* gs, const uint16_t* gc, const uint8_t* ge, int geb, const uint16_t* us, const uint16_t* uc,
               const uint8_t* ue, int ueb, int rows, int K, const float* x, float* a) {
    double* g = (double*) malloc(sizeof(double) * (size_t) rows * 2);
    double* u = g + rows;
    orc_matvec_f64(gs, gc, ge, geb, rows, K, x, K, 1, g, rows, NULL);
    orc_matvec_f64(us, uc, ue, ueb, rows, K, x, K, 1, u, rows, NULL);
    for (int r = 0; r < rows; ++r) a[r] = orc_bfr(orc_silu_bf(orc_bfr((float) g[r])) * orc_bfr((float) u[r]));
    free(g);
}

/* a = bf16(silu_bf(g) * u) on already rounded g, u (engine/kernels_moe.cu:775-778). */
void orc_swiglu(const float* g, const float* u, float* a, int n) {
    for (int i = 0; i < n; ++i) a[i] = orc_bfr(orc_silu_bf(g[i]) * u[i]);
}

/* ------------------------------------------------------------------------------------------------------------------
 * Router: softmax over all E with the max subtracted, the k largest, equal scores to the HIGHER index, output best
 * first, weights renormalised over the k picked (nslm/lib_qwen4_ops.c:106-122). */
void orc_route(const float* logits, int E, int k, int32_t* ind, float* wt) {
    double* pr = (double*) malloc(sizeof(double) * (size_t) E);
    char* taken = (char*) calloc((size_t) E, 1);
    double mx = -INFINITY, top = 0;
    for (int e = 0; e < E; ++e)
        if (logits[e] > mx) mx = logits[e];
    for (int e = 0; e < E; ++e) pr[e] = exp((double) logits[e] - mx);
    for (int j = 0; j < k; ++j) {
        int best = -1;
        for (int e = 0; e < E; ++e) {
            if (taken[e]) continue;
            if (best < 0 || pr[e] > pr[best] || (pr[e] == pr[best] && e > best)) best = e;
        }
        taken[best] = 1;
        ind[j] = best;
        top += pr[best];
    }
    for (int j = 0; j < k; ++j) wt[j] = (float) (pr[ind[j]] / top);
    free(pr);
    free(taken);
}

static float sigm_f(float x) { return 1.0f / (1.0f + expf(-x)); }

/* MoVA router of one row (nslm/lib_mova_ref.c:171-201): logit = bf16(dot over the first hw inputs) + bf16(dot over the
 * rest), both sums in double over BF16 weights; score = f32 sigmoid; selection score = score + bf16 bias; the k largest
 * selection scores with equal ones to the LOWEST id, best first; weight = score / sum of the picked scores * scale. */
void orc_mova_topk(const float* score, const float* sel, int n, int k, float scale, int32_t* inds, float* wts) {
    float* se = (float*) malloc(sizeof(float) * (size_t) n);
    memcpy(se, sel, sizeof(float) * (size_t) n);
    float sum = 0;
    for (int j = 0; j < k; ++j) {
        int best = -1;
        for (int e = 0; e < n; ++e)
            if (se[e] != -INFINITY && (best < 0 || se[e] > se[best])) best = e;
        inds[j] = best;
        sum += score[best];
        se[best] = -INFINITY;
    }
    for (int j = 0; j < k; ++j) wts[j] = score[inds[j]] / sum * scale;
    free(se);
}

void orc_mova_router(int d, int hw, int n, int k, float scale, const uint16_t* W, const uint16_t* bias, const float* x,
                     float* score, float* sel, int32_t* inds, float* wts) {
    for (int e = 0; e < n; ++e) {
        double s0 = 0, s1 = 0;
        for (int c = 0; c < d; ++c) {
            const double v = (double) orc_bf2f(W[(size_t) e * d + c]) * x[c];
            if (c < hw) s0 += v; else s1 += v;
        }
        score[e] = 1.0f / (1.0f + expf(-(orc_bfr((float) s0) + orc_bfr((float) s1))));
        sel[e] = score[e] + orc_bf2f(bias[e]);
    }
    orc_mova_topk(score, sel, n, k, scale, inds, wts);
}

/* The gate of the per-head maps: softplus with beta = ln 2 in f32, then BF16 (engine/kernels_moe.cu:215-218). */
float orc_softplus_gate(float g) {
    const float gx = g * 0.69314718055994531f;
    return orc_bfr((fmaxf(gx, 0.0f) + logf(1.0f + expf(-fabsf(gx)))) / 0.69314718055994531f);
}

/* out[t] = sigmoid(sg[t*sgld]) sh[t] + sum_j wt[t][j] D[t*k+j], plain f32, j ascending
 * (engine/kernels_qwen4.cu:506-512). */
void orc_q4_moe_combine(int d, int k, const float* D, const float* wt, const float* sh, const float* sg, int sgld,
                        float* out, int T) {
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < d; ++i) {
            float a = sigm_f(sg[(size_t) t * sgld]) * sh[(size_t) t * d + i];
            for (int j = 0; j < k; ++j) a += wt[t * k + j] * D[((size_t) t * k + j) * d + i];
            out[(size_t) t * d + i] = a;
        }
}

/* x = bf16(x + bf16(bf16(sum_j bf16(D_j bf16(w_j))) + shared)) (engine/kernels_moe.cu:779-788). */
void orc_moe_combine(const float* D, const float* w, const float* shared, float* x, int d, int k, int T) {
    for (int t = 0; t < T; ++t)
        for (int c = 0; c < d; ++c) {
            float s = 0;
            for (int j = 0; j < k; ++j) s += orc_bfr(D[((size_t) t * k + j) * d + c] * orc_bfr(w[t * k + j]));
            const size_t i = (size_t) t * d + c;
            x[i] = orc_bfr(x[i] + orc_bfr(orc_bfr(s) + shared[i]));
        }
}

/* ------------------------------------------------------------------------------------------------------------------
 * Grouping: pairs sorted by expert, ascending pair id within an expert; runs of <= bn pairs become tiles
 * (engine/kernels_moe.cu:527-573; host form tests/test_qwen4_engine.c:50-56). */
int orc_bucket(const int32_t* inds, int count, int n, int bn, int32_t* perm, OrcTile* tiles) {
    int at = 0, nt = 0;
    for (int e = 0; e < n; ++e) {
        const int start = at;
        for (int i = 0; i < count; ++i)
            if (inds[i] == e) perm[at++] = i;
        for (int s = start; s < at; s += bn) {
            OrcTile t = {e, s, at - s < bn ? at - s : bn, 0};
            tiles[nt++] = t;
        }
    }
    return nt;
}

/* Grouped prompt GEMM, per pair: y[p][r] = bf16(sum_c wv x[p/xdiv][c]); the default mode rounds seed weights to
 * bf16 first, the exact mode keeps f32 (engine/kernels_moe.cu:405-412; tests/test_mova_kernels.c:286-300). */
void orc_mm_pairs(const uint16_t* const* seeds, const uint16_t* const* coefs, const uint8_t* const* codes, const int32_t* eb,
                  const int32_t* slice_of_pair, int P, int xdiv, int rows, int K, const float* x, int xs, int exact,
                  float* y, int ys) {
    const int nb = K / 8;
    float* w = (float*) malloc(sizeof(float) * (size_t) K);
    for (int p = 0; p < P; ++p) {
        const int s = slice_of_pair[p];
        const float* xp = x + (size_t) (p / xdiv) * xs;
        for (int r = 0; r < rows; ++r) {
            for (int b = 0; b < nb; ++b) {
                const size_t g = (size_t) r * nb + b;
                orc_decode_block_f32(seeds[s][g], coefs[s][g], eb[s] + block_code(codes[s], g), w + 8 * b);
            }
            double acc = 0;
            for (int c = 0; c < K; ++c) acc += (double) (exact ? w[c] : orc_bfr(w[c])) * (double) xp[c];
            y[(size_t) p * ys + r] = orc_bfr((float) acc);
        }
    }
    free(w);
}

/* ------------------------------------------------------------------------------------------------------------------
 * One MoE layer as the CPU reference forward computes it: route, then per picked expert
 * y = down(silu(gate x) * up x) with double sums stored as f32 and no bf16 rounding, out += wt * y
 * (nslm/lib_qwen4_ref.c:177-207; silu/sigmoid in double, :27-28).  No shared expert here (added by the caller). */
static void lin_f64(const uint16_t* s, const uint16_t* c, const uint8_t* e, int eb, int rows, int K, const float* x,
                    float* y) {
    double* acc = (double*) malloc(sizeof(double) * (size_t) rows);
    orc_matvec_f64(s, c, e, eb, rows, K, x, K, 1, acc, rows, NULL);
    for (int r = 0; r < rows; ++r) y[r] = (float) acc[r];
    free(acc);
}

void orc_moe_layer(const OrcMoe* m, const float* x, const float* logits, int T, float* out, int32_t* ind_out,
                   float* wt_out) {
    const int d = m->d, ff = m->ff;
    const size_t gu_b = (size_t) ff * (d / 8), dn_b = (size_t) d * (ff / 8);
    float* g = (float*) malloc(sizeof(float) * (size_t) ff * 2);
    float* u = g + ff;
    float* y = (float*) malloc(sizeof(float) * (size_t) d);
    int32_t* ind = (int32_t*) malloc(sizeof(int32_t) * (size_t) m->k);
    float* wt = (float*) malloc(sizeof(float) * (size_t) m->k);
    for (int t = 0; t < T; ++t) {
        const float* xt = x + (size_t) t * d;
        float* ot = out + (size_t) t * d;
        orc_route(logits + (size_t) t * m->E, m->E, m->k, ind, wt);
        memset(ot, 0, sizeof(float) * (size_t) d);
        for (int j = 0; j < m->k; ++j) {
            const int e = ind[j];
            lin_f64(m->gs + e * gu_b, m->gc + e * gu_b, m->ge + e * (gu_b / 2), m->geb[e], ff, d, xt, g);
            lin_f64(m->us + e * gu_b, m->uc + e * gu_b, m->ue + e * (gu_b / 2), m->ueb[e], ff, d, xt, u);
            for (int i = 0; i < ff; ++i) g[i] = (float) ((double) g[i] / (1.0 + exp(-(double) g[i]))) * u[i];
            lin_f64(m->ds + e * dn_b, m->dc + e * dn_b, m->de + e * (dn_b / 2), m->deb[e], d, ff, g, y);
            for (int i = 0; i < d; ++i) ot[i] += wt[j] * y[i];
            if (ind_out) ind_out[t * m->k + j] = e;
            if (wt_out) wt_out[t * m->k + j] = wt[j];
        }
    }
    free(g);
    free(y);
    free(ind);
    free(wt);
}

/* ------------------------------------------------------------------------------------------------------------------
 * P = 3 blocks (format SEED4; nslm/lfsr.h:82-124, nslm/lib_rows.c:49-76): 8 weights = u16 seed + u16 nibble word whose
 * bits 0-3 are the exponent code and bits 4p+4..4p+7 the int4 coefficient q_p, p = 0..2; states 1..24 after the seed;
 * isum_c = sum_p (state_(3c+p+1) - 32768) q_p; weight = fl((float) isum_c * fl(R32 2^(bias + code))). */
static int q3(uint16_t nib, int p) {
    const int v = (nib >> (4 + 4 * p)) & 15;
    return v >= 8 ? v - 16 : v;
}
void orc_decode3_block_f32(uint16_t seed, uint16_t nib, int bias, float out[8]) {
    uint16_t st[24];
    orc_lfsr_states(seed, 24, st);
    const float sc = orc_scale(bias + (nib & 15));
    for (int c = 0; c < 8; ++c) {
        int32_t isum = 0;
        for (int p = 0; p < 3; ++p) isum += ((int32_t) st[3 * c + p] - 32768) * q3(nib, p);
        out[c] = (float) isum * sc;
    }
}
void orc_decode3_block_bf16(uint16_t seed, uint16_t nib, int bias, uint16_t out[8]) {
    float w[8];
    orc_decode3_block_f32(seed, nib, bias, w);
    for (int c = 0; c < 8; ++c) out[c] = orc_f2bf(w[c]);
}
void orc_decode3_rows_f32(const uint16_t* seeds, const uint16_t* nibs, int bias, int rows, int K, float* out) {
    const size_t nb = (size_t) rows * (K / 8);
    for (size_t g = 0; g < nb; ++g) orc_decode3_block_f32(seeds[g], nibs[g], bias, out + g * 8);
}

/* ------------------------------------------------------------------------------------------------------------------
 * The affine int4 dense mat-vec of the LM head, in the form the reference's kernel test states it
 * (tests/test_mova_kernels.c:146-157, 181-199): weight (r, c) = bf16 scale[(r K + c) / 64] * code + bf16 bias[same group],
 * code = bits 4 (i % 8) .. of word i / 8; y = bf16(sum in double), or with add bf16(y0 + bf16(sum)).  mag (optional) gets
 * sum |w x| per output for the f32-accumulation bound. */
void orc_q4_mv(const uint32_t* codes, const uint16_t* scales, const uint16_t* biases, int K, int R, const float* x, int T,
               int add, float* y, double* mag) {
    for (int t = 0; t < T; ++t)
        for (int r = 0; r < R; ++r) {
            double acc = 0, m = 0;
            for (int c = 0; c < K; ++c) {
                const size_t i = (size_t) r * K + c;
                const double w = (double) orc_bf2f(scales[i / 64]) * (double) ((codes[i / 8] >> (4 * (i % 8))) & 15u) +
                                 (double) orc_bf2f(biases[i / 64]);
                const double v = w * (double) x[(size_t) t * K + c];
                acc += v;
                m += fabs(v);
            }
            float* yo = y + (size_t) t * R + r;
            *yo = add ? orc_bfr(*yo + orc_bfr((float) acc)) : orc_bfr((float) acc);
            if (mag) mag[(size_t) t * R + r] = m;
        }
}

/* Greedy arg-max (ties: the lowest id) and the softmax probability of the winner (engine/kernels_moe.cu:2115-2151). */
void orc_argmax(const float* logits, int V, int32_t* out, double* prob) {
    int best = 0;
    for (int i = 1; i < V; ++i)
        if (logits[i] > logits[best]) best = i;
    double tot = 0;
    for (int i = 0; i < V; ++i) tot += exp((double) logits[i] - (double) logits[best]);
    *out = best;
    if (prob) *prob = 1.0 / tot;
}

/* ------------------------------------------------------------------------------------------------------------------
 * Seeded inputs: splitmix64 (the reference's nslm/rng.h:7-14 uses the same public generator), seeds in [1,65535],
 * coefficient words = 16 random bits (four int4 in [-8,7]), codes in [0,15] two per byte, low nibble first. */
uint64_t orc_splitmix64(uint64_t* state) {
    uint64_t z = (*state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

void orc_gen_matrix(uint64_t seed, int rows, int K, uint16_t* seeds, uint16_t* coefs, uint8_t* codes) {
    const size_t nb = (size_t) rows * (K / 8);
    uint64_t st = seed;
    for (size_t g = 0; g < nb; ++g) {
        const uint64_t r = orc_splitmix64(&st);
        seeds[g] = (uint16_t) (1 + (r & 0xFFFFFFFFull) % 65535);
        coefs[g] = (uint16_t) (r >> 32);
        const unsigned code = (unsigned) (r >> 48) & 15u;
        if (g & 1) codes[g >> 1] = (uint8_t) (codes[g >> 1] | (code << 4));
        else codes[g >> 1] = (uint8_t) code;
    }
}

void orc_gen_normal(uint64_t seed, size_t n, int round_bf16, float* out) {
    uint64_t st = seed ^ 0xA5A5A5A5DEADBEEFull;
    for (size_t i = 0; i < n; i += 2) {
        const double u1 = ((orc_splitmix64(&st) >> 11) + 1.0) * (1.0 / 9007199254740993.0);
        const double u2 = (orc_splitmix64(&st) >> 11) * (1.0 / 9007199254740992.0);
        const double rad = sqrt(-2.0 * log(u1)), ang = 6.283185307179586476925 * u2;
        const float a = (float) (rad * cos(ang)), b = (float) (rad * sin(ang));
        out[i] = round_bf16 ? orc_bfr(a) : a;
        if (i + 1 < n) out[i + 1] = round_bf16 ? orc_bfr(b) : b;
    }
}
