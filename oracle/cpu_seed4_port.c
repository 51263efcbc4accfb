/* The timed CPU baseline: a gcc restatement of the reference's P=4 CPU seed mat-vec.  TEST/BENCH INFRASTRUCTURE ONLY.
 *
 * The reference's kernel (nslm/lib_cpu_seed4.c) is written with Clang vector extensions and does not compile with
 * gcc (the reference itself links an aborting stub for gcc, CMakeLists.txt:74-86), so this file restates it with gcc
 * vector types: 16 rows per step (rows16, nslm/lib_cpu_seed4.c:39-74), a scalar form for left-over rows (rows1,
 * :76-101), per-block input sums (:103-109) and worker threads that claim 64-row chunks (:136-164).  The arithmetic
 * per block, in this order (fused multiply-adds exactly where the reference calls fma16 / __builtin_fmaf):
 *   v_k   = as_float(0x3F800000 | state_k << 7)               (= 1 + state_k / 2^16)
 *   a_p   = fma(x_c, v_(4c+p+1), a_p)   c = 0..7 ascending
 *   d     = (((a0 q0 + a1 q1) + a2 q2) + a3 q3) - (1.5 (((q0+q1)+q2)+q3)) xs_b
 *   acc   = fma(d, 2^(bias+16+code) R32, acc)
 * The vector path and the scalar path give the same bits (checked by tests), as the reference's do
 * (tests/test_cpu_seed4.c:63). */
#define _GNU_SOURCE
#include <pthread.h>
#include <stdatomic.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "nslm_oracle.h"

#define LANES 16
typedef float vf __attribute__((vector_size(4 * LANES)));
typedef uint32_t vu __attribute__((vector_size(4 * LANES)));
typedef int32_t vi __attribute__((vector_size(4 * LANES)));

#define CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))

static inline __attribute__((always_inline)) vf vfma(vf a, vf b, vf c) {
    vf r;
    for (int i = 0; i < LANES; ++i) r[i] = __builtin_fmaf(a[i], b[i], c[i]);
    return r;
}

static inline __attribute__((always_inline)) vf state_float(vu lo, vu hi, int k) {
    /* state k = bits k..k+15 of the 48-bit window; lo holds bits 0..31, hi bits 16..47 */
    const vu src = k <= 16 ? lo >> k : hi >> (k - 16);
    const vu bits = ((src << 7) & 0x007FFF80u) | 0x3F800000u;
    return (vf) bits;
}

CLONES static void rows_vec(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                            const uint32_t* table, const float* x, const float* xs, int kb, int r, float* y) {
    const float r32 = 1.0f / 32767.0f;
    vf acc = {0};
    for (int b = 0; b < kb; ++b) {
        uint32_t sa[LANES], ta[LANES], ca[LANES], ea[LANES];   // gathered into arrays, then loaded as vectors
        for (int i = 0; i < LANES; ++i) {
            const size_t g = (size_t) (r + i) * kb + b;
            sa[i] = seeds[g];
            ta[i] = table[seeds[g]];
            ca[i] = coefs[g];
            ea[i] = (codes[g >> 1] >> ((g & 1) * 4)) & 15u;
        }
        vu s, t, cw, code;
        memcpy(&s, sa, sizeof s);
        memcpy(&t, ta, sizeof t);
        memcpy(&cw, ca, sizeof cw);
        memcpy(&code, ea, sizeof code);
        const vu lo = s | (t << 16);
        vf a0 = {0}, a1 = {0}, a2 = {0}, a3 = {0};
        for (int c = 0; c < 8; ++c) {
            const float xv = x[8 * b + c];
            vf xc;
            for (int i = 0; i < LANES; ++i) xc[i] = xv;
            a0 = vfma(xc, state_float(lo, t, 4 * c + 1), a0);
            a1 = vfma(xc, state_float(lo, t, 4 * c + 2), a1);
            a2 = vfma(xc, state_float(lo, t, 4 * c + 3), a2);
            a3 = vfma(xc, state_float(lo, t, 4 * c + 4), a3);
        }
        const vi ci = (vi) cw;
        const vf q0 = __builtin_convertvector((ci << 28) >> 28, vf), q1 = __builtin_convertvector((ci << 24) >> 28, vf);
        const vf q2 = __builtin_convertvector((ci << 20) >> 28, vf), q3 = __builtin_convertvector((ci << 16) >> 28, vf);
        const vf qs = 1.5f * (((q0 + q1) + q2) + q3);
        const vu ebits = (code + (uint32_t) (bias + 16 + 127)) << 23;
        const vf sc = (vf) ebits * r32;
        const vf d = (((a0 * q0 + a1 * q1) + a2 * q2) + a3 * q3) - qs * xs[b];
        acc = vfma(d, sc, acc);
    }
    memcpy(y + r, &acc, sizeof acc);
}

static void row_scalar(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                       const uint32_t* table, const float* x, const float* xs, int kb, int r, float* y) {
    const float r32 = 1.0f / 32767.0f;
    float acc = 0.0f;
    for (int b = 0; b < kb; ++b) {
        const size_t g = (size_t) r * kb + b;
        const uint32_t s = seeds[g], t = table[s], lo = s | (t << 16), cw = coefs[g];
        const uint32_t code = (codes[g >> 1] >> ((g & 1) * 4)) & 15u;
        float a[4] = {0, 0, 0, 0};
        for (int c = 0; c < 8; ++c)
            for (int p = 0; p < 4; ++p) {
                const int k = 4 * c + p + 1;
                const uint32_t src = k <= 16 ? lo >> k : t >> (k - 16);
                const uint32_t bits = ((src << 7) & 0x007FFF80u) | 0x3F800000u;
                float v;
                memcpy(&v, &bits, 4);
                a[p] = __builtin_fmaf(x[8 * b + c], v, a[p]);
            }
        const float q0 = (float) ((int32_t) (cw << 28) >> 28), q1 = (float) ((int32_t) (cw << 24) >> 28);
        const float q2 = (float) ((int32_t) (cw << 20) >> 28), q3 = (float) ((int32_t) (cw << 16) >> 28);
        const float qs = 1.5f * (((q0 + q1) + q2) + q3);
        const float d = (((a[0] * q0 + a[1] * q1) + a[2] * q2) + a[3] * q3) - qs * xs[b];
        const uint32_t ebits = (code + (uint32_t) (bias + 16 + 127)) << 23;
        float p2;
        memcpy(&p2, &ebits, 4);
        acc = __builtin_fmaf(d, p2 * r32, acc);
    }
    y[r] = acc;
}

static void input_sums(const float* x, int kb, float* xs) {
    for (int b = 0; b < kb; ++b) {
        float s = 0.0f;
        for (int c = 0; c < 8; ++c) s += x[8 * b + c];
        xs[b] = s;
    }
}

typedef struct {
    const uint16_t *seeds, *coefs;
    const uint8_t* codes;
    int bias, kb, rows;
    const uint32_t* table;
    const float *x, *xs;
    float* y;
    atomic_int next;
} Task;

static void row_range(const Task* j, int r0, int r1) {
    int r = r0;
    for (; r + LANES <= r1; r += LANES) rows_vec(j->seeds, j->coefs, j->codes, j->bias, j->table, j->x, j->xs, j->kb, r, j->y);
    for (; r < r1; ++r) row_scalar(j->seeds, j->coefs, j->codes, j->bias, j->table, j->x, j->xs, j->kb, r, j->y);
}

static void* claim_rows(void* arg) {
    Task* j = (Task*) arg;
    for (;;) {
        const int r0 = atomic_fetch_add(&j->next, 64);
        if (r0 >= j->rows) return NULL;
        row_range(j, r0, r0 + 64 < j->rows ? r0 + 64 : j->rows);
    }
}

void orc_cpu_seed4_matvec_mt(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                             const uint32_t* table, const float* x, int rows, int kb, float* y, int threads) {
    float* xs = (float*) malloc(sizeof(float) * (size_t) kb);
    input_sums(x, kb, xs);
    Task j = {seeds, coefs, codes, bias, kb, rows, table, x, xs, y, 0};
    if (threads <= 1) claim_rows(&j);
    else {
        pthread_t* th = (pthread_t*) malloc(sizeof(pthread_t) * (size_t) (threads - 1));
        for (int i = 0; i < threads - 1; ++i) pthread_create(&th[i], NULL, claim_rows, &j);
        claim_rows(&j);
        for (int i = 0; i < threads - 1; ++i) pthread_join(th[i], NULL);
        free(th);
    }
    free(xs);
}

void orc_cpu_seed4_matvec_scalar(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                                 const uint32_t* table, const float* x, int rows, int kb, float* y) {
    float* xs = (float*) malloc(sizeof(float) * (size_t) kb);
    input_sums(x, kb, xs);
    for (int r = 0; r < rows; ++r) row_scalar(seeds, coefs, codes, bias, table, x, xs, kb, r, y);
    free(xs);
}

/* Best of `reps` after one warm-up call, CLOCK_MONOTONIC (the reference bench's protocol,
 * harness/nslm-cpu-seed-bench.c:57-66). */
double orc_cpu_seed4_time(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                          const float* x, int rows, int kb, float* y, int threads, int reps) {
    static uint32_t* table;
    if (!table) {
        table = (uint32_t*) malloc(sizeof(uint32_t) * 65536);
        orc_table32(table);
    }
    orc_cpu_seed4_matvec_mt(seeds, coefs, codes, bias, table, x, rows, kb, y, threads);
    double best = 1e30;
    for (int i = 0; i < reps; ++i) {
        struct timespec a, b;
        clock_gettime(CLOCK_MONOTONIC, &a);
        orc_cpu_seed4_matvec_mt(seeds, coefs, codes, bias, table, x, rows, kb, y, threads);
        clock_gettime(CLOCK_MONOTONIC, &b);
        const double dt = (double) (b.tv_sec - a.tv_sec) + 1e-9 * (double) (b.tv_nsec - a.tv_nsec);
        if (dt < best) best = dt;
    }
    return best;
}
