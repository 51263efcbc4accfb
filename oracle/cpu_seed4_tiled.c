/* The timed CPU baseline, tiled form: a gcc restatement of the reference's CPU-tiled P=4 seed mat-vec / mat-mul.
 * TEST/BENCH INFRASTRUCTURE ONLY.
 *
 * Layout (nslm/cpu_seed4.h:26-38, nslm/lib_cpu_seed4.c:171-190): rows in tiles of 16; inside a tile block b's 16 seeds
 * are contiguous, likewise its 16 coefficient words, and per pair of blocks 16 code bytes (block 2j in the low nibble):
 * vector loads instead of gathers.  A partial last tile is padded with seed 1 and zero coefficients.  kb must be even.
 * Arithmetic: one tile = the 16-row step of the row-major kernel (tile_rows, :214-253); for several tokens a block's 32
 * state values are made once and every token runs its own multiply-adds in the same order (tile_rows_n, :302-349), so
 * a token's rows equal a one-token call bit for bit (tests/test_cpu_seed4.c:70-93).  Threads claim 4 tiles at a time
 * (:262-281). */
#define _GNU_SOURCE
#include <pthread.h>
#include <stdatomic.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "nslm_oracle.h"

#define LANES 16
#define MAX_TOK 8
typedef float vf __attribute__((vector_size(4 * LANES)));
typedef uint32_t vu __attribute__((vector_size(4 * LANES)));
typedef int32_t vi __attribute__((vector_size(4 * LANES)));
typedef uint16_t vh __attribute__((vector_size(2 * LANES)));
typedef uint8_t vb __attribute__((vector_size(LANES)));

#define CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))

struct OrcTiled {
    uint16_t *seeds, *coefs;
    uint8_t* codes;
    int bias, rows, kb, tiles;
};

OrcTiled* orc_cpu_seed4_tile(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias, int rows, int kb) {
    if (kb & 1) return NULL;
    OrcTiled* t = (OrcTiled*) calloc(1, sizeof *t);
    const int tiles = (rows + LANES - 1) / LANES;
    t->seeds = (uint16_t*) malloc((size_t) tiles * kb * LANES * 2);
    t->coefs = (uint16_t*) calloc((size_t) tiles * kb * LANES, 2);
    t->codes = (uint8_t*) calloc((size_t) tiles * (kb / 2) * LANES, 1);
    t->bias = bias, t->rows = rows, t->kb = kb, t->tiles = tiles;
    for (int tile = 0; tile < tiles; ++tile)
        for (int b = 0; b < kb; ++b)
            for (int i = 0; i < LANES; ++i) {
                const int r = tile * LANES + i;
                const size_t o = ((size_t) tile * kb + b) * LANES + i;
                if (r >= rows) { t->seeds[o] = 1; continue; }
                const size_t g = (size_t) r * kb + b;
                t->seeds[o] = seeds[g];
                t->coefs[o] = coefs[g];
                const int code = (codes[g >> 1] >> ((g & 1) * 4)) & 15;
                t->codes[((size_t) tile * (kb / 2) + b / 2) * LANES + i] |= (uint8_t) (code << ((b & 1) * 4));
            }
    return t;
}

void orc_cpu_seed4_tiled_free(OrcTiled* t) {
    if (!t) return;
    free(t->seeds), free(t->coefs), free(t->codes), free(t);
}

static inline __attribute__((always_inline)) vf vfma(vf a, vf b, vf c) {
    vf r;
    for (int i = 0; i < LANES; ++i) r[i] = __builtin_fmaf(a[i], b[i], c[i]);
    return r;
}

static inline __attribute__((always_inline)) vf state_float(vu lo, vu hi, int k) {
    const vu src = k <= 16 ? lo >> k : hi >> (k - 16);
    return (vf) (((src << 7) & 0x007FFF80u) | 0x3F800000u);
}

static inline __attribute__((always_inline)) vf splat(float v) {
    vf r;
    for (int i = 0; i < LANES; ++i) r[i] = v;
    return r;
}

/* One block of one tile: the window halves, the four coefficients, 1.5 * their sum, the block's scale. */
typedef struct { vu lo, hi; vf q0, q1, q2, q3, qs, sc; } Blk;

static inline __attribute__((always_inline)) Blk load_block(const OrcTiled* m, int tile, int b, const uint32_t* table) {
    const uint16_t* sp = m->seeds + ((size_t) tile * m->kb + b) * LANES;
    vh s16, q16;
    vb c16;
    memcpy(&s16, sp, sizeof s16);
    memcpy(&q16, m->coefs + ((size_t) tile * m->kb + b) * LANES, sizeof q16);
    memcpy(&c16, m->codes + ((size_t) tile * (m->kb / 2) + b / 2) * LANES, sizeof c16);
    const vu s = __builtin_convertvector(s16, vu), q = __builtin_convertvector(q16, vu);
    const vu code = (__builtin_convertvector(c16, vu) >> ((b & 1) * 4)) & 15u;
    uint32_t ta[LANES];
    for (int i = 0; i < LANES; ++i) ta[i] = table[sp[i]];
    Blk k;
    memcpy(&k.hi, ta, sizeof k.hi);
    k.lo = s | (k.hi << 16);
    const vi qi = (vi) q;
    k.q0 = __builtin_convertvector((qi << 28) >> 28, vf), k.q1 = __builtin_convertvector((qi << 24) >> 28, vf);
    k.q2 = __builtin_convertvector((qi << 20) >> 28, vf), k.q3 = __builtin_convertvector((qi << 16) >> 28, vf);
    k.qs = 1.5f * (((k.q0 + k.q1) + k.q2) + k.q3);
    k.sc = (vf) ((code + (uint32_t) (m->bias + 16 + 127)) << 23) * (1.0f / 32767.0f);
    return k;
}

/* One token: no array of states. */
CLONES static void tile_one(const OrcTiled* m, int tile, const uint32_t* table, const float* x, const float* xs, float* out) {
    vf acc = {0};
    for (int b = 0; b < m->kb; ++b) {
        const Blk k = load_block(m, tile, b, table);
        vf a0 = {0}, a1 = {0}, a2 = {0}, a3 = {0};
        for (int c = 0; c < 8; ++c) {
            const vf xc = splat(x[8 * b + c]);
            a0 = vfma(xc, state_float(k.lo, k.hi, 4 * c + 1), a0);
            a1 = vfma(xc, state_float(k.lo, k.hi, 4 * c + 2), a1);
            a2 = vfma(xc, state_float(k.lo, k.hi, 4 * c + 3), a2);
            a3 = vfma(xc, state_float(k.lo, k.hi, 4 * c + 4), a3);
        }
        const vf d = (((a0 * k.q0 + a1 * k.q1) + a2 * k.q2) + a3 * k.q3) - k.qs * xs[b];
        acc = vfma(d, k.sc, acc);
    }
    memcpy(out, &acc, sizeof acc);
}

/* ntok tokens: a block's states once, then each token's sums in tile_one's order. */
CLONES static void tile_many(const OrcTiled* m, int tile, const uint32_t* table, const float* x, const float* xs, int ntok,
                             float* out) {
    vf acc[MAX_TOK];
    for (int t = 0; t < ntok; ++t) acc[t] = splat(0.0f);
    for (int b = 0; b < m->kb; ++b) {
        const Blk k = load_block(m, tile, b, table);
        vf v[32];
        for (int j = 0; j < 32; ++j) v[j] = state_float(k.lo, k.hi, j + 1);
        for (int t = 0; t < ntok; ++t) {
            const float* xb = x + (size_t) t * m->kb * 8 + 8 * b;
            vf a0 = {0}, a1 = {0}, a2 = {0}, a3 = {0};
            for (int c = 0; c < 8; ++c) {
                const vf xc = splat(xb[c]);
                a0 = vfma(xc, v[4 * c], a0);
                a1 = vfma(xc, v[4 * c + 1], a1);
                a2 = vfma(xc, v[4 * c + 2], a2);
                a3 = vfma(xc, v[4 * c + 3], a3);
            }
            const vf d = (((a0 * k.q0 + a1 * k.q1) + a2 * k.q2) + a3 * k.q3) - k.qs * xs[(size_t) t * m->kb + b];
            acc[t] = vfma(d, k.sc, acc[t]);
        }
    }
    for (int t = 0; t < ntok; ++t) memcpy(out + (size_t) t * LANES, &acc[t], sizeof acc[t]);
}

typedef struct {
    const OrcTiled* m;
    const uint32_t* table;
    const float *x, *xs;
    float* y;
    int ntok;
    atomic_int next;
} TileTask;

static void* claim_tiles(void* arg) {
    TileTask* j = (TileTask*) arg;
    float out[MAX_TOK * LANES];
    for (;;) {
        const int t0 = atomic_fetch_add(&j->next, 4);
        if (t0 >= j->m->tiles) return NULL;
        const int t1 = t0 + 4 < j->m->tiles ? t0 + 4 : j->m->tiles;
        for (int tile = t0; tile < t1; ++tile) {
            if (j->ntok == 1) tile_one(j->m, tile, j->table, j->x, j->xs, out);
            else tile_many(j->m, tile, j->table, j->x, j->xs, j->ntok, out);
            const int r0 = tile * LANES, n = j->m->rows - r0 < LANES ? j->m->rows - r0 : LANES;
            for (int t = 0; t < j->ntok; ++t)
                memcpy(j->y + (size_t) t * j->m->rows + r0, out + (size_t) t * LANES, sizeof(float) * (size_t) n);
        }
    }
}

/* x [ntok][kb * 8] -> y [ntok][rows], ntok <= 8 (nslm/lib_cpu_seed4.c:283-298, 423-442). */
int orc_cpu_seed4_tiled_matmul_mt(const OrcTiled* m, const uint32_t* table, const float* x, int ntok, float* y, int threads) {
    if (!m || ntok < 1 || ntok > MAX_TOK) return -1;
    float* xs = (float*) malloc(sizeof(float) * (size_t) ntok * m->kb);
    for (int t = 0; t < ntok; ++t)
        for (int b = 0; b < m->kb; ++b) {
            float s = 0.0f;
            for (int c = 0; c < 8; ++c) s += x[(size_t) t * m->kb * 8 + 8 * b + c];
            xs[(size_t) t * m->kb + b] = s;
        }
    TileTask j = {m, table, x, xs, y, ntok, 0};
    if (threads <= 1) claim_tiles(&j);
    else {
        pthread_t* th = (pthread_t*) malloc(sizeof(pthread_t) * (size_t) (threads - 1));
        for (int i = 0; i < threads - 1; ++i) pthread_create(&th[i], NULL, claim_tiles, &j);
        claim_tiles(&j);
        for (int i = 0; i < threads - 1; ++i) pthread_join(th[i], NULL);
        free(th);
    }
    free(xs);
    return 0;
}

/* Several independent products in one parallel region: what a host engine does for one MoE phase (every routed
 * expert's gate and up, then every down), so that small matrices still fill all threads.  Threads claim (job, 4 tiles)
 * units from one flat list; each unit runs the same tile code as above, so results equal the single calls bit for bit. */
typedef struct {
    const OrcTiledJob* jobs;
    const int* first;      /* unit index of each job's first chunk; first[njobs] = total */
    float* const* xs;
    int njobs;
    const uint32_t* table;
    atomic_int next;
} JobSet;

static void* claim_units(void* arg) {
    JobSet* s = (JobSet*) arg;
    float out[MAX_TOK * LANES];
    int j = 0;
    for (;;) {
        const int u = atomic_fetch_add(&s->next, 1);
        if (u >= s->first[s->njobs]) return NULL;
        while (u >= s->first[j + 1]) ++j;   /* units are claimed in ascending order per thread */
        const OrcTiledJob* job = &s->jobs[j];
        const OrcTiled* m = job->m;
        const int t0 = (u - s->first[j]) * 4, t1 = t0 + 4 < m->tiles ? t0 + 4 : m->tiles;
        for (int tile = t0; tile < t1; ++tile) {
            if (job->ntok == 1) tile_one(m, tile, s->table, job->x, s->xs[j], out);
            else tile_many(m, tile, s->table, job->x, s->xs[j], job->ntok, out);
            const int r0 = tile * LANES, n = m->rows - r0 < LANES ? m->rows - r0 : LANES;
            for (int t = 0; t < job->ntok; ++t)
                memcpy(job->y + (size_t) t * m->rows + r0, out + (size_t) t * LANES, sizeof(float) * (size_t) n);
        }
    }
}

int orc_cpu_seed4_tiled_jobs(const OrcTiledJob* jobs, int njobs, const uint32_t* table, int threads) {
    if (njobs <= 0) return 0;
    int* first = (int*) malloc(sizeof(int) * (size_t) (njobs + 1));
    float** xs = (float**) malloc(sizeof(float*) * (size_t) njobs);
    first[0] = 0;
    for (int j = 0; j < njobs; ++j) {
        const OrcTiled* m = jobs[j].m;
        if (!m || jobs[j].ntok < 1 || jobs[j].ntok > MAX_TOK) { free(first); free(xs); return -1; }
        first[j + 1] = first[j] + (m->tiles + 3) / 4;
        xs[j] = (float*) malloc(sizeof(float) * (size_t) jobs[j].ntok * m->kb);
        for (int t = 0; t < jobs[j].ntok; ++t)
            for (int b = 0; b < m->kb; ++b) {
                float sum = 0.0f;
                for (int c = 0; c < 8; ++c) sum += jobs[j].x[(size_t) t * m->kb * 8 + 8 * b + c];
                xs[j][(size_t) t * m->kb + b] = sum;
            }
    }
    JobSet s = {jobs, first, xs, njobs, table, 0};
    if (threads <= 1) claim_units(&s);
    else {
        pthread_t* th = (pthread_t*) malloc(sizeof(pthread_t) * (size_t) (threads - 1));
        for (int i = 0; i < threads - 1; ++i) pthread_create(&th[i], NULL, claim_units, &s);
        claim_units(&s);
        for (int i = 0; i < threads - 1; ++i) pthread_join(th[i], NULL);
        free(th);
    }
    for (int j = 0; j < njobs; ++j) free(xs[j]);
    free(first);
    free(xs);
    return 0;
}

/* Best of reps after one warm-up call, CLOCK_MONOTONIC (harness/nslm-cpu-seed-bench.c:57-66). */
double orc_cpu_seed4_tiled_time(const OrcTiled* m, const float* x, int ntok, float* y, int threads, int reps) {
    static uint32_t* table;
    if (!table) {
        table = (uint32_t*) malloc(sizeof(uint32_t) * 65536);
        orc_table32(table);
    }
    if (orc_cpu_seed4_tiled_matmul_mt(m, table, x, ntok, y, threads)) return -1.0;
    double best = 1e30;
    for (int i = 0; i < reps; ++i) {
        struct timespec a, b;
        clock_gettime(CLOCK_MONOTONIC, &a);
        orc_cpu_seed4_tiled_matmul_mt(m, table, x, ntok, y, threads);
        clock_gettime(CLOCK_MONOTONIC, &b);
        const double dt = (double) (b.tv_sec - a.tv_sec) + 1e-9 * (double) (b.tv_nsec - a.tv_nsec);
        if (dt < best) best = dt;
    }
    return best;
}
