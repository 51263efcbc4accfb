/* CPU oracle for the seed-decode matmul path.  TEST INFRASTRUCTURE ONLY: the checker that the CUDA kernels are
 * compared against (tests, the smoke check, the bench's cpu_baseline leg).  Nothing in the product library links,
 * calls or falls back to this code.
 *
 * Every function restates, in plain C, the arithmetic of the NanoSeedLM reference; the reference file:line each one
 * follows is given at the definition in nslm_oracle.c.  Parity is pinned: the restatement reproduces the reference's
 * own known answers (states after seed 1, period 65535, FNV-1a 0x740e86e513d34463 over 24 states of every seed,
 * GF(2) linearity of the stream table, P=4 decode vs a double recomputation, router tie rule 300-before-7) and is
 * cross-checked against the reference's C sources compiled as-is (oracle/_ref, built by oracle/Makefile). */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- LFSR spec ---- */
uint16_t orc_lfsr_step(uint16_t s);
void orc_lfsr_states(uint16_t s, int n, uint16_t* out);
uint32_t orc_stream32(uint16_t s);
void orc_table32(uint32_t* table /* [65536] */);
uint64_t orc_fnv24_all_seeds(void);
int orc_period(void);

/* ---- scalar helpers ---- */
uint16_t orc_f2bf(float f);
float orc_bf2f(uint16_t h);
float orc_bfr(float f);
float orc_scale(int e);
int orc_q4(uint16_t coef, int p);

/* ---- P=4 block decode ---- */
void orc_decode_block_bf16(uint16_t seed, uint16_t coef, int e, uint16_t out[8]);
void orc_decode_block_f32(uint16_t seed, uint16_t coef, int e, float out[8]);
/* rows x K matrix of one slice: seeds/coefs [rows][K/8], codes nibble g&1 of byte g>>1 with g = r*(K/8)+b */
void orc_decode_rows_f32(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K,
                         float* out);
void orc_decode_rows_bf16(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K,
                          uint16_t* out);

/* ---- mat-vec references (double accumulation over exact f32 weights) ---- */
/* y[t*ys + r] = sum_c W[r][c] x[t*xs + c] as double; mag (optional) = sum |w x| */
void orc_matvec_f64(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K,
                    const float* x, int xs, int T, double* y, int ys, double* mag);
/* the engines' rounding point: y = bf16(acc), or add: y = bf16(y + bf16(acc)) */
void orc_mv(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int eb, int rows, int K, const float* x,
            int xs, int T, int add, float* y, int ys);
/* a[r] = bf16(silu_bf(bf16(g_r)) * bf16(u_r)) */
void orc_mv_gu(const uint16_t* gs, const uint16_t* gc, const uint8_t* ge, int geb, const uint16_t* us, const uint16_t* uc,
               const uint8_t* ue, int ueb, int rows, int K, const float* x, float* a);
float orc_silu_bf(float g);
void orc_swiglu(const float* g, const float* u, float* a, int n);

/* ---- router and combine ---- */
void orc_route(const float* logits, int E, int k, int32_t* ind, float* wt);
void orc_q4_moe_combine(int d, int k, const float* D, const float* wt, const float* sh, const float* sg, int sgld,
                        float* out, int T);
void orc_moe_combine(const float* D, const float* w, const float* shared, float* x, int d, int k, int T);
void orc_mova_topk(const float* score, const float* sel, int n, int k, float scale, int32_t* inds, float* wts);
void orc_mova_router(int d, int hw, int n, int k, float scale, const uint16_t* W, const uint16_t* bias, const float* x,
                     float* score, float* sel, int32_t* inds, float* wts);
float orc_softplus_gate(float g);
void orc_decode3_block_f32(uint16_t seed, uint16_t nib, int bias, float out[8]);
void orc_decode3_block_bf16(uint16_t seed, uint16_t nib, int bias, uint16_t out[8]);
void orc_decode3_rows_f32(const uint16_t* seeds, const uint16_t* nibs, int bias, int rows, int K, float* out);
void orc_q4_mv(const uint32_t* codes, const uint16_t* scales, const uint16_t* biases, int K, int R, const float* x, int T,
               int add, float* y, double* mag);
void orc_argmax(const float* logits, int V, int32_t* out, double* prob);

/* ---- grouping ---- */
typedef struct { int32_t slice, start, count, pad; } OrcTile;
/* perm: pair ids by expert, ascending within an expert; tiles of <= bn pairs; returns the tile count */
int orc_bucket(const int32_t* inds, int count, int n, int bn, int32_t* perm, OrcTile* tiles);

/* ---- grouped GEMM reference: y[p][r] = bf16(sum_c wv(r,c) x[p/xdiv][c]), wv rounded to bf16 unless exact ---- */
void orc_mm_pairs(const uint16_t* const* seeds, const uint16_t* const* coefs, const uint8_t* const* codes, const int32_t* eb,
                  const int32_t* slice_of_pair, int P, int xdiv, int rows, int K, const float* x, int xs, int exact,
                  float* y, int ys);

/* ---- one MoE layer, the CPU reference forward's arithmetic (double sums, f32 stores, no bf16 points) ---- */
typedef struct {
    int d, ff, E, k;
    const uint16_t *gs, *gc, *us, *uc, *ds, *dc;   /* [E][rows][K/8] */
    const uint8_t *ge, *ue, *de;                    /* [E][rows*K/16] */
    const int32_t *geb, *ueb, *deb;                 /* [E] */
} OrcMoe;
void orc_moe_layer(const OrcMoe* m, const float* x, const float* logits, int T, float* out, int32_t* ind_out,
                   float* wt_out);

/* ---- the vectorised CPU seed mat-vec (timed baseline; restates the reference's 16-rows-per-step kernel) ---- */
void orc_cpu_seed4_matvec_mt(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                             const uint32_t* table, const float* x, int rows, int kb, float* y, int threads);
void orc_cpu_seed4_matvec_scalar(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                                 const uint32_t* table, const float* x, int rows, int kb, float* y);
/* best-of-reps wall seconds for one call; fills y */
double orc_cpu_seed4_time(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias,
                          const float* x, int rows, int kb, float* y, int threads, int reps);
/* the CPU-tiled layout (cpu_seed4_tiled.c): x [ntok][kb*8] -> y [ntok][rows], ntok <= 8, kb even */
typedef struct OrcTiled OrcTiled;
OrcTiled* orc_cpu_seed4_tile(const uint16_t* seeds, const uint16_t* coefs, const uint8_t* codes, int bias, int rows, int kb);
void orc_cpu_seed4_tiled_free(OrcTiled* t);
int orc_cpu_seed4_tiled_matmul_mt(const OrcTiled* m, const uint32_t* table, const float* x, int ntok, float* y, int threads);
typedef struct { const OrcTiled* m; const float* x; int ntok; float* y; } OrcTiledJob;
int orc_cpu_seed4_tiled_jobs(const OrcTiledJob* jobs, int njobs, const uint32_t* table, int threads);
double orc_cpu_seed4_tiled_time(const OrcTiled* m, const float* x, int ntok, float* y, int threads, int reps);

/* ---- seeded generator shared by host tests and device uploads (splitmix64) ---- */
uint64_t orc_splitmix64(uint64_t* state);
void orc_gen_matrix(uint64_t seed, int rows, int K, uint16_t* seeds, uint16_t* coefs, uint8_t* codes);
void orc_gen_normal(uint64_t seed, size_t n, int round_bf16, float* out);

#ifdef __cplusplus
}
#endif
