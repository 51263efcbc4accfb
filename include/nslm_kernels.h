/* nslm_kernels.h - C ABI of the B200 (sm_100a) seed-decode kernels.
 *
 * The kc_* / kq4_* entry points below have the names, argument order and meaning of NanoSeedLM's CUDA kernel
 * interface (engine/kernels_cuda.h, engine/kernels_qwen4.h), so the reference's C host code (engine/qwen4_cuda.c,
 * engine/mova_cuda.c, tests/kernel_backend_cuda.c, harness/nslm-mova-kbench.c) links against this library for the
 * seed mat-vec / grouped GEMM / grouping / combine / expert-cache part of a forward without source changes.  Each
 * declaration cites the reference declaration it replaces.  The nsl_* entry points are additions (raw-f32 outputs for
 * parity tests, the bit-exact decode, status words, the expert-parallel layer).
 *
 * Conventions (engine/kernels_cuda.h:1-7; engine/qwen4_cuda.c:1219-1234): the first argument is the stream; calls
 * are asynchronous launches that return void and allocate nothing; the caller owns every buffer; errors surface at the
 * caller's cudaStreamSynchronize + cudaGetLastError.  Activations are f32 arrays of bf16-rounded values; xs / ys are
 * row strides in floats.  The SEED4P4 weight format (MF_SEED4P4) is implemented everywhere; the mat-vec and GEMM entry
 * points (kc_mv, kc_mv_sel, kc_mv_gu, kc_mm*) also serve MF_SEED4 (P = 3: p[0] seeds, p[1] nibble words -- exponent code
 * in bits 0-3, coefficient p in bits 4p+4..4p+7 --, eb the exponent bias, G the 24- or 32-bit stream table), the dense
 * kc_mv MF_Q4, and the dense kc_mv / kc_mm stored BF16 values (MF_BF16: p[0] = [R][K]): a call with another format
 * launches nothing and records an error that nsl_last_error() returns. */
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Weight formats: numeric values of engine/kernels_moe.metal:15. */
enum { MF_BF16 = 0, MF_SEED4 = 1, MF_Q8 = 2, MF_Q4 = 3, MF_SEED4P4 = 4, MF_SEED6P8 = 5, MF_TCQ = 8 };

#define MV_MAXT 8                 /* engine/kernels_moe.metal:16  dense mat-vec: tokens per call */
#define MMT_BM 64                 /* engine/kernels_cuda.h:115    GEMM tile constants callers size buffers with */
#define MMT_BN 128                /* engine/kernels_cuda.h:116    pairs per tile-table entry */
#define MMT_BK 32                 /* engine/kernels_cuda.h:118 */
#define BUCKET_MAX_EXPERTS 1024   /* engine/kernels_cuda.h:104 */
#define CACHE_MAX_PER_LAYER 1024  /* engine/kernels_cuda.h:52 */
#define CACHE_TICK_BASE 0x40000000u /* engine/kernels_cuda.h:48 */
enum { CACHE_PROTECT_PREV = 2 };  /* engine/kernels_cuda.h:51 */

/* One slice's streams (engine/kernels_cuda.h:19-24).  SEED4P4: p[0] seeds u16 [R][K/8], p[1] coefficient words u16
 * [R][K/8], p[3] exponent codes, two per byte, block g = r*(K/8)+b in nibble g&1 of byte g>>1; eb the slice's
 * exponent bias.  Streams may live in device memory or in mapped pinned host memory. */
typedef struct {
    const void* p[4];
    int32_t eb;
    int32_t gs;
    int32_t pad[2];
} WSlice;

/* Grouped GEMM: one expert's run of pairs in perm[] (engine/kernels_moe.metal:130). */
typedef struct { int32_t slice, start, count, pad; } MmTile;

/* The expert cache (engine/kernels_cuda.h:32-47): field order is the ABI. */
typedef struct {
    int32_t* unit_slot;
    int32_t* slot_unit;
    uint32_t* slot_last;
    uint32_t* tick;
    uint32_t* stats;
    int32_t* jobs;
    int32_t* njobs;
    uint8_t* vram;
    const uint8_t* host;
    uint64_t unit_bytes;
    int32_t slots, per_layer, ntens;
    WSlice* tab;
    uint32_t off[3][4];
    uint64_t hits, misses;
} CachePool;

/* ---- mat-vec (decode and multi-token verify, T <= MV_MAXT) ---------------------------------------------------------- */
/* engine/kernels_cuda.h:79  y[t][r] = bf16(W[r] . x[t]); add = 1: y = bf16(y + bf16(acc)).  G: the 65536-entry
 * lfsr_stream32 table in device memory.  A token's result does not depend on T.
 * fmt = MF_Q4 (the LM head, engine/kernels_moe.cu:171-189) is served too: p[0] codes u32 [R][K/8] (value i of a word in
 * bits 4i..4i+3), p[1] / p[2] bf16 scales / biases per group of 64 weights (gs 0 or 6), weight = s q + b; K a multiple of
 * 64; activations must be bf16-valued (as every activation of the engine is): they enter the tensor cores as bf16. */
void kc_mv(cudaStream_t s, int fmt, WSlice w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add,
           const uint32_t* G);
/* engine/kernels_cuda.h:82  pair p uses slice sel[p], input row p / xdiv, output row p. */
void kc_mv_sel(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
               const int32_t* sel, int P, int xdiv, const uint32_t* G);
/* engine/kernels_cuda.h:85  a[p][r] = bf16(silu_bf(bf16(gate . x)) * bf16(up . x)). */
void kc_mv_gu(cudaStream_t s, int fmt, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* a,
              int ys, const int32_t* sel, int P, int xdiv, const uint32_t* G);

/* ---- prompt GEMM (tcgen05 tensor-core path) ------------------------------------------------------------------------- */
/* engine/kernels_cuda.h:96  1: seed weights exact in f32 (three bf16 terms); 0 (default): rounded to bf16. */
void kc_seed_gemm_f32(int on);
/* engine/kernels_cuda.h:97 */
void kc_mm(cudaStream_t s, int fmt, WSlice w, int K, int R, const float* x, int xs, float* y, int ys, int T, int add,
           const uint32_t* G);
/* engine/kernels_cuda.h:99 */
void kc_mm_grouped(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                   int xdiv, const int32_t* perm, const MmTile* tiles, int ntiles, const uint32_t* G);
/* engine/kernels_cuda.h:105  count selections over n experts -> perm, tiles, ntiles (2n+3 ints, [0] = tile count). */
void kc_bucket(cudaStream_t s, const int32_t* inds, int count, int n, int32_t* perm, MmTile* tiles, int32_t* ntiles);
/* engine/kernels_cuda.h:106  the tile count read on the device; the grid is max_tiles. */
void kc_mm_grouped_dev(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                       int xdiv, const int32_t* perm, const MmTile* tiles, const int32_t* ntiles, int max_tiles,
                       const uint32_t* G);
/* engine/kernels_cuda.h:110-114  activations packed to bf16 once, then reused by the GEMMs. */
void kc_pack_input_bf16(cudaStream_t s, const float* x, uint16_t* y, size_t n);
void kc_mm_packed(cudaStream_t s, int fmt, WSlice w, int K, int R, const uint16_t* x, int xs, float* y, int ys, int T, int add,
                  const uint32_t* G);
void kc_mm_grouped_packed(cudaStream_t s, int fmt, const WSlice* ws, int K, int R, const uint16_t* x, int xs, float* y, int ys,
                          int xdiv, const int32_t* perm, const MmTile* tiles, const int32_t* nt, int max_tiles,
                          const uint32_t* G);

/* ---- elementwise and combine ------------------------------------------------------------------------------------- */
/* engine/kernels_cuda.h:124  a = bf16(silu_bf(g) * u). */
void kc_swiglu(cudaStream_t s, const float* g, const float* u, float* a, int n);
/* engine/kernels_cuda.h:125  x = bf16(x + bf16(bf16(sum_j bf16(D_j bf16(w_j))) + shared)). */
void kc_moe_combine(cudaStream_t s, const float* D, const float* w, const float* shared, float* x, int d, int k, int T);

/* ---- router and combine of the qwen4 engine ------------------------------------------------------------------------ */
/* engine/kernels_qwen4.h:53-54  softmax over all experts, top-k, ties to the higher index, weights renormalised.
 * cfg points at the reference's Qwen4Cfg (nslm/qwen4_cfg.h:9-22); only its n_exp and top_k fields (ints 21 and 22)
 * are read.  n_exp <= 1024, top_k <= 32. */
void kq4_route(cudaStream_t s, const void* cfg, const float* logits, int32_t* ind, float* wt, int T);
void kq4_route_ld(cudaStream_t s, const void* cfg, const float* logits, int ld, int32_t* ind, float* wt, int T);
/* engine/kernels_qwen4.h:71  out[t] = sum_j wt[t][j] D[t*k+j] + sigmoid(sg[t*sgld]) sh[t], plain f32. */
void kq4_moe_combine(cudaStream_t s, int d, int k, const float* D, const float* wt, const float* sh, const float* sg,
                     int sgld, float* out, int T);

/* ---- router of the MoVA engine --------------------------------------------------------------------------------------- */
/* engine/kernels_moe.metal:72-76: field order is the ABI. */
typedef struct {
    int32_t d, n, top_k;   /* input width, experts, selected */
    int32_t hw;            /* width of the first partition of the input (d / 2) */
    float scale;           /* the weights' final factor */
} RouterArgs;
/* engine/kernels_cuda.h:120  W [n][d] and bias [n] are BF16.  logit = bf16(dot over inputs < hw) + bf16(dot over the
 * rest); score = sigmoid(logit); sel = score + bias; the top_k largest sel, ties to the lowest id, best first;
 * wts = score / sum of the picked scores * scale.  score and sel [T][n] are outputs too.  n <= 1024, top_k <= 64,
 * d a multiple of 8. */
void kc_router(cudaStream_t s, RouterArgs a, const uint16_t* W, const uint16_t* bias, const float* x, float* score,
               float* sel, int32_t* inds, float* wts, int T);
/* engine/kernels_cuda.h:123  the top-k step alone, from scores and selection scores. */
void kc_router_topk(cudaStream_t s, RouterArgs a, const float* score, const float* sel, int32_t* inds, float* wts, int T);

/* ---- per-head maps (the SEED4P4 branch) ------------------------------------------------------------------------------- */
/* engine/kernels_moe.metal:111-114: field order is the ABI. */
typedef struct {
    int32_t H, O, I, xs, hs, gate;
    int32_t pad[2];
} HmvArgs;
/* engine/kernels_cuda.h:142  y[t][h][o] = bf16(W_h[o] . x[t*xs + h*hs ..]); with a.gate, bf16(that *
 * bf16(softplus(g[t][h][o]; beta = ln 2))).  W is one stacked matrix [H*O][I]: p[0] seeds, p[1] coefficient words,
 * p[2] the heads' exponent biases (int32 [H], device memory), p[3] exponent codes.  I a multiple of 8; any T. */
void kc_heads_mv(cudaStream_t s, HmvArgs a, int fmt, WSlice W, const uint32_t* G, const float* x, const float* g, float* y,
                 int T);
/* engine/kernels_cuda.h:145  the stacked matrix decoded to BF16 [H][O][I], each weight the exact f32 weight rounded to
 * nearest even (what the GEMM feeds the tensor cores). */
void kc_heads_deq(cudaStream_t s, int fmt, WSlice W, const uint32_t* G, int H, int O, int I, uint16_t* out);

/* ---- decode attention over a BF16 or 8-bit KV cache -------------------------------------------------------------------- */
/* engine/kernels_moe.metal:78-84, engine/kernels_cuda.h:56-72: field order is the ABI. */
typedef struct {
    int32_t n_head, n_kv, chunk, n_splits;   /* chunk: target keys per split; a row at position pos uses
                                                min(n_splits, ceil((pos + 1) / chunk)) splits (see nsl_attn_batch_invariant) */
    float scale;
} AttnArgs;
typedef struct { int32_t pos, kv0; int32_t pad[2]; } RowInfo;   /* kv0: the cache row of the sequence slot's position 0 */
enum { KV_BF16 = 0, KV_Q8 = 1, KV_FP8 = 2, KV_FP4 = 3 };
typedef struct { void* k; void* v; float* ks; float* vs; } KvSeg;   /* rows of n_kv heads x 128 values */
typedef struct { KvSeg a, b; int32_t nv, fmt; } KvView;             /* positions [0, nv) in a, the rest in b */
/* engine/kernels_cuda.h:130  q [T][n_head][128] (f32), row t attends cache rows kv0 .. kv0 + pos of its KV head
 * (head h uses KV head h / (n_head / n_kv)); part: T x n_head x n_splits x 130 floats of partials; o [T][n_head][128] =
 * bf16(bf16(softmax(scale q.K) V) * bf16(softplus(g; beta = ln 2))) (g NULL: no gate).  kv.fmt = KV_BF16, or KV_Q8 (int8
 * codes, ks / vs [rows][n_kv] f32: a value is bf16(code * scale), engine/kernels_moe.cu:807-824); FP8 / FP4 are refused.
 * Any group size n_head / n_kv up to 16. */
void kc_attn(cudaStream_t s, AttnArgs a, const float* q, KvView kv, const RowInfo* ri, float* part, const float* g, float* o, int T);
/* No counterpart in the reference.  kc_attn's first pass runs on the tensor cores (the heads of a KV head are the columns of
 * the products).  By default, when a.n_splits >= 3 and T <= 1024, the step's keys are dealt evenly to the blocks whatever
 * a.n_splits asks: the cuts of a row's keys then depend on all rows of the step, so the same row run alone and run in a
 * batch can differ in the last bits of the f32 sums (both within the reference's bound).  on = 1 makes every call use one
 * block per (split, KV head, row), the reference's cuts: a row's output is then bit-identical whatever rows share the call.
 * The partials' use of `part` is internal to the two kernels in both forms and never exceeds the size above. */
void nsl_attn_batch_invariant(int on);

/* ---- greedy decoding over the LM head's logits ------------------------------------------------------------------------ */
/* engine/kernels_cuda.h:177-178  out[i] = arg max of row i of logits [n][V] (ties: the lowest id); prob[i] (optional) =
 * its softmax probability. */
void kc_argmax(cudaStream_t s, const float* logits, int32_t* out, int V, int n);
void kc_argmax_p(cudaStream_t s, const float* logits, int32_t* out, float* prob, int V, int n);
/* ---- expert cache -------------------------------------------------------------------------------------------------- */
/* engine/kernels_cuda.h:53  LRU admit of the units selected by inds[count] of sparse layer sl. */
void kc_cache_admit(cudaStream_t s, const CachePool* p, int sl, const int32_t* inds, int count, int flags);
/* engine/kernels_cuda.h:55  the queued units, host arena -> VRAM slots; blocks = the copy's grid. */
void kc_cache_copy(cudaStream_t s, const CachePool* p, int blocks);

/* ---- additions (no counterpart in the reference's header) ---------------------------------------------------------- */
/* No counterpart in the reference.  kc_bucket for callers that cannot allocate device memory: code running inside a
 * host framework that owns the allocator, a plugin loaded after the memory pool was sized, a latency path that may not
 * call cudaMalloc.  The 2n+3 ints of work memory that kc_bucket takes from its caller live in an array built into the
 * library (8 KB, held by every GPU that loads the library until the process exits), so the caller passes inputs and
 * outputs only: perm and tiles as kc_bucket, ntiles_out[0] = the tile count.  n <= BUCKET_MAX_EXPERTS, else nothing is
 * launched and nsl_last_error() says why.  Nothing is allocated or freed.  The first call on a device looks up the
 * array's address (a host-side query): make that call before any stream capture starts.  All calls on a device share
 * the array, which keeps the last call's offsets: calls that overlap on the GPU (two streams) race. */
void nsl_bucket_noalloc(cudaStream_t s, const int32_t* inds, int count, int n, int32_t* perm, MmTile* tiles,
                        int32_t* ntiles_out);
/* The whole decode step of an expert layer -- router, gate + up + SwiGLU, down projection, weighted combine (the four
 * launches of engine/qwen4_cuda.c:1033-1078) -- as ONE launch whose blocks pass from phase to phase and wait on counters
 * for what other blocks produce (every wait bounded).  Results are bit for bit those of nsl_mv_gu_routed + kc_mv_sel +
 * kq4_moe_combine.  Measured slower than those three as dependent launches (config 1, 8 rows: 126.3 against 114.2 us a
 * step): the dependent launches already hide ramp and prologue, and a block here waits for its neighbours at each phase
 * change.  Returns 1 = launched; 0 = a size is outside what it serves (T <= MV_MAXT rows, d and ff = 64 * 2^j <=
 * 2048, aligned rows) and nothing was launched.  sync: 4 * (2 + T + T * top_k) bytes of device memory, zero before the
 * first call; every call leaves its counters zero; sync[0] = 1 after a launch in which a wait ran out (output not valid). */
int nsl_mv_step(cudaStream_t s, const WSlice* wg, const WSlice* wu, const WSlice* wd, int d, int ff, const float* x, int xs,
                int n_exp, int top_k, const float* logits, int ld, int T, int32_t* ind, float* wt, float* A, float* D,
                float* out, int raw, unsigned* sync, const uint32_t* G);
/* kc_swiglu with the results stored as packed bf16 (they are bf16 values): the input form of kc_mm_grouped_packed for
 * the down projection.  n even. */
void nsl_swiglu_packed(cudaStream_t s, const float* g, const float* u, uint16_t* a, int n);
/* The router with its two sizes passed directly. */
void nsl_route(cudaStream_t s, int n_exp, int top_k, const float* logits, int ld, int32_t* ind, float* wt, int T);
/* Mat-vec with the f32 accumulator stored unrounded (the CPU seed path's result convention,
 * nslm/lib_cpu_seed4.c:73,100), dense (sel == NULL: ws is a HOST pointer to the one slice, P = T tokens, xdiv = 1) or gathered (ws a device table). */
void nsl_mv_raw(cudaStream_t s, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                const int32_t* sel, int P, int xdiv, const uint32_t* G);
/* kc_mv_gu without the bf16 rounding points: a = silu(gate . x) * (up . x) in f32. */
void nsl_mv_gu_raw(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* a,
                   int ys, const int32_t* sel, int P, int xdiv, const uint32_t* G);
/* Rows [0,R) of one slice decoded to the exact f32 weights (nslm/lib_rows.c:49-76) or their bf16 rounding
 * (nslm/lib_search4.c:22-31): bit-exact.  out is [R][K]. */
void nsl_decode_f32(cudaStream_t s, WSlice w, int K, int R, float* out, const uint32_t* G);
void nsl_decode_bf16(cudaStream_t s, WSlice w, int K, int R, uint16_t* out, const uint32_t* G);
/* 0, or the code of the first bounded device-side wait that ran out in a GEMM block since the last call (1 a producer
 * waiting for a free stage, 2 the epilogue waiting for the accumulator, 3 the MMA issuer waiting for a full stage); a
 * block that gives up frees its tensor memory and returns without storing.  Call after synchronising the stream. */
int nsl_mm_status(void);
/* Fills a 65536-entry host array with the stream table the G arguments expect (lfsr_stream32 of every seed,
 * nslm/lfsr.h:53-59). */
void nsl_stream_table(uint32_t* host_table);
/* Message of the first host-side argument error since the last call (format not SEED4P4, bad shape), or "". */
const char* nsl_last_error(void);
/* Number of kernels this library has launched since it was loaded (bench bookkeeping). */
uint64_t nsl_launch_count(void);
/* Multiprocessor count the persistent grids are sized for (queried once per device). */
int nsl_sm_count(void);
/* nsl_decode_f32 / nsl_decode_bf16 for a P = 3 (MF_SEED4) slice. */
void nsl_decode3_f32(cudaStream_t s, WSlice w, int K, int R, float* out, const uint32_t* G);
void nsl_decode3_bf16(cudaStream_t s, WSlice w, int K, int R, uint16_t* out, const uint32_t* G);
/* kc_mv_gu with the router folded into its prologue (one launch less on the decode path): T <= MV_MAXT rows of logits
 * [T][ld] -> ind / wt [T][top_k] as kq4_route gives them, and a [T * top_k][R] as kc_mv_gu gives it for sel = ind,
 * xdiv = top_k.  K = 64 * 2^j <= 2048; raw: unrounded f32 outputs.  n_exp <= 1024, top_k <= 32. */
void nsl_mv_gu_routed(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* a, int ys,
                      int n_exp, int top_k, const float* logits, int ld, int T, int32_t* ind, float* wt, int raw,
                      const uint32_t* G);
/* Programmatic dependent launch for the calling thread's next launches of: the seed mat-vecs (kc_mv, kc_mv_sel, kc_mv_gu,
 * nsl_mv*), the MF_Q4 and MF_BF16 forms of kc_mv / kc_mm's decode-batch kernel, kq4_moe_combine, nsl_ep_combine and the
 * peer-memory exchange kernels, kc_attn (whose reduction is always a dependent launch of its first pass), kc_gnorm,
 * kc_rope_kv and nsl_residual_add.  While on, such a kernel may become resident before the previous kernel in its stream
 * has finished; it waits on the device for that kernel's completion before it reads or writes anything a neighbour
 * touches, so it is safe after any kernel; after a copy or another kind of node it is an ordinary launch.  Thread-local;
 * turn it off again (0) before launching anything else on the stream. */
void nsl_dependent_launch(int on);

#ifdef __cplusplus
}
#endif
