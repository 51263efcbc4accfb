/* nslm_decoder.h - host side of a whole MoE decoder step above the kernel ABI: the loop the reference engine runs per
 * decode forward (engine/qwen4_cuda.c:1096-1111 run_layer, :1160-1176 enqueue, :1023-1083 moe; engine/mova_cuda.c:1658-1672
 * the continuous-batching rows) for the shape of BASELINE config 4: per layer grouped RMSNorm, dense seed projections
 * q / k / v, RoPE + KV-cache write, decode attention over the BF16 cache (GQA), the output projection added to the residual
 * stream, RMSNorm, router logits, the routed seed experts (top-k, gate + up + SwiGLU, down) with ONE shared expert running
 * on a second stream and joined before the combine, the residual add; then the output norm, the affine-int4 LM head and a
 * greedy arg-max.  Every row of a step is its own sequence (RowInfo: position and the sequence slot's first cache row).
 *
 * Expert parallel: with a peer-memory window given (nslm_ep.h) the ranks split the batch's rows (data parallel for the
 * dense parts and the attention) and the routed experts (each rank holds n_exp / ranks of them); the routed part of every
 * layer is then the exchange of nslm_ep.h inside the layer.  A step only enqueues work on the caller's stream.  Calls
 * return 0, or -1 with a message in nsl_last_error(). */
#pragma once
#include "nslm_ep.h"
#include "nslm_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int32_t n_layer, d, n_head, n_kv;          /* heads are 128 wide */
    int32_t n_exp, top_k, ff_exp, ff_shared;   /* n_exp: routed experts of the whole model */
    int32_t vocab, max_rows, ctx;              /* rows per step at most; positions per sequence slot */
    int32_t exp_lo, exp_hi;                    /* the routed experts this rank holds (0, n_exp on one GPU) */
    float eps, rope_theta;
    int32_t dense_bf16;                        /* 1: the dense matrices (q, k, v, o, router, shared expert) are expanded ONCE at
                                                  creation to BF16 in device memory (the values the tensor-core path rounds seed
                                                  weights to, engine/kernels_moe.cu:405-412) and served from there; 0: regenerated
                                                  from their seeds in every call, as the routed experts always are */
} NslDecoderCfg;

typedef struct {                               /* one layer's weights in device memory (the caller owns them) */
    const uint16_t *norm_attn, *norm_ffn;      /* BF16 [d] */
    WSlice wq, wk, wv, wo;                     /* SEED4P4 dense: [n_head*128][d], [n_kv*128][d] twice, [d][n_head*128] */
    WSlice router;                             /* SEED4P4 dense [n_exp + 1][d]: the experts' logits, then the shared expert's gate */
    const WSlice *eg, *eu, *ed;                /* device tables of this rank's routed experts (exp_hi - exp_lo entries each) */
    WSlice sg, su, sd;                         /* the shared expert: gate, up [ff_shared][d] and down [d][ff_shared], dense */
} NslDecoderLayer;

typedef struct NslDecoder NslDecoder;

/* embed: BF16 table [vocab][d] in p[0]; norm_out BF16 [d]; head: affine int4 (MF_Q4, see kc_mv) [vocab][d]; G the stream
 * table; win: NULL, or this rank's view of the ranks' windows with win->t_loc = the rows this rank runs per step. */
NslDecoder* nsl_decoder_create(const NslDecoderCfg* cfg, const NslDecoderLayer* layers, WSlice embed, const uint16_t* norm_out,
                               WSlice head, const uint32_t* G, const NslEpWindow* win);
void nsl_decoder_destroy(NslDecoder* m);
/* One decode step of T rows: ids and ri in device memory, next (device, T ints) receives the greedy next tokens.  With a
 * window, T must equal its t_loc on every rank, every step. */
int nsl_decoder_step(NslDecoder* m, cudaStream_t s, const int32_t* ids, const RowInfo* ri, int T, int32_t* next);
/* Device buffers of the last step, for tests: the final hidden rows [T][d] (before the output norm) and the head's logits. */
const float* nsl_decoder_hidden(const NslDecoder* m);
const float* nsl_decoder_logits(const NslDecoder* m);
/* Copies rows [0, T) of one of them (what = 0 hidden, 1 logits) into dst (device memory) after the device has drained. */
int nsl_decoder_copy_out(NslDecoder* m, int what, int T, float* dst);
/* Layer l's KV cache (BF16 [max_rows * ctx][n_kv][128] each), to prefill or inspect. */
uint16_t* nsl_decoder_kcache(NslDecoder* m, int layer);
uint16_t* nsl_decoder_vcache(NslDecoder* m, int layer);
/* Copies n BF16 values (device memory) into the start of layer l's K and V caches (a prefilled context for timing). */
int nsl_decoder_fill_cache(NslDecoder* m, int layer, const uint16_t* k, const uint16_t* v, size_t n);
/* x = bf16(x + y) over n floats (the residual add of the decoder's stream). */
void nsl_residual_add(cudaStream_t s, float* x, const float* y, size_t n);
/* engine/kernels_cuda.h:75  x[t] = row ids[t] of a BF16 table (other table formats are refused). */
void kc_embed(cudaStream_t s, int fmt, WSlice w, int d, const int32_t* ids, float* x, int T);
/* engine/kernels_cuda.h:77  grouped RMSNorm (two groups: each half of the row by its own mean square), w in BF16. */
void kc_gnorm(cudaStream_t s, int d, float eps, const float* x, const uint16_t* w, float* y, int T);
/* engine/kernels_cuda.h:127  RoPE on q in place and on k into the cache, v into the cache; inv: 64 inverse frequencies
 * (device); BF16 and 8-bit caches. */
void kc_rope_kv(cudaStream_t s, float* q, const float* k, const float* v, KvView kv, const RowInfo* ri, const float* inv, int n_head,
                int n_kv, int T);

#ifdef __cplusplus
}
#endif
