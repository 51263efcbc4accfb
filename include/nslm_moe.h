/* nslm_moe.h - host side of one resident MoE expert layer above the kernel ABI (nslm_kernels.h).
 *
 * It issues, for T rows, what the reference engine's moe() issues between the router logits and the combined output
 * (engine/qwen4_cuda.c:1023-1083): top-k routing, the routed experts' gate + up + SwiGLU and down projections over
 * the T * top_k (row, expert) pairs -- the mat-vec path for T <= MV_MAXT rows (:1071-1074), the grouped prompt path
 * for more (:1058-1065) -- and the weighted combine (:1078).  The reference has no stand-alone entry point for this
 * slice (it is a static function of its engine object, engine/qwen4_eng.h:38-62); these calls give it one, with the
 * reference's conventions: int results are 0 or -1 with a message in nsl_last_error(), work buffers are allocated at
 * creation only, the device form only enqueues launches on the caller's stream. */
#pragma once
#include "nslm_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct NslMoe NslMoe;

/* wg / wu / wd: device arrays of n_exp WSlice entries (gate and up: ff rows x d; down: d rows x ff); G: the device
 * stream table.  NULL on a bad shape or when memory runs out. */
NslMoe* nsl_moe_create(int d, int ff, int n_exp, int top_k, int max_tokens, const WSlice* wg, const WSlice* wu,
                       const WSlice* wd, const uint32_t* G);
void nsl_moe_destroy(NslMoe* m);
/* Point the object at another layer's slice tables (same shapes). */
void nsl_moe_set_layer(NslMoe* m, const WSlice* wg, const WSlice* wu, const WSlice* wd);
/* Rows from which the grouped prompt path is taken (default MV_MAXT + 1, the reference's rule). */
void nsl_moe_set_grouped_min_tokens(NslMoe* m, int t);
/* 1 (default): the engine's bf16 rounding points (activations and expert outputs rounded to bf16 as kc_mv_gu and
 * kc_mv_sel do).  0: f32 throughout on the mat-vec path (nsl_mv_gu_raw, nsl_mv_raw), for comparison with the CPU
 * reference forward, which keeps f32 (nslm/lib_qwen4_ref.c:177-207). */
void nsl_moe_set_rounding(NslMoe* m, int bf16_points);
/* Programmatic dependent launch of the decode path's kernels (default on): each kernel's blocks become resident while
 * the previous kernel drains and wait for its completion before they touch its results.  0 = ordinary launches. */
void nsl_moe_set_dependent_launch(NslMoe* m, int on);
/* 1 (default): in the host and pinned forms the combine kernel stores the result rows straight into the pinned output buffer
 * (no device-to-host copy is enqueued).  0: the result goes to device memory and a copy brings it to the host. */
void nsl_moe_set_direct_output(NslMoe* m, int on);
/* 1: a decode step whose sizes nsl_mv_step serves is one launch; 0 (default): the three dependent launches, which
 * measured faster (config 1: 114.2 against 126.3 us at 8 rows, 26.2 against 26.7 us at 1 row). */
void nsl_moe_set_one_launch(NslMoe* m, int on);
/* 0, or 1 when a bounded wait inside a one-launch step ran out since the last call (that step's output is not valid).
 * Reads device memory: call it after the layer's work has been waited for. */
int nsl_moe_step_status(NslMoe* m);
/* x [T][d], logits [T][n_exp] and out [T][d] in device memory; launches only. */
int nsl_moe_forward_dev(NslMoe* m, cudaStream_t s, const float* x, const float* logits, int T, float* out);
/* The same with host buffers: staged through pinned memory, copied both ways on the layer's stream, synchronised.
 * ind_out (optional): the T * top_k routed expert ids. */
int nsl_moe_forward_host(NslMoe* m, const float* x, const float* logits, int T, float* out, int32_t* ind_out);
/* The layer's pinned staging buffers and the forward that uses them in place (no extra host copy). */
float* nsl_moe_host_x(NslMoe* m);
float* nsl_moe_host_logits(NslMoe* m);
float* nsl_moe_host_out(NslMoe* m);
int nsl_moe_forward_pinned(NslMoe* m, int T);
/* The same in two halves: submit enqueues the copies and the layer on the handle's stream and returns; wait blocks until
 * the result is in the pinned output buffer.  Two handles used alternately keep two steps in flight. */
int nsl_moe_submit_pinned(NslMoe* m, int T);
/* nsl_moe_submit_pinned from the caller's own pinned memory: block = max_tokens rows of d floats followed by max_tokens rows
 * of n_exp logits (a full batch), copied to the device as it lies (one copy, no staging copy on the host); the result lands in
 * nsl_moe_host_out as usual.  Pair with nsl_moe_wait. */
int nsl_moe_submit_block(NslMoe* m, const float* block);
int nsl_moe_wait(NslMoe* m);
/* Routing of the last forward (device memory) and the layer's stream. */
const int32_t* nsl_moe_dev_ind(NslMoe* m);
const float* nsl_moe_dev_wt(NslMoe* m);
cudaStream_t nsl_moe_stream(NslMoe* m);

#ifdef __cplusplus
}
#endif
