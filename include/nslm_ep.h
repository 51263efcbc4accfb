/* nslm_ep.h - device steps of the expert-parallel dispatch / combine layer.
 *
 * The reference is single-GPU (engine/mova_cuda.c:590 selects device 0 and no collective exists in its tree): its
 * experts are tiered between VRAM and host memory, never sharded.  This layer has therefore no counterpart in the
 * reference; it follows the reference's kernel-call conventions (stream first, asynchronous, caller-owned buffers,
 * nothing allocated) and sits between its router (kq4_route) and its combine (kq4_moe_combine).
 *
 * Experts are sharded evenly: rank r owns experts [r E/N, (r+1) E/N).  Every rank routes its own tokens; the token
 * rows (packed bf16) and their routing travel to every rank in one all-to-all; each rank keeps the (token, expert)
 * pairs it owns (nsl_ep_plan), runs them through the seed mat-vec kernels on the received rows (nsl_mv_gu_rows,
 * nsl_mv_sel_rows), pre-sums each token's local experts (nsl_ep_combine); the partial rows go back in a second
 * all-to-all and the source rank adds them in rank order (nsl_ep_reduce).  The two exchanges are either collective calls
 * issued by the host layer (the kernels of the first part read only local memory) or stores into peer memory by the
 * kernels of the second part below. */
#pragma once
#include "nslm_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Gathered routing of T = n_ranks * t_loc tokens: token (r, t) has its k expert ids at ind[r * rank_stride + t * k ..]
 * and weights at wt[the same index] (rank_stride in 4-byte elements: the receive buffer's per-rank chunk).  Keeps the
 * pairs whose expert lies in [lo, hi), in token order:  sel[p] = expert - lo,  xrow[p] = r * row_stride + t (the row of
 * the received input buffer),  wsel[p] = the routing weight;  tok_off[g] = index of the first pair of token
 * g = r * t_loc + t, tok_off[T] = *count = the number of pairs kept.  T * k <= 65536. */
void nsl_ep_plan(cudaStream_t s, const int32_t* ind, const float* wt, int n_ranks, int t_loc, int k, int rank_stride,
                 int row_stride, int lo, int hi, int32_t* sel, int32_t* xrow, float* wsel, int32_t* tok_off,
                 int32_t* count);
/* Gather mat-vecs over a compacted pair list whose length is on the device (see nsl_ep_plan): pair p uses slice
 * sel[p]; the gate+up form reads input row xrow[p] of x (packed bf16 rows of stride xs elements when x_bf16, else f32),
 * the second form reads row p.  max_pairs bounds the list, *count is its length, raw = 1 stores unrounded f32 (no bf16 rounding points). */
void nsl_mv_gu_rows(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const void* x, int xs, int x_bf16,
                    float* a, int ys, const int32_t* sel, const int32_t* xrow, int max_pairs, const int32_t* count,
                    int raw, const uint32_t* G);
void nsl_mv_sel_rows(cudaStream_t s, const WSlice* ws, int K, int R, const float* x, int xs, float* y, int ys,
                     const int32_t* sel, int max_pairs, const int32_t* count, int raw, const uint32_t* G);
/* partial[g][:] = sum over pairs p in [tok_off[g], tok_off[g+1]) of wsel[p] * D[p][:], pairs ascending (zeros when the
 * token has no expert here).  T tokens of width d. */
void nsl_ep_combine(cudaStream_t s, const float* D, const float* wsel, const int32_t* tok_off, int T, int d, float* partial);
/* out[t][:] = parts[0][t][:] + parts[1][t][:] + ... in rank order; parts is [n_ranks][t_loc][d]. */
void nsl_ep_reduce(cudaStream_t s, const float* parts, int n_ranks, int t_loc, int d, float* out);

/* ---- dispatch and combine over peer memory ----------------------------------------------------------------------------
 * Instead of two collective calls, the producer kernels store into the consumers' memory over NVLink and bump counters
 * there; the consumer kernels wait (bounded, about two seconds) on counters in their own memory.  Every rank owns one
 * WINDOW of device memory that all ranks of the node map (nsl_ep_window_alloc on the owner, the 64-byte handle carried
 * to the others by any host transport, nsl_ep_window_open there).  All windows share one layout:
 *   recv_off   n chunks of chunk_bytes: chunk r = rank r's t_loc token rows (bf16), expert ids and weights of this step
 *   parts_off  n x t_loc x d floats: slot r = rank r's pre-summed rows for this rank's tokens
 *   dflag_off, cflag_off   n counters each, 128 bytes apart: rows rank r has delivered here so far (dispatch / combine)
 *   local_off  64 bytes touched only by the owner: epoch, a grid ticket, status
 * A step on every rank, on one stream: nsl_ep_p2p_route_dispatch (or nsl_route + kc_pack_input_bf16 into a local chunk
 * and nsl_ep_p2p_dispatch); nsl_ep_p2p_plan (waits for every rank's rows, then plans); nsl_mv_gu_rows and
 * nsl_mv_sel_rows on the receive area; nsl_ep_p2p_combine; nsl_ep_p2p_reduce.  All ranks must run the same number of
 * steps.  The kernels of different ranks wait on one another, so every rank needs its own GPU. */
#define NSL_EP_MAX_RANKS 16
typedef struct {
    void* win[NSL_EP_MAX_RANKS];   /* every rank's window as mapped in this process; win[me] is the local one */
    int32_t n, me;
    int32_t t_loc, reserved;       /* token rows per rank and step */
    uint64_t bytes;                /* size of a window */
    uint64_t chunk_bytes, recv_off, parts_off, dflag_off, cflag_off, local_off;
} NslEpWindow;
/* Window memory: alloc (zeroed) + handle on the owner, open / close on the peers, free on the owner.  0 on success. */
int nsl_ep_window_alloc(size_t bytes, void** ptr, void* handle64);
int nsl_ep_window_open(const void* handle64, void** ptr);
int nsl_ep_window_close(void* ptr);
int nsl_ep_window_free(void* ptr);
/* chunk (chunk_bytes, 16-byte aligned, local) -> slot `me` of every window's receive area; t_loc rows signalled. */
void nsl_ep_p2p_dispatch(cudaStream_t s, NslEpWindow w, const void* chunk);
/* Router, bf16 packing and dispatch in one kernel: logits [t_loc][ld] and x [t_loc][d] (f32, local) -> each token's row,
 * ids and weights in slot `me` of every window (ind_off / wt_off = byte offsets of ids and weights inside a chunk,
 * rows first).  n_exp <= 1024, top_k <= 32, d a multiple of 8.  ind_out / wt_out (device, [t_loc][top_k], optional): the
 * caller's own copy of its tokens' routing. */
void nsl_ep_p2p_route_dispatch(cudaStream_t s, NslEpWindow w, int n_exp, int top_k, const float* logits, int ld, const float* x,
                               int d, uint64_t ind_off, uint64_t wt_off, int32_t* ind_out, float* wt_out);
/* Returns (on the stream) when every rank's rows of this step have landed in the local window. */
void nsl_ep_p2p_wait_dispatch(cudaStream_t s, NslEpWindow w);
/* nsl_ep_plan on the window's receive area with the wait inside the kernel (replaces nsl_ep_p2p_wait_dispatch +
 * nsl_ep_plan).  Mirrored ranks (lo2 < hi2; pass 0, 0, 0 otherwise): this rank also holds its partner's experts
 * [lo2, hi2) after its own in its slice tables and the partner holds this rank's; both plan the pairs of either range
 * in token order and split that list in the middle, the rank with upper = 0 taking the first ceil(n/2) pairs: the two
 * shares differ by at most one pair whatever the routing.  sel = e - lo, or (hi - lo) + e - lo2 for the partner's. */
void nsl_ep_p2p_plan(cudaStream_t s, NslEpWindow w, uint64_t ind_off, uint64_t wt_off, int k, int row_stride, int lo, int hi,
                     int lo2, int hi2, int upper, int32_t* sel, int32_t* xrow, float* wsel, int32_t* tok_off, int32_t* count);
/* nsl_ep_combine whose rows go to slot `me` of the owning rank's partial-row area; one row signalled per token.
 * d a multiple of 4. */
void nsl_ep_p2p_combine(cudaStream_t s, NslEpWindow w, const float* D, const float* wsel, const int32_t* tok_off, int d);
/* Waits for every rank's partial rows, out[t][:] = their sum in rank order, and closes the step (epoch + 1). */
void nsl_ep_p2p_reduce(cudaStream_t s, NslEpWindow w, int d, float* out);
/* 0 when no wait has run out since the last call; else code * 256 + (rank waited for + 1), code 1 = dispatch,
 * 2 = combine.  Synchronous (reads the window's status word); call it after the stream has drained. */
int nsl_ep_p2p_status(NslEpWindow w);

#ifdef __cplusplus
}
#endif
