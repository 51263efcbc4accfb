// Host side of one MoE expert layer above the kernel ABI: the sequence the reference engine's moe() issues
// (engine/qwen4_cuda.c:1023-1083) -- router top-k, routed experts' gate+up+SwiGLU and down projections over the
// (token, expert) pairs, weighted combine -- for a layer whose experts are resident in device memory.  Rows <= MV_MAXT
// take the mat-vec path (kc_mv_gu + kc_mv_sel), more rows the grouped prompt path (kc_bucket + kc_mm_grouped_dev x 3 +
// kc_swiglu), as the reference decides at engine/qwen4_cuda.c:1058-1075.  Work buffers are allocated once at creation;
// a forward allocates nothing and, in its device form, only enqueues launches (graph-capturable).
#include <cstdlib>
#include <cstring>

#include "common.cuh"

extern "C" {

struct NslMoe {
    int d, ff, n_exp, top_k, max_tokens;
    const WSlice *wg, *wu, *wd;   // device tables [n_exp]
    const uint32_t* G;            // device stream table
    float *x, *logits, *wt, *A, *Dx, *Gb, *out;
    uint16_t *xp, *Ap;            // prompt path: the rows and the SwiGLU results as packed bf16 (the GEMMs' input form)
    int32_t *ind, *perm, *ntiles;
    MmTile* tiles;
    float *hx, *hlogits, *hout;   // pinned staging for the host-buffer entry point
    int32_t* hind;
    cudaStream_t stream;
    int grouped_min_tokens;       // rows from which the grouped prompt path is taken (MV_MAXT + 1)
    int raw;                      // 1: no bf16 rounding points on the mat-vec path
    int pdl;                      // 1 (default): the decode path's kernels are programmatic dependent launches
    int direct_out;               // 1 (default): the pinned forms' combine kernel stores the result straight into pinned host memory
    int one_launch;               // 1: a decode step whose sizes the fused kernel serves is ONE launch (nsl_mv_step); default 0: it measured slower
    unsigned* step_sync;          // its counters and status word (zero between launches)
};

static void* dalloc(size_t n) {
    void* p = NULL;
    if (cudaMalloc(&p, n ? n : 16) != cudaSuccess) return NULL;
    return p;
}

void nsl_moe_destroy(NslMoe* m);

NslMoe* nsl_moe_create(int d, int ff, int n_exp, int top_k, int max_tokens, const WSlice* wg, const WSlice* wu,
                       const WSlice* wd, const uint32_t* G) {
    if (d % 8 || ff % 8 || n_exp < 1 || n_exp > BUCKET_MAX_EXPERTS || top_k < 1 || top_k > 32 || max_tokens < 1) {
        nsl::set_error("nsl_moe_create: unsupported shape d %d ff %d experts %d top_k %d tokens %d", d, ff, n_exp, top_k, max_tokens);
        return NULL;
    }
    NslMoe* m = (NslMoe*) calloc(1, sizeof(NslMoe));
    m->d = d; m->ff = ff; m->n_exp = n_exp; m->top_k = top_k; m->max_tokens = max_tokens;
    m->wg = wg; m->wu = wu; m->wd = wd; m->G = G;
    m->grouped_min_tokens = MV_MAXT + 1;
    m->pdl = 1;
    const size_t T = (size_t) max_tokens, P = T * top_k;
    m->x = (float*) dalloc(T * d * 4 + T * n_exp * 4);      // inputs in one block (rows, then logits): one copy brings both
    m->logits = m->x ? m->x + T * d : NULL;
    m->wt = (float*) dalloc(P * 4);
    m->ind = (int32_t*) dalloc(P * 4);
    m->A = (float*) dalloc(P * ff * 4);
    m->Dx = (float*) dalloc(P * d * 4);
    m->out = (float*) dalloc(T * d * 4);
    const bool big = max_tokens > MV_MAXT;
    m->Gb = big ? (float*) dalloc(P * ff * 4) : NULL;
    m->xp = big ? (uint16_t*) dalloc(T * d * 2) : NULL;
    m->Ap = big ? (uint16_t*) dalloc(P * ff * 2) : NULL;
    m->perm = (int32_t*) dalloc(P * 4);
    m->tiles = (MmTile*) dalloc((P / MMT_BN + n_exp + 1) * sizeof(MmTile));
    m->ntiles = (int32_t*) dalloc((2 * (size_t) n_exp + 3) * 4);
    cudaHostAlloc((void**) &m->hx, T * d * 4 + T * n_exp * 4, cudaHostAllocDefault);      // the same layout in pinned memory
    m->hlogits = m->hx ? m->hx + T * d : NULL;
    m->direct_out = 1;
    m->one_launch = 0;
    m->step_sync = (unsigned*) dalloc(4 * ((size_t) MV_MAXT * top_k + MV_MAXT + 2));
    if (m->step_sync) cudaMemset(m->step_sync, 0, 4 * ((size_t) MV_MAXT * top_k + MV_MAXT + 2));
    cudaHostAlloc((void**) &m->hout, T * d * 4, cudaHostAllocDefault);
    cudaHostAlloc((void**) &m->hind, P * 4, cudaHostAllocDefault);
    cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
    if (!m->x || !m->logits || !m->wt || !m->ind || !m->A || !m->Dx || !m->out || !m->perm || !m->tiles || !m->ntiles ||
        !m->hx || !m->hlogits || !m->hout || !m->hind || !m->stream || (big && (!m->Gb || !m->xp || !m->Ap)) || !m->step_sync) {
        nsl::set_error("nsl_moe_create: out of memory");
        nsl_moe_destroy(m);      // frees whatever was obtained
        return NULL;
    }
    return m;
}

void nsl_moe_set_layer(NslMoe* m, const WSlice* wg, const WSlice* wu, const WSlice* wd) { m->wg = wg; m->wu = wu; m->wd = wd; }
void nsl_moe_set_grouped_min_tokens(NslMoe* m, int t) { m->grouped_min_tokens = t; }
void nsl_moe_set_rounding(NslMoe* m, int bf16_points) { m->raw = !bf16_points; }
void nsl_moe_set_dependent_launch(NslMoe* m, int on) { m->pdl = on != 0; }
void nsl_moe_set_direct_output(NslMoe* m, int on) { m->direct_out = on != 0; }
void nsl_moe_set_one_launch(NslMoe* m, int on) { m->one_launch = on != 0; }

// 0, or 1 when a wait inside a one-launch decode step ran out since the last call (the step's output is then not valid).
// Reads device memory: call it after the layer's work has been waited for.
int nsl_moe_step_status(NslMoe* m) {
    int v = 0;
    if (cudaMemcpy(&v, m->step_sync, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(m->step_sync, 0, 4);
    return v;
}

void nsl_moe_destroy(NslMoe* m) {
    if (!m) return;
    void* dv[] = {m->x, m->wt, m->ind, m->A, m->Dx, m->out, m->Gb, m->xp, m->Ap, m->perm, m->tiles, m->ntiles, m->step_sync};
    for (void* p : dv) if (p) cudaFree(p);
    void* hv[] = {m->hx, m->hout, m->hind};
    for (void* p : hv) if (p) cudaFreeHost(p);
    if (m->stream) cudaStreamDestroy(m->stream);
    free(m);
}

// Device form: x [T][d] and logits [T][n_exp] in device memory -> out [T][d]; ind_out / wt_out (device, optional) get
// the routing.  Only launches are enqueued on s.
int nsl_moe_forward_dev(NslMoe* m, cudaStream_t s, const float* x, const float* logits, int T, float* out) {
    if (T < 1 || T > m->max_tokens) { nsl::set_error("nsl_moe_forward: %d rows, at most %d", T, m->max_tokens); return -1; }
    const int k = m->top_k, P = T * k, d = m->d, ff = m->ff;
    if (T >= m->grouped_min_tokens) {
        const int mt = P / MMT_BN + m->n_exp;
        nsl_route(s, m->n_exp, k, logits, m->n_exp, m->ind, m->wt, T);
        kc_bucket(s, m->ind, P, m->n_exp, m->perm, m->tiles, m->ntiles);
        // The rows are packed to bf16 once (every row tile of every expert reads them), the up projection is launched as
        // a dependent of the gate projection it does not depend on (its blocks fill the gate grid's last wave), and the
        // SwiGLU results (bf16 values) go to the down projection packed.  (SwiGLU in the up GEMM's epilogue measured
        // 27 us slower a layer.)
        kc_pack_input_bf16(s, x, m->xp, (size_t) T * d);
        kc_mm_grouped_packed(s, MF_SEED4P4, m->wg, d, ff, m->xp, d, m->Gb, ff, k, m->perm, m->tiles, m->ntiles, mt, m->G);
        nsl::tl_mm_overlap = true;
        kc_mm_grouped_packed(s, MF_SEED4P4, m->wu, d, ff, m->xp, d, m->A, ff, k, m->perm, m->tiles, m->ntiles, mt, m->G);
        nsl::tl_mm_overlap = false;
        nsl_swiglu_packed(s, m->Gb, m->A, m->Ap, P * ff);
        kc_mm_grouped_packed(s, MF_SEED4P4, m->wd, ff, d, m->Ap, ff, m->Dx, d, 1, m->perm, m->tiles, m->ntiles, mt, m->G);
        kq4_moe_combine(s, d, k, m->Dx, m->wt, NULL, NULL, 0, out, T);
        return 0;
    }
    // decode rows: three launches -- router + gate + up + SwiGLU (the router runs in that kernel's prologue), down, combine --
    // as dependent launches (a kernel's blocks come in while the previous kernel drains and wait for its completion
    // before touching anything a neighbour writes)
    nsl::PdlScope pdl(m->pdl);
    const bool fused = T <= MV_MAXT && d % 64 == 0 && d <= 2048 && (d & (d - 1)) == 0;
    // on request, one launch for the whole step where the fused kernel serves the sizes (measured slower than the three
    // dependent launches: 126.3 against 114.2 us at 8 rows, 70.1 / 65.5 at 4, 26.7 / 26.2 at 1)
    if (fused && m->one_launch &&
        nsl_mv_step(s, m->wg, m->wu, m->wd, d, ff, x, d, m->n_exp, k, logits, m->n_exp, T, m->ind, m->wt, m->A, m->Dx, out, m->raw, m->step_sync, m->G))
        return 0;
    if (fused) nsl_mv_gu_routed(s, m->wg, m->wu, d, ff, x, d, m->A, ff, m->n_exp, k, logits, m->n_exp, T, m->ind, m->wt, m->raw, m->G);
    else {
        nsl_route(s, m->n_exp, k, logits, m->n_exp, m->ind, m->wt, T);
        if (m->raw) nsl_mv_gu_raw(s, m->wg, m->wu, d, ff, x, d, m->A, ff, m->ind, P, k, m->G);
        else kc_mv_gu(s, MF_SEED4P4, m->wg, m->wu, d, ff, x, d, m->A, ff, m->ind, P, k, m->G);
    }
    if (m->raw) nsl_mv_raw(s, m->wd, ff, d, m->A, ff, m->Dx, d, m->ind, P, 1, m->G);
    else kc_mv_sel(s, MF_SEED4P4, m->wd, ff, d, m->A, ff, m->Dx, d, m->ind, P, 1, m->G);
    kq4_moe_combine(s, d, k, m->Dx, m->wt, NULL, NULL, 0, out, T);
    return 0;
}

// The pinned forms' device work: the inputs' copy, the layer, the result to pinned memory.  A full batch's rows and logits
// are adjacent in both staging blocks and travel as ONE copy; the combine kernel stores its rows straight into the pinned
// output (posted writes over PCIe: no device-to-host copy to launch and wait for) unless direct output is switched off.
static int submit_pinned(NslMoe* m, int T, const float* block = NULL) {
    if (T < 1 || T > m->max_tokens) { nsl::set_error("nsl_moe_forward: %d rows, at most %d", T, m->max_tokens); return -1; }
    const size_t xb = (size_t) T * m->d * 4, lb = (size_t) T * m->n_exp * 4;
    if (block) cudaMemcpyAsync(m->x, block, xb + lb, cudaMemcpyHostToDevice, m->stream);      // the caller's own pinned block (T == max_tokens)
    else if (T == m->max_tokens) cudaMemcpyAsync(m->x, m->hx, xb + lb, cudaMemcpyHostToDevice, m->stream);
    else {
        cudaMemcpyAsync(m->x, m->hx, xb, cudaMemcpyHostToDevice, m->stream);
        cudaMemcpyAsync(m->logits, m->hlogits, lb, cudaMemcpyHostToDevice, m->stream);
    }
    if (m->direct_out && xb <= 256 * 1024) return nsl_moe_forward_dev(m, m->stream, m->x, m->logits, T, m->hout);      // decode-sized results
    if (nsl_moe_forward_dev(m, m->stream, m->x, m->logits, T, m->out)) return -1;
    return cudaMemcpyAsync(m->hout, m->out, xb, cudaMemcpyDeviceToHost, m->stream) == cudaSuccess ? 0 : -1;
}

// Host form: x and logits in HOST memory, out to host memory.  Copies go through the layer's pinned staging buffers on
// its own stream; returns after the result is on the host (-1 on an argument or CUDA error).
int nsl_moe_forward_host(NslMoe* m, const float* x, const float* logits, int T, float* out, int32_t* ind_out) {
    if (T < 1 || T > m->max_tokens) { nsl::set_error("nsl_moe_forward: %d rows, at most %d", T, m->max_tokens); return -1; }
    const size_t xb = (size_t) T * m->d * 4, lb = (size_t) T * m->n_exp * 4;
    memcpy(m->hx, x, xb);
    memcpy(m->hlogits, logits, lb);
    if (submit_pinned(m, T)) return -1;
    if (ind_out) cudaMemcpyAsync(m->hind, m->ind, (size_t) T * m->top_k * 4, cudaMemcpyDeviceToHost, m->stream);
    if (cudaStreamSynchronize(m->stream) != cudaSuccess || cudaGetLastError() != cudaSuccess) {
        nsl::set_error("nsl_moe_forward_host: CUDA error");
        return -1;
    }
    memcpy(out, m->hout, xb);
    if (ind_out) memcpy(ind_out, m->hind, (size_t) T * m->top_k * 4);
    return 0;
}

// Pinned staging buffers, for callers that fill inputs in place and skip the two host copies.
float* nsl_moe_host_x(NslMoe* m) { return m->hx; }
float* nsl_moe_host_logits(NslMoe* m) { return m->hlogits; }
float* nsl_moe_host_out(NslMoe* m) { return m->hout; }
const int32_t* nsl_moe_dev_ind(NslMoe* m) { return m->ind; }
const float* nsl_moe_dev_wt(NslMoe* m) { return m->wt; }
cudaStream_t nsl_moe_stream(NslMoe* m) { return m->stream; }

// The same with inputs already in the pinned buffers and the result left there: H2D, the layer, D2H, one sync.
// nsl_moe_submit_pinned enqueues without waiting and nsl_moe_wait waits, so that a caller with two handles keeps two
// steps in flight (one's copies and launch latency under the other's kernels).
int nsl_moe_submit_pinned(NslMoe* m, int T) { return submit_pinned(m, T); }

// The same from the caller's own pinned memory: block = max_tokens rows of d floats followed by max_tokens rows of n_exp logits
// (a full batch), copied as it lies; the result lands in the layer's pinned output (nsl_moe_host_out).
int nsl_moe_submit_block(NslMoe* m, const float* block) {
    if (!block) { nsl::set_error("nsl_moe_submit_block: no input block"); return -1; }
    return submit_pinned(m, m->max_tokens, block);
}

int nsl_moe_wait(NslMoe* m) { return cudaStreamSynchronize(m->stream) == cudaSuccess ? 0 : -1; }

int nsl_moe_forward_pinned(NslMoe* m, int T) {
    if (nsl_moe_submit_pinned(m, T)) return -1;
    return nsl_moe_wait(m);
}

}   // extern "C"
