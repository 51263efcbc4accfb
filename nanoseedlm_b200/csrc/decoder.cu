// Host side of a whole MoE decoder step (include/nslm_decoder.h): the sequence of kernel launches the reference engine
// issues per decode forward (engine/qwen4_cuda.c:1096-1111, 1160-1176, 1023-1083), for BASELINE config 4's shape, on one
// GPU or with the routed experts sharded over the ranks of a peer-memory window (csrc/ep_p2p.cu).  Buffers are allocated at
// creation; a step only enqueues launches (and two event records / waits for the shared expert's side stream).
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "../../include/nslm_decoder.h"

extern "C" {
// declared in nslm_kernels.h / nslm_ep.h; the routed form of the gate+up mat-vec
void nsl_mv_gu_routed(cudaStream_t s, const WSlice* wg, const WSlice* wu, int K, int R, const float* x, int xs, float* a, int ys,
                      int n_exp, int top_k, const float* logits, int ld, int T, int32_t* ind, float* wt, int raw, const uint32_t* G);
void nsl_ep_p2p_plan(cudaStream_t s, NslEpWindow w, uint64_t ind_off, uint64_t wt_off, int k, int row_stride, int lo, int hi,
                     int lo2, int hi2, int upper, int32_t* sel, int32_t* xrow, float* wsel, int32_t* tok_off, int32_t* count);
void nsl_ep_p2p_route_dispatch(cudaStream_t s, NslEpWindow w, int n_exp, int top_k, const float* logits, int ld, const float* x,
                               int d, uint64_t ind_off, uint64_t wt_off, int32_t* ind_out, float* wt_out);
void nsl_ep_p2p_combine(cudaStream_t s, NslEpWindow w, const float* D, const float* wsel, const int32_t* tok_off, int d);
void nsl_ep_p2p_reduce(cudaStream_t s, NslEpWindow w, int d, float* out);
void nsl_route(cudaStream_t s, int n_exp, int top_k, const float* logits, int ld, int32_t* ind, float* wt, int T);

struct NslDecoder {
    NslDecoderCfg c;
    std::vector<NslDecoderLayer> L;
    WSlice embed, head;
    const uint16_t* norm_out;
    const uint32_t* G;
    bool ep;
    NslEpWindow win;
    uint64_t ind_off, wt_off;
    int chunk_rows;
    std::vector<void*> dev;
    // activations of a step
    float *x, *h, *q, *k, *v, *o, *logits, *wt, *A, *Dx, *As, *Gs, *Us, *sh, *br, *moe, *part, *lm, *inv, *ones, *wsel;
    int32_t *ind, *zero_sel, *sel, *xrow, *tok_off, *count;
    WSlice* shared_tab;      // device: per layer the shared expert's gate and up as one-entry tables
    std::vector<uint16_t*> kc, vc;
    cudaStream_t s2;
    cudaEvent_t ev_x, ev_sh;
};

static void* dec_alloc(NslDecoder* m, size_t n) {
    void* p = NULL;
    if (cudaMalloc(&p, n ? n : 16) != cudaSuccess) return NULL;
    cudaMemset(p, 0, n ? n : 16);
    m->dev.push_back(p);
    return p;
}

void nsl_decoder_destroy(NslDecoder* m) {
    if (!m) return;
    for (void* p : m->dev) cudaFree(p);
    if (m->ev_x) cudaEventDestroy(m->ev_x);
    if (m->ev_sh) cudaEventDestroy(m->ev_sh);
    if (m->s2) cudaStreamDestroy(m->s2);
    delete m;
}

static bool expand_dense(NslDecoder* m, WSlice& w, int K, int R);

NslDecoder* nsl_decoder_create(const NslDecoderCfg* cfg, const NslDecoderLayer* layers, WSlice embed, const uint16_t* norm_out,
                               WSlice head, const uint32_t* G, const NslEpWindow* win) {
    const NslDecoderCfg& c = *cfg;
    const int e_loc = c.exp_hi - c.exp_lo;
    if (c.n_layer < 1 || c.d < 64 || c.d % 64 || c.n_head < 1 || c.n_kv < 1 || c.n_head % c.n_kv || c.n_head / c.n_kv > 16 || c.n_exp < 1 ||
        c.n_exp > 1024 || c.top_k < 1 || c.top_k > 32 || c.top_k > c.n_exp || c.ff_exp % 64 || c.ff_shared % 64 || c.max_rows < 1 || c.ctx < 1 ||
        c.vocab < 1 || e_loc < 1 || c.exp_lo < 0 || c.exp_hi > c.n_exp) {
        nsl::set_error("nsl_decoder_create: unsupported configuration");
        return NULL;
    }
    if (win && (win->t_loc < 1 || win->t_loc > c.max_rows || (long long) win->n * win->t_loc * c.top_k > 65536)) {
        nsl::set_error("nsl_decoder_create: the window's rows per rank (%d) do not fit max_rows (%d)", win->t_loc, c.max_rows);
        return NULL;
    }
    NslDecoder* m = new NslDecoder();
    m->c = c;
    m->L.assign(layers, layers + c.n_layer);
    m->embed = embed; m->head = head; m->norm_out = norm_out; m->G = G;
    m->ep = win != NULL;
    if (win) {
        m->win = *win;
        const uint64_t row = 2ull * c.d;      // the dispatch chunk: t_loc bf16 rows, then ids, then weights, padded to whole rows
        m->ind_off = (uint64_t) win->t_loc * row;
        m->wt_off = m->ind_off + 4ull * win->t_loc * c.top_k;
        m->chunk_rows = (int) (win->chunk_bytes / row);
    }
    const size_t T = (size_t) c.max_rows, d = (size_t) c.d, HQ = (size_t) c.n_head * 128, HK = (size_t) c.n_kv * 128;
    const size_t Tall = win ? (size_t) win->n * win->t_loc : T, P = Tall * c.top_k;      // pairs a rank may see
    bool ok = true;
#define DEC_F(field, count) ok = ok && (m->field = (float*) dec_alloc(m, 4 * (size_t) (count))) != NULL
#define DEC_I(field, count) ok = ok && (m->field = (int32_t*) dec_alloc(m, 4 * (size_t) (count))) != NULL
    DEC_F(x, T * d); DEC_F(h, T * d); DEC_F(q, T * HQ); DEC_F(k, T * HK); DEC_F(v, T * HK); DEC_F(o, T * HQ);
    DEC_F(logits, T * (c.n_exp + 1)); DEC_F(wt, T * c.top_k); DEC_F(A, P * c.ff_exp); DEC_F(Dx, P * d);
    DEC_F(As, T * c.ff_shared); DEC_F(Gs, T * c.ff_shared); DEC_F(Us, T * c.ff_shared); DEC_F(sh, T * d); DEC_F(br, T * d); DEC_F(moe, T * d);
    DEC_F(part, T * c.n_head * 32 * 130); DEC_F(lm, T * (size_t) c.vocab); DEC_F(inv, 64); DEC_F(ones, T); DEC_F(wsel, P);
    DEC_I(ind, T * c.top_k); DEC_I(zero_sel, T); DEC_I(sel, P); DEC_I(xrow, P); DEC_I(tok_off, Tall + 1); DEC_I(count, 4);
    for (int l = 0; ok && l < c.n_layer; ++l) {
        uint16_t* kc = (uint16_t*) dec_alloc(m, 2 * T * c.ctx * HK);
        uint16_t* vc = (uint16_t*) dec_alloc(m, 2 * T * c.ctx * HK);
        ok = kc && vc;
        m->kc.push_back(kc);
        m->vc.push_back(vc);
    }
    ok = ok && (m->shared_tab = (WSlice*) dec_alloc(m, sizeof(WSlice) * 2 * (size_t) c.n_layer)) != NULL;
    ok = ok && cudaStreamCreateWithFlags(&m->s2, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&m->ev_x, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&m->ev_sh, cudaEventDisableTiming) == cudaSuccess;
    if (ok) {
        std::vector<float> inv(64), ones(T, 1.0f);
        for (int p = 0; p < 64; ++p) inv[p] = (float) std::pow((double) c.rope_theta, -(double) p / 64.0);
        std::vector<WSlice> st(2 * (size_t) c.n_layer);      // (the seed form: used when the dense matrices are not expanded)
        for (int l = 0; l < c.n_layer; ++l) { st[2 * l] = layers[l].sg; st[2 * l + 1] = layers[l].su; }
        ok = cudaMemcpy(m->inv, inv.data(), 256, cudaMemcpyHostToDevice) == cudaSuccess &&
             cudaMemcpy(m->ones, ones.data(), 4 * T, cudaMemcpyHostToDevice) == cudaSuccess &&
             cudaMemcpy(m->shared_tab, st.data(), sizeof(WSlice) * st.size(), cudaMemcpyHostToDevice) == cudaSuccess;
    }
    if (ok && c.dense_bf16) {
        const int dd = c.d, HQi = c.n_head * 128, HKi = c.n_kv * 128;
        for (int l = 0; ok && l < c.n_layer; ++l) {
            NslDecoderLayer& Ly = m->L[l];
            ok = expand_dense(m, Ly.wq, dd, HQi) && expand_dense(m, Ly.wk, dd, HKi) && expand_dense(m, Ly.wv, dd, HKi) && expand_dense(m, Ly.wo, HQi, dd) &&
                 expand_dense(m, Ly.router, dd, c.n_exp + 1) && expand_dense(m, Ly.sg, dd, c.ff_shared) && expand_dense(m, Ly.su, dd, c.ff_shared) &&
                 expand_dense(m, Ly.sd, c.ff_shared, dd);
        }
        ok = ok && cudaDeviceSynchronize() == cudaSuccess;
    }
    if (!ok) {
        nsl::set_error("nsl_decoder_create: out of memory");
        nsl_decoder_destroy(m);
        return NULL;
    }
    return m;
}


// y (+)= W x for T rows: the mat-vec for up to MV_MAXT rows, the tensor-core GEMM beyond (engine/qwen4_cuda.c: mv()).
static void dense(NslDecoder* m, cudaStream_t s, const WSlice& w, int K, int R, const float* x, float* y, int T, int add) {
    const int fmt = m->c.dense_bf16 ? MF_BF16 : MF_SEED4P4;
    if (T <= MV_MAXT) kc_mv(s, fmt, w, K, R, x, K, y, R, T, add, m->G);
    else kc_mm(s, fmt, w, K, R, x, K, y, R, T, add, m->G);
}

// A dense SEED4P4 matrix expanded once to BF16 [R][K] in device memory; w then points at the expansion.
static bool expand_dense(NslDecoder* m, WSlice& w, int K, int R) {
    uint16_t* out = (uint16_t*) dec_alloc(m, 2 * (size_t) R * K);
    if (!out) return false;
    nsl_decode_bf16(0, w, K, R, out, m->G);
    WSlice b;
    memset(&b, 0, sizeof b);
    b.p[0] = out;
    w = b;
    return true;
}

int nsl_decoder_step(NslDecoder* m, cudaStream_t s, const int32_t* ids, const RowInfo* ri, int T, int32_t* next) {
    const NslDecoderCfg& c = m->c;
    if (T < 1 || T > c.max_rows || (m->ep && T != m->win.t_loc)) {
        nsl::set_error("nsl_decoder_step: %d rows (1 .. %d%s)", T, c.max_rows, m->ep ? ", and equal to the window's rows per rank" : "");
        return -1;
    }
    const int d = c.d, HQ = c.n_head * 128, HK = c.n_kv * 128, k = c.top_k, ld = c.n_exp + 1, ff = c.ff_exp, fs = c.ff_shared;
    const AttnArgs aa = {c.n_head, c.n_kv, 128, 32, 1.0f / sqrtf(128.0f)};
    nsl::PdlScope pdl(true);      // the kernels that know how wait on the device for their predecessor; the others launch as usual
    kc_embed(s, MF_BF16, m->embed, d, ids, m->x, T);
    for (int l = 0; l < c.n_layer; ++l) {
        const NslDecoderLayer& L = m->L[l];
        KvView kv;
        memset(&kv, 0, sizeof kv);
        kv.a.k = m->kc[l]; kv.a.v = m->vc[l]; kv.nv = c.max_rows * c.ctx; kv.fmt = KV_BF16;
        // attention
        kc_gnorm(s, d, c.eps, m->x, L.norm_attn, m->h, T);
        dense(m, s, L.wq, d, HQ, m->h, m->q, T, 0);
        dense(m, s, L.wk, d, HK, m->h, m->k, T, 0);
        dense(m, s, L.wv, d, HK, m->h, m->v, T, 0);
        kc_rope_kv(s, m->q, m->k, m->v, kv, ri, m->inv, c.n_head, c.n_kv, T);
        kc_attn(s, aa, m->q, kv, ri, m->part, NULL, m->o, T);
        dense(m, s, L.wo, HQ, d, m->o, m->x, T, 1);      // x = bf16(x + bf16(Wo o))
        // experts: the shared one on the side stream, joined before the combine (engine/qwen4_cuda.c:1026-1032, 1076-1078)
        kc_gnorm(s, d, c.eps, m->x, L.norm_ffn, m->h, T);
        cudaEventRecord(m->ev_x, s);
        cudaStreamWaitEvent(m->s2, m->ev_x, 0);
        {
            nsl::PdlScope off(false);      // the side stream's first kernel follows an event, not a kernel
            if (T <= MV_MAXT && !c.dense_bf16) {
                kc_mv_gu(m->s2, MF_SEED4P4, m->shared_tab + 2 * l, m->shared_tab + 2 * l + 1, d, fs, m->h, d, m->As, fs, m->zero_sel, T, 1, m->G);
                kc_mv(m->s2, MF_SEED4P4, L.sd, fs, d, m->As, fs, m->sh, d, T, 0, m->G);
            } else {
                dense(m, m->s2, L.sg, d, fs, m->h, m->Gs, T, 0);
                dense(m, m->s2, L.su, d, fs, m->h, m->Us, T, 0);
                kc_swiglu(m->s2, m->Gs, m->Us, m->As, T * fs);
                dense(m, m->s2, L.sd, fs, d, m->As, m->sh, T, 0);
            }
        }
        cudaEventRecord(m->ev_sh, m->s2);
        dense(m, s, L.router, d, ld, m->h, m->logits, T, 0);
        if (!m->ep) {
            const int P = T * k;
            if (T <= MV_MAXT) nsl_mv_gu_routed(s, L.eg, L.eu, d, ff, m->h, d, m->A, ff, c.n_exp, k, m->logits, ld, T, m->ind, m->wt, 0, m->G);
            else {
                nsl_route(s, c.n_exp, k, m->logits, ld, m->ind, m->wt, T);
                kc_mv_gu(s, MF_SEED4P4, L.eg, L.eu, d, ff, m->h, d, m->A, ff, m->ind, P, k, m->G);
            }
            kc_mv_sel(s, MF_SEED4P4, L.ed, ff, d, m->A, ff, m->Dx, d, m->ind, P, 1, m->G);
            cudaStreamWaitEvent(s, m->ev_sh, 0);
            kq4_moe_combine(s, d, k, m->Dx, m->wt, m->sh, m->logits + c.n_exp, ld, m->br, T);
        } else {
            const NslEpWindow& w = m->win;
            const int P = w.n * w.t_loc * k;
            const void* recv = (const char*) w.win[w.me] + w.recv_off;
            nsl_ep_p2p_route_dispatch(s, w, c.n_exp, k, m->logits, ld, m->h, d, m->ind_off, m->wt_off, m->ind, m->wt);
            nsl_ep_p2p_plan(s, w, m->ind_off, m->wt_off, k, m->chunk_rows, c.exp_lo, c.exp_hi, 0, 0, 0, m->sel, m->xrow, m->wsel, m->tok_off, m->count);
            nsl_mv_gu_rows(s, L.eg, L.eu, d, ff, recv, d, 1, m->A, ff, m->sel, m->xrow, P, m->count, 0, m->G);
            nsl_mv_sel_rows(s, L.ed, ff, d, m->A, ff, m->Dx, d, m->sel, P, m->count, 0, m->G);
            nsl_ep_p2p_combine(s, w, m->Dx, m->wsel, m->tok_off, d);
            nsl_ep_p2p_reduce(s, w, d, m->moe);
            cudaStreamWaitEvent(s, m->ev_sh, 0);
            kq4_moe_combine(s, d, 1, m->moe, m->ones, m->sh, m->logits + c.n_exp, ld, m->br, T);      // the shared expert's share + the routed sum
        }
        nsl_residual_add(s, m->x, m->br, (size_t) T * d);
    }
    kc_gnorm(s, d, c.eps, m->x, m->norm_out, m->h, T);
    for (int t0 = 0; t0 < T; t0 += MV_MAXT) {
        const int n = T - t0 < MV_MAXT ? T - t0 : MV_MAXT;
        kc_mv(s, MF_Q4, m->head, d, c.vocab, m->h + (size_t) t0 * d, d, m->lm + (size_t) t0 * c.vocab, c.vocab, n, 0, NULL);
    }
    kc_argmax(s, m->lm, next, c.vocab, T);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

const float* nsl_decoder_hidden(const NslDecoder* m) { return m->x; }
const float* nsl_decoder_logits(const NslDecoder* m) { return m->lm; }
int nsl_decoder_copy_out(NslDecoder* m, int what, int T, float* dst) {
    if (T < 1 || T > m->c.max_rows) return -1;
    const size_t n = (size_t) T * (what ? (size_t) m->c.vocab : (size_t) m->c.d) * 4;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    return cudaMemcpy(dst, what ? m->lm : m->x, n, cudaMemcpyDeviceToDevice) == cudaSuccess ? 0 : -1;
}
uint16_t* nsl_decoder_kcache(NslDecoder* m, int layer) { return layer >= 0 && layer < m->c.n_layer ? m->kc[layer] : NULL; }
int nsl_decoder_fill_cache(NslDecoder* m, int layer, const uint16_t* k, const uint16_t* v, size_t n) {
    const size_t cap = (size_t) m->c.max_rows * m->c.ctx * m->c.n_kv * 128;
    if (layer < 0 || layer >= m->c.n_layer || n > cap) { nsl::set_error("nsl_decoder_fill_cache: layer %d or %zu values out of range", layer, n); return -1; }
    return cudaMemcpy(m->kc[layer], k, 2 * n, cudaMemcpyDeviceToDevice) == cudaSuccess &&
           cudaMemcpy(m->vc[layer], v, 2 * n, cudaMemcpyDeviceToDevice) == cudaSuccess ? 0 : -1;
}
uint16_t* nsl_decoder_vcache(NslDecoder* m, int layer) { return layer >= 0 && layer < m->c.n_layer ? m->vc[layer] : NULL; }

}   // extern "C"
