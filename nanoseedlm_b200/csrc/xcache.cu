// Host side of the VRAM expert cache (include/nslm_cache.h): arena, pool, tables and the two upload paths.  What it
// mirrors in the reference: engine/qwen4_cuda.c:368-451 (build_cache), :1043-1056 (a layer's admit and copies),
// :1143-1162 (prefetch, layer_start).  All CUDA calls go through a table of function pointers (NslCacheOps) so that the
// logic runs against fakes on a machine without a GPU and can be made to fail at any call.
#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "../../include/nslm_cache.h"

namespace nsl {

static int real_host_alloc(void** p, size_t n, int mapped) { return cudaHostAlloc(p, n ? n : 16, mapped ? cudaHostAllocMapped : cudaHostAllocDefault) == cudaSuccess ? 0 : -1; }
static int real_host_free(void* p) { return cudaFreeHost(p) == cudaSuccess ? 0 : -1; }
static int real_dev_ptr(void** d, void* h) { return cudaHostGetDevicePointer(d, h, 0) == cudaSuccess ? 0 : -1; }
static int real_dev_alloc(void** p, size_t n) { return cudaMalloc(p, n ? n : 16) == cudaSuccess ? 0 : -1; }
static int real_dev_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
static int real_copy_async(void* dst, const void* src, size_t n, int kind, cudaStream_t s) {
    return cudaMemcpyAsync(dst, src, n, kind == 1 ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, s) == cudaSuccess ? 0 : -1;
}
static int real_fill_async(void* dst, int v, size_t n, cudaStream_t s) { return cudaMemsetAsync(dst, v, n, s) == cudaSuccess ? 0 : -1; }
static int real_stream_create(cudaStream_t* s) { return cudaStreamCreateWithFlags(s, cudaStreamNonBlocking) == cudaSuccess ? 0 : -1; }
static int real_stream_destroy(cudaStream_t s) { return cudaStreamDestroy(s) == cudaSuccess ? 0 : -1; }
static int real_stream_sync(cudaStream_t s) { return cudaStreamSynchronize(s) == cudaSuccess ? 0 : -1; }
static int real_event_create(cudaEvent_t* e) { return cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess ? 0 : -1; }
static int real_event_destroy(cudaEvent_t e) { return cudaEventDestroy(e) == cudaSuccess ? 0 : -1; }
static int real_event_record(cudaEvent_t e, cudaStream_t s) { return cudaEventRecord(e, s) == cudaSuccess ? 0 : -1; }
static int real_event_sync(cudaEvent_t e) { return cudaEventSynchronize(e) == cudaSuccess ? 0 : -1; }
static int real_stream_wait(cudaStream_t s, cudaEvent_t e) { return cudaStreamWaitEvent(s, e, 0) == cudaSuccess ? 0 : -1; }
static int real_admit(cudaStream_t s, const CachePool* p, int sl, const int32_t* inds, int count, int flags) {
    kc_cache_admit(s, p, sl, inds, count, flags);
    return 0;
}
static int real_copy_kernel(cudaStream_t s, const CachePool* p, int blocks) {
    kc_cache_copy(s, p, blocks);
    return 0;
}
static const NslCacheOps REAL_OPS = {real_host_alloc, real_host_free, real_dev_ptr, real_dev_alloc, real_dev_free, real_copy_async,
                                     real_fill_async, real_stream_create, real_stream_destroy, real_stream_sync, real_event_create,
                                     real_event_destroy, real_event_record, real_event_sync, real_stream_wait, real_admit, real_copy_kernel};
static NslCacheOps g_ops = REAL_OPS;

}   // namespace nsl

using namespace nsl;

extern "C" {

struct NslXCache {
    int layers, per_layer, units, slots;
    uint64_t len[3][4], ub;
    CachePool pool;                   // the layers' demand admits: jobs in device memory (the copy kernel reads them)
    CachePool pf;                     // the prefetch's admits: the same tables, its own job list
    int32_t *mail, *mail_pf;          // mapped pinned mailboxes [4 + 2 * per_layer]: [0] the job count, [4..] (unit, slot) pairs
    int32_t *mail_d, *mail_pf_d;      // their device addresses
    uint8_t* arena;                   // pinned, mapped: every unit
    int32_t* all_ids;                 // device: 0 .. per_layer - 1
    cudaStream_t cs;                  // the copy stream
    cudaEvent_t ev_admit, ev_copy;
    std::vector<cudaEvent_t> ev_ready;
    std::vector<char> ready_set;      // the layer's ready event has been recorded since it was last waited for
    std::vector<void*> dev, host;     // everything to release
    uint64_t up_units, up_bytes, up_runs;
    bool finished;
};

void nsl_xcache_set_ops(const NslCacheOps* ops) { g_ops = ops ? *ops : REAL_OPS; }

static void* xc_dev(NslXCache* c, size_t n) {
    void* p = NULL;
    if (g_ops.dev_alloc(&p, n) || !p) return NULL;
    c->dev.push_back(p);
    return p;
}
static void* xc_host(NslXCache* c, size_t n, int mapped) {
    void* p = NULL;
    if (g_ops.host_alloc(&p, n, mapped) || !p) return NULL;
    c->host.push_back(p);
    return p;
}

void nsl_xcache_destroy(NslXCache* c) {
    if (!c) return;
    if (c->cs) g_ops.stream_sync(c->cs);
    for (cudaEvent_t e : c->ev_ready) if (e) g_ops.event_destroy(e);
    if (c->ev_admit) g_ops.event_destroy(c->ev_admit);
    if (c->ev_copy) g_ops.event_destroy(c->ev_copy);
    if (c->cs) g_ops.stream_destroy(c->cs);
    for (void* p : c->dev) g_ops.dev_free(p);
    for (void* p : c->host) g_ops.host_free(p);
    delete c;
}

NslXCache* nsl_xcache_create(int layers, int per_layer, const uint64_t len[3][4], int slots) {
    if (layers < 1 || per_layer < 1 || per_layer > CACHE_MAX_PER_LAYER || !len) {
        set_error("nsl_xcache_create: %d layers x %d experts (1 .. %d per layer)", layers, per_layer, CACHE_MAX_PER_LAYER);
        return NULL;
    }
    NslXCache* c = new NslXCache();
    c->layers = layers; c->per_layer = per_layer; c->units = layers * per_layer;
    c->slots = slots > c->units ? c->units : slots < per_layer ? per_layer : slots;
    memcpy(c->len, len, sizeof c->len);
    CachePool& p = c->pool;
    memset(&p, 0, sizeof p);
    uint64_t ub = 0;
    for (int i = 0; i < 3; ++i)
        for (int s = 0; s < 4; ++s) {
            p.off[i][s] = len[i][s] ? (uint32_t) ub : 0xFFFFFFFFu;
            ub += (len[i][s] + 255) & ~255ull;      // every stream starts on a 256-byte boundary of its slot
        }
    c->ub = p.unit_bytes = ub;
    p.slots = c->slots; p.per_layer = per_layer; p.ntens = 3;
    bool ok = ub > 0;
    ok = ok && (c->arena = (uint8_t*) xc_host(c, ub * (uint64_t) c->units, 1)) != NULL;
    void* dh = NULL;
    ok = ok && g_ops.dev_ptr(&dh, c->arena) == 0;
    p.host = (const uint8_t*) dh;
    ok = ok && (p.vram = (uint8_t*) xc_dev(c, ub * (uint64_t) c->slots)) != NULL;
    ok = ok && (p.unit_slot = (int32_t*) xc_dev(c, 4 * (size_t) c->units)) != NULL;
    ok = ok && (p.slot_unit = (int32_t*) xc_dev(c, 4 * (size_t) c->slots)) != NULL;
    ok = ok && (p.slot_last = (uint32_t*) xc_dev(c, 4 * (size_t) c->slots)) != NULL;
    ok = ok && (p.tick = (uint32_t*) xc_dev(c, 16)) != NULL;
    ok = ok && (p.stats = (uint32_t*) xc_dev(c, 16)) != NULL;
    ok = ok && (p.jobs = (int32_t*) xc_dev(c, 8 * (size_t) per_layer)) != NULL;
    ok = ok && (p.njobs = (int32_t*) xc_dev(c, 16)) != NULL;
    ok = ok && (p.tab = (WSlice*) xc_dev(c, sizeof(WSlice) * (size_t) c->units * 3)) != NULL;
    c->pf = p;
    ok = ok && (c->pf.jobs = (int32_t*) xc_dev(c, 8 * (size_t) per_layer)) != NULL;
    ok = ok && (c->pf.njobs = (int32_t*) xc_dev(c, 16)) != NULL;
    ok = ok && (c->all_ids = (int32_t*) xc_dev(c, 4 * (size_t) per_layer)) != NULL;
    const size_t mail_bytes = 4 * (4 + 2 * (size_t) per_layer);
    ok = ok && (c->mail = (int32_t*) xc_host(c, mail_bytes, 1)) != NULL;
    ok = ok && (c->mail_pf = (int32_t*) xc_host(c, mail_bytes, 1)) != NULL;
    void *md = NULL, *mpd = NULL;
    ok = ok && g_ops.dev_ptr(&md, c->mail) == 0 && g_ops.dev_ptr(&mpd, c->mail_pf) == 0;
    c->mail_d = (int32_t*) md; c->mail_pf_d = (int32_t*) mpd;
    ok = ok && g_ops.stream_create(&c->cs) == 0;
    ok = ok && g_ops.event_create(&c->ev_admit) == 0 && g_ops.event_create(&c->ev_copy) == 0;
    c->ev_ready.assign(layers, (cudaEvent_t) NULL);
    c->ready_set.assign(layers, 0);
    for (int l = 0; ok && l < layers; ++l) ok = g_ops.event_create(&c->ev_ready[l]) == 0;
    if (!ok) {
        set_error("nsl_xcache_create: cannot allocate the cache (%.2f GB pinned arena, %.2f GB of slots)", (double) ub * c->units / 1e9,
                  (double) ub * c->slots / 1e9);
        nsl_xcache_destroy(c);
        return NULL;
    }
    return c;
}

uint8_t* nsl_xcache_host_unit(NslXCache* c, int unit) { return unit >= 0 && unit < c->units ? c->arena + (uint64_t) unit * c->ub : NULL; }
uint32_t nsl_xcache_offset(const NslXCache* c, int tensor, int stream) { return c->pool.off[tensor][stream]; }
uint64_t nsl_xcache_unit_bytes(const NslXCache* c) { return c->ub; }
const CachePool* nsl_xcache_pool(const NslXCache* c) { return &c->pool; }
const WSlice* nsl_xcache_table(const NslXCache* c, int layer, int tensor) {
    return c->pool.tab + ((size_t) layer * 3 + tensor) * c->per_layer;
}

}   // extern "C"

// ---- filling and the two upload paths ---------------------------------------------------------------------------------
extern "C" {

int nsl_xcache_finish(NslXCache* c, const int32_t* eb) {
    const int E = c->per_layer, NL = c->layers;
    CachePool& p = c->pool;
    std::vector<WSlice> tab((size_t) c->units * 3);
    memset(tab.data(), 0, sizeof(WSlice) * tab.size());
    std::vector<int32_t> us(c->units, -1), su(c->slots, -1), ids(E);
    for (int x = 0; x < E; ++x) ids[x] = x;
    for (int l = 0; l < NL; ++l)
        for (int i = 0; i < 3; ++i)
            for (int x = 0; x < E; ++x) tab[((size_t) l * 3 + i) * E + x].eb = eb ? eb[((size_t) l * 3 + i) * E + x] : 0;
    bool ok = true;
    int s = 0;
    for (int x = 0; x < E && s < c->slots; ++x)      // round-robin: every layer starts with the same share of the slots
        for (int l = 0; l < NL && s < c->slots; ++l, ++s) {
            const int u = l * E + x;
            us[u] = s;
            su[s] = u;
            ok = ok && g_ops.copy_async(p.vram + (uint64_t) s * c->ub, c->arena + (uint64_t) u * c->ub, c->ub, 1, c->cs) == 0;
            for (int i = 0; i < 3; ++i)
                for (int st = 0; st < 4; ++st)
                    if (c->len[i][st]) tab[((size_t) l * 3 + i) * E + x].p[st] = p.vram + (uint64_t) s * c->ub + p.off[i][st];
        }
    c->up_units += (uint64_t) s;
    c->up_bytes += (uint64_t) s * c->ub;
    const uint32_t tick0[4] = {CACHE_TICK_BASE, 0, 0, 0};
    ok = ok && g_ops.copy_async(p.unit_slot, us.data(), 4 * us.size(), 1, c->cs) == 0;
    ok = ok && g_ops.copy_async(p.slot_unit, su.data(), 4 * su.size(), 1, c->cs) == 0;
    ok = ok && g_ops.fill_async(p.slot_last, 0, 4 * (size_t) c->slots, c->cs) == 0;
    ok = ok && g_ops.copy_async(p.tick, tick0, 16, 1, c->cs) == 0;
    ok = ok && g_ops.fill_async(p.stats, 0, 16, c->cs) == 0;
    ok = ok && g_ops.fill_async(p.njobs, 0, 16, c->cs) == 0 && g_ops.fill_async(c->pf.njobs, 0, 16, c->cs) == 0;
    ok = ok && g_ops.copy_async(p.tab, tab.data(), sizeof(WSlice) * tab.size(), 1, c->cs) == 0;
    ok = ok && g_ops.copy_async(c->all_ids, ids.data(), 4 * (size_t) E, 1, c->cs) == 0;
    ok = g_ops.stream_sync(c->cs) == 0 && ok;      // the host vectors above are read by the copies until here
    if (!ok) { set_error("nsl_xcache_finish: a copy to the device failed"); return -1; }
    c->finished = true;
    return 0;
}

// The jobs an admit left in a mailbox, as runs of consecutive units that go to consecutive slots: one copy each.
static int copy_jobs(NslXCache* c, const int32_t* mail) {
    const int n = mail[0];
    if (n < 0 || n > c->per_layer) { set_error("expert cache: the admit reported %d jobs", n); return -1; }
    const int32_t* job = mail + 4;
    for (int j = 0; j < n;) {
        int k = j + 1;
        while (k < n && job[2 * k] == job[2 * (k - 1)] + 1 && job[2 * k + 1] == job[2 * (k - 1) + 1] + 1) ++k;
        const int unit = job[2 * j], slot = job[2 * j + 1];
        if (unit < 0 || unit + (k - j) > c->units || slot < 0 || slot + (k - j) > c->slots) { set_error("expert cache: job (%d, %d) out of range", unit, slot); return -1; }
        if (g_ops.copy_async(c->pool.vram + (uint64_t) slot * c->ub, c->arena + (uint64_t) unit * c->ub, c->ub * (uint64_t) (k - j), 1, c->cs)) {
            set_error("expert cache: the copy of units %d..%d to slot %d failed", unit, unit + (k - j) - 1, slot);
            return -1;
        }
        c->up_runs += 1;
        j = k;
    }
    c->up_units += (uint64_t) n;
    c->up_bytes += (uint64_t) n * c->ub;
    return 0;
}

// The admit with its job list in a mailbox the host can read, the wait for it, and the copies on the copy stream.
static int admit_and_dma(NslXCache* c, cudaStream_t s, const CachePool& base, int32_t* mail, int32_t* mail_d, int layer, const int32_t* inds,
                         int count, int flags) {
    CachePool p = base;
    p.njobs = mail_d;
    p.jobs = mail_d + 4;
    if (g_ops.admit(s, &p, layer, inds, count, flags) || g_ops.event_record(c->ev_admit, s) || g_ops.event_sync(c->ev_admit)) {
        set_error("expert cache: the admit of layer %d failed", layer);
        return -1;
    }
    // everything enqueued on s before the admit has finished too: no kernel still reads the slots about to be overwritten
    return copy_jobs(c, mail);
}

int nsl_xcache_fetch(NslXCache* c, cudaStream_t s, int layer, const int32_t* inds, int count, int mode) {
    if (!c->finished || layer < 0 || layer >= c->layers) { set_error("nsl_xcache_fetch: layer %d of %d (or the cache is not finished)", layer, c->layers); return -1; }
    if (mode == NSL_XCACHE_KERNEL) {
        if (g_ops.admit(s, &c->pool, layer, inds, count, 0) || g_ops.copy_kernel(s, &c->pool, 64)) { set_error("nsl_xcache_fetch: launch failed"); return -1; }
        return 0;
    }
    if (admit_and_dma(c, s, c->pool, c->mail, c->mail_d, layer, inds, count, 0)) return -1;
    if (g_ops.event_record(c->ev_copy, c->cs) || g_ops.stream_wait(s, c->ev_copy)) { set_error("nsl_xcache_fetch: event failed"); return -1; }
    return 0;
}

int nsl_xcache_prefetch(NslXCache* c, cudaStream_t s, int layer, int mode) {
    if (!c->finished || layer < 0 || layer >= c->layers) { set_error("nsl_xcache_prefetch: layer %d of %d (or the cache is not finished)", layer, c->layers); return -1; }
    if (c->slots < 2 * c->per_layer) {      // a layer's prefetch must not push out the layer that is running
        set_error("nsl_xcache_prefetch: %d slots, a prefetch needs room for two layers (%d)", c->slots, 2 * c->per_layer);
        return -1;
    }
    if (mode == NSL_XCACHE_KERNEL) {
        if (g_ops.admit(s, &c->pf, layer, c->all_ids, c->per_layer, 0) || g_ops.event_record(c->ev_admit, s) || g_ops.stream_wait(c->cs, c->ev_admit) ||
            g_ops.copy_kernel(c->cs, &c->pf, 8)) { set_error("nsl_xcache_prefetch: launch failed"); return -1; }
    } else if (admit_and_dma(c, s, c->pf, c->mail_pf, c->mail_pf_d, layer, c->all_ids, c->per_layer, 0)) return -1;
    if (g_ops.event_record(c->ev_ready[layer], c->cs)) { set_error("nsl_xcache_prefetch: event failed"); return -1; }
    c->ready_set[layer] = 1;
    return 0;
}

int nsl_xcache_layer_start(NslXCache* c, cudaStream_t s, int layer, int mode) {
    if (layer < 0 || layer >= c->layers) { set_error("nsl_xcache_layer_start: layer %d of %d", layer, c->layers); return -1; }
    if (!c->ready_set[layer] && nsl_xcache_prefetch(c, s, layer, mode)) return -1;      // the first layer, or a layer entered out of order
    if (g_ops.stream_wait(s, c->ev_ready[layer])) { set_error("nsl_xcache_layer_start: event failed"); return -1; }
    c->ready_set[layer] = 0;
    if (layer + 1 < c->layers) return nsl_xcache_prefetch(c, s, layer + 1, mode);
    return 0;
}

int nsl_xcache_stats(NslXCache* c, uint64_t* hits, uint64_t* misses, uint64_t* units, uint64_t* bytes, uint64_t* runs) {
    uint32_t st[4] = {0, 0, 0, 0};
    if (g_ops.stream_sync(c->cs) || g_ops.copy_async(st, c->pool.stats, 16, 2, c->cs) || g_ops.stream_sync(c->cs)) {
        set_error("nsl_xcache_stats: the device counters cannot be read");
        return -1;
    }
    if (hits) *hits = st[0];
    if (misses) *misses = st[1];
    if (units) *units = c->up_units;
    if (bytes) *bytes = c->up_bytes;
    if (runs) *runs = c->up_runs;
    return 0;
}

}   // extern "C"
