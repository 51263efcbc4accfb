/* nslm_cache.h - host side of the VRAM expert cache: the pinned arena, the pool of slots, and the upload paths.
 *
 * What the reference engine builds and drives around kc_cache_admit / kc_cache_copy (engine/qwen4_cuda.c:368-451
 * build_cache, :1043-1056 the layer's admit and copies, :1143-1162 prefetch and layer_start; engine/mova_cuda.c:311-404,
 * 1437-1446): a unit = one expert's gate, up and down streams at 256-byte aligned offsets; all units of all layers in a
 * pinned host arena; `slots` of them in VRAM, filled round-robin over the layers at start, then least-recently-used;
 * the layers' slice tables point at the slots and are rewritten by the admit kernel.
 *
 * Two ways to bring a missing unit into its slot:
 *   NSL_XCACHE_KERNEL  the copy kernel reads the arena (mapped pinned memory) over PCIe itself: no host involvement, the
 *                      form for decode steps, where the host must not wait for the router (engine/qwen4_cuda.c:1045);
 *   NSL_XCACHE_DMA     pinned asynchronous copies on a side stream: the admit kernel leaves its (unit, slot) jobs in a
 *                      mapped mailbox, the host reads them once the admit's event has fired and issues one
 *                      cudaMemcpyAsync per run of consecutive units and slots on the copy stream; the consumer stream
 *                      waits on the copies' event.  The copy engines move the bytes, no SM is used, but the host waits
 *                      for the admit: the form for prefill and large batches, where a layer takes milliseconds.
 * Calls return 0, or -1 with a message in nsl_last_error().  One host thread drives a cache. */
#pragma once
#include "nslm_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct NslXCache NslXCache;
enum { NSL_XCACHE_KERNEL = 0, NSL_XCACHE_DMA = 1 };

/* layers x per_layer units; len[i][s] = bytes of stream s of tensor i (gate, up, down) of ONE expert, 0 for a stream the
 * format does not have; slots = units kept in VRAM (clamped to [per_layer, layers * per_layer]).  Allocates the pinned
 * arena, the pool and the tables; NULL when something cannot be allocated (everything obtained so far is released). */
NslXCache* nsl_xcache_create(int layers, int per_layer, const uint64_t len[3][4], int slots);
void nsl_xcache_destroy(NslXCache* c);
/* Where the caller writes unit u = layer * per_layer + expert: stream s of tensor i at nsl_xcache_offset(c, i, s). */
uint8_t* nsl_xcache_host_unit(NslXCache* c, int unit);
uint32_t nsl_xcache_offset(const NslXCache* c, int tensor, int stream);
uint64_t nsl_xcache_unit_bytes(const NslXCache* c);
/* After the arena is filled: eb[layer][tensor][expert] (NULL: all 0) = the slices' exponent biases; fills the slots
 * round-robin over the layers (expert 0 of every layer, expert 1 of every layer, ...) by asynchronous copies on the copy
 * stream, uploads the tables, and waits for all of it. */
int nsl_xcache_finish(NslXCache* c, const int32_t* eb);
/* Device table of layer / tensor (0 gate, 1 up, 2 down): per_layer WSlice entries, kept current by the admits. */
const WSlice* nsl_xcache_table(const NslXCache* c, int layer, int tensor);
const CachePool* nsl_xcache_pool(const NslXCache* c);
/* A layer's demand path, after its router: bring the units inds[count] (device memory, expert ids of `layer`) that are
 * not in VRAM.  On return, work enqueued on s after this call finds them resident. */
int nsl_xcache_fetch(NslXCache* c, cudaStream_t s, int layer, const int32_t* inds, int count, int mode);
/* Every expert of `layer`: the admit on s (after the last reader of the slots it may replace), the copies on the copy
 * stream, the layer's ready event when they are done (engine/qwen4_cuda.c:1143-1151). */
int nsl_xcache_prefetch(NslXCache* c, cudaStream_t s, int layer, int mode);
/* At a layer's start (engine/qwen4_cuda.c:1156-1162): s waits for the layer's prefetch (issued here for layer 0), and
 * the next layer's prefetch is started. */
int nsl_xcache_layer_start(NslXCache* c, cudaStream_t s, int layer, int mode);
/* Totals since creation: hits and misses of the admits (device counters; synchronises), units and bytes uploaded, runs
 * (copies issued by the DMA form). */
int nsl_xcache_stats(NslXCache* c, uint64_t* hits, uint64_t* misses, uint64_t* units, uint64_t* bytes, uint64_t* runs);

/* The CUDA runtime calls and kernel launches the cache makes, replaceable as a table so that the host logic can be run
 * without a GPU and made to fail at a chosen call (tests).  NULL restores the real ones.  kind: 1 host->device,
 * 2 device->host.  Every function returns 0 on success. */
typedef struct {
    int (*host_alloc)(void** p, size_t bytes, int mapped);
    int (*host_free)(void* p);
    int (*dev_ptr)(void** d, void* host);              /* device address of mapped host memory */
    int (*dev_alloc)(void** p, size_t bytes);
    int (*dev_free)(void* p);
    int (*copy_async)(void* dst, const void* src, size_t bytes, int kind, cudaStream_t s);
    int (*fill_async)(void* dst, int value, size_t bytes, cudaStream_t s);
    int (*stream_create)(cudaStream_t* s);
    int (*stream_destroy)(cudaStream_t s);
    int (*stream_sync)(cudaStream_t s);
    int (*event_create)(cudaEvent_t* e);
    int (*event_destroy)(cudaEvent_t e);
    int (*event_record)(cudaEvent_t e, cudaStream_t s);
    int (*event_sync)(cudaEvent_t e);
    int (*stream_wait)(cudaStream_t s, cudaEvent_t e);
    int (*admit)(cudaStream_t s, const CachePool* p, int sl, const int32_t* inds, int count, int flags);
    int (*copy_kernel)(cudaStream_t s, const CachePool* p, int blocks);
} NslCacheOps;
void nsl_xcache_set_ops(const NslCacheOps* ops);

#ifdef __cplusplus
}
#endif
