// Host-side state of the library: the argument-error record, the launch counter, cached device properties and the
// host stream table.  The product fails loudly: a call it cannot serve launches nothing and records why.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

namespace nsl {

static char g_err[256];
static std::mutex g_err_mu;
static std::atomic<uint64_t> g_launches{0};
thread_local bool tl_pdl = false;

void set_error(const char* fmt, ...) {
    std::lock_guard<std::mutex> lk(g_err_mu);
    if (g_err[0]) return;   // keep the first
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    fprintf(stderr, "nslm_b200: %s\n", g_err);
}

void count_launch(int n) { g_launches.fetch_add((uint64_t) n, std::memory_order_relaxed); }

struct DevProps { int sms, smem; };
static DevProps props() {
    static DevProps cache[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cache[dev].sms) {
        int sms = 0, smem = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cache[dev].sms = sms > 0 ? sms : 148;
        cache[dev].smem = smem > 0 ? smem : 232448;
    }
    return cache[dev];
}
int sm_count() { return props().sms; }
int max_smem_optin() { return props().smem; }

}   // namespace nsl

extern "C" {

const char* nsl_last_error(void) {
    static thread_local char out[256];
    std::lock_guard<std::mutex> lk(nsl::g_err_mu);
    snprintf(out, sizeof out, "%s", nsl::g_err);
    nsl::g_err[0] = 0;
    return out;
}

uint64_t nsl_launch_count(void) { return nsl::g_launches.load(std::memory_order_relaxed); }
int nsl_sm_count(void) { return nsl::sm_count(); }
void nsl_dependent_launch(int on) { nsl::tl_pdl = on != 0; }

// The 32 stream bits that follow each seed: bit k is the top bit of the (k+1)-th state of the 16-bit LFSR with taps
// 0, 1, 3, 12 (reference: nslm/lfsr.h:20-23, 53-59).
void nsl_stream_table(uint32_t* t) {
    for (uint32_t s = 0; s < 65536; ++s) {
        uint32_t st = s, g = 0;
        for (int k = 0; k < 32; ++k) {
            const uint32_t fb = (st ^ (st >> 1) ^ (st >> 3) ^ (st >> 12)) & 1u;
            st = (st >> 1) | (fb << 15);
            g |= (st >> 15) << k;
        }
        t[s] = g;
    }
}

}   // extern "C"
