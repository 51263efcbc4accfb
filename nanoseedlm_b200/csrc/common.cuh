// Host-side helpers shared by the launchers: error record, launch counter, device properties.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nslm_kernels.h"

namespace nsl {

void set_error(const char* fmt, ...);
void count_launch(int n = 1);
int sm_count();
int max_smem_optin();

inline bool aligned16(const void* p) { return ((uintptr_t) p & 15u) == 0; }

// Programmatic dependent launch.  While a PdlScope(true) is alive on the calling thread, launch() marks the kernel as
// allowed to start before the previous kernel in its stream has finished: its blocks become resident as the previous
// kernel's blocks retire and run their prologue (the stream table, index arithmetic) until grid_dependency_wait(),
// which returns once the previous kernel has completed and its writes are visible.  Every kernel launched through
// launch() calls grid_dependency_wait() before it reads or writes anything a neighbouring kernel touches; without the
// scope the launch is an ordinary one and the wait returns at once.
extern thread_local bool tl_pdl;
extern thread_local bool tl_mm_overlap;   // seed_gemm.cu: the next GEMM launch is independent of its predecessor in the stream
struct PdlScope {
    bool prev;
    explicit PdlScope(bool on) : prev(tl_pdl) { tl_pdl = on; }
    ~PdlScope() { tl_pdl = prev; }
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tl_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_go() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

}   // namespace nsl
