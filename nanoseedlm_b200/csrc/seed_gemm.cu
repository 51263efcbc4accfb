// placeholder until the tcgen05 grouped GEMM lands: records an error, launches nothing
#include "common.cuh"
using namespace nsl;
extern "C" {
void kc_seed_gemm_f32(int on) { (void) on; }
void kc_mm(cudaStream_t, int, WSlice, int, int, const float*, int, float*, int, int, int, const uint32_t*) { set_error("kc_mm: not built yet"); }
void kc_mm_grouped(cudaStream_t, int, const WSlice*, int, int, const float*, int, float*, int, int, const int32_t*, const MmTile*, int, const uint32_t*) { set_error("kc_mm_grouped: not built yet"); }
void kc_mm_grouped_dev(cudaStream_t, int, const WSlice*, int, int, const float*, int, float*, int, int, const int32_t*, const MmTile*, const int32_t*, int, const uint32_t*) { set_error("kc_mm_grouped_dev: not built yet"); }
void kc_mm_packed(cudaStream_t, int, WSlice, int, int, const uint16_t*, int, float*, int, int, int, const uint32_t*) { set_error("kc_mm_packed: not built yet"); }
void kc_mm_grouped_packed(cudaStream_t, int, const WSlice*, int, int, const uint16_t*, int, float*, int, int, const int32_t*, const MmTile*, const int32_t*, int, const uint32_t*) { set_error("kc_mm_grouped_packed: not built yet"); }
}
