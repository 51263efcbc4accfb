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

}   // namespace nsl
