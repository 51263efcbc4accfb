"""B200 (sm_100a) seed-decode MoE kernels behind NanoSeedLM's CUDA kernel ABI.

lib      -- the C ABI (ctypes view of libnslm_b200.so); build -- the nvcc build; kernels -- the host-side mirror of the
reference's kernel test backend; moe -- synthetic expert layers and the handle of the C host layer."""
