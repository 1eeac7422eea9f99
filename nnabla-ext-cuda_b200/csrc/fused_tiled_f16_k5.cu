// Tiled fused kernels: element type __half, 5x5 kernel.
#define DWBNQ_INST_T __half
#define DWBNQ_INST_K 5
#include "dwbnq_fused_tiled_inst.cuh"
