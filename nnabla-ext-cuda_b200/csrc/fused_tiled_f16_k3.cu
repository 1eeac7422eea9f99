// Tiled fused kernels: element type __half, 3x3 kernel.
#define DWBNQ_INST_T __half
#define DWBNQ_INST_K 3
#include "dwbnq_fused_tiled_inst.cuh"
