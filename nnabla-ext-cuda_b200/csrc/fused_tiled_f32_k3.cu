// Tiled fused kernels: element type float, 3x3 kernel.
#define DWBNQ_INST_T float
#define DWBNQ_INST_K 3
#include "dwbnq_fused_tiled_inst.cuh"
