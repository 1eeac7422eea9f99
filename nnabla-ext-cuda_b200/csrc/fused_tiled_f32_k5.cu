// Tiled fused kernels: element type float, 5x5 kernel.
#define DWBNQ_INST_T float
#define DWBNQ_INST_K 5
#include "dwbnq_fused_tiled_inst.cuh"
