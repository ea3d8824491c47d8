// Reduce-tensor kernels for element type __nv_bfloat16 (accumulating in float).
#include "dd_reduce_kernels.cuh"

DD_REDUCE_DEFINE(__nv_bfloat16, float)
