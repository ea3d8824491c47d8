// Reduce-tensor kernels for element type __half (accumulating in float).
#include "dd_reduce_kernels.cuh"

DD_REDUCE_DEFINE(__half, float)
