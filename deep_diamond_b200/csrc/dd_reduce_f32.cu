// Reduce-tensor kernels for element type float (accumulating in float).
#include "dd_reduce_kernels.cuh"

DD_REDUCE_DEFINE(float, float)
