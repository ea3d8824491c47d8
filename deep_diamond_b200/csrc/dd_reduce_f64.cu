// Reduce-tensor kernels for element type double (accumulating in double).
#include "dd_reduce_kernels.cuh"

DD_REDUCE_DEFINE(double, double)
