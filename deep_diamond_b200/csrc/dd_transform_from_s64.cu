// Reorder/convert kernels with source element type int64_t, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(int64_t)
