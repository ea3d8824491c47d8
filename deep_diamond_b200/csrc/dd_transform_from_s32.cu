// Reorder/convert kernels with source element type int32_t, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(int32_t)
