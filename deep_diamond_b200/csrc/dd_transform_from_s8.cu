// Reorder/convert kernels with source element type int8_t, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(int8_t)
