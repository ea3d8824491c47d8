// Reorder/convert kernels with source element type __nv_bfloat16, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(__nv_bfloat16)
