// Reorder/convert kernels with source element type float, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(float)
