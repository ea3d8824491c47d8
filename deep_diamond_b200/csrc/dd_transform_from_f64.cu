// Reorder/convert kernels with source element type double, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(double)
