// Reorder/convert kernels with source element type __half, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(__half)
