// Reorder/convert kernels with source element type uint8_t, for every destination type.
#include "dd_transform_kernels.cuh"

DD_XFORM_DEFINE_FROM(uint8_t)
