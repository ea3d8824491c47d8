// ddTransformTensor / ddGatherTransform: planning (canonical iteration space, kernel family
// choice) and the bit-copy instantiations.  Typed conversions live in dd_transform_from_*.cu.
#include "dd_transform_kernels.cuh"

ddStatus_t dd_xform_raw(ddHandle_t h, int width, const ddXformPlan &pl) {
  switch (width) {
    case 1: return dd_xform_typed<uint8_t, uint8_t, float, true>(h, pl);
    case 2: return dd_xform_typed<uint16_t, uint16_t, float, true>(h, pl);
    case 4: return dd_xform_typed<uint32_t, uint32_t, float, true>(h, pl);
    case 8: return dd_xform_typed<uint64_t, uint64_t, float, true>(h, pl);
  }
  return DD_STATUS_INTERNAL_ERROR;
}

ddStatus_t dd_gather_raw(ddHandle_t h, int width, const ddGatherPlan &pl) {
  switch (width) {
    case 1: return dd_gather_typed<uint8_t, uint8_t, float, true>(h, pl);
    case 2: return dd_gather_typed<uint16_t, uint16_t, float, true>(h, pl);
    case 4: return dd_gather_typed<uint32_t, uint32_t, float, true>(h, pl);
    case 8: return dd_gather_typed<uint64_t, uint64_t, float, true>(h, pl);
  }
  return DD_STATUS_INTERNAL_ERROR;
}

static void plan_canon(ddCanon *c, const ddTensorStruct *xd, const ddTensorStruct *yd) {
  int64_t st[2][DD_DIM_MAX];
  for (int i = 0; i < xd->nd; i++) {
    st[0][i] = xd->strides[i];
    st[1][i] = yd->strides[i];
  }
  dd_canonicalize(c, xd->nd, xd->dims, 2, st, /*orderBy=*/1);
}

ddStatus_t dd_transform_impl(ddHandle_t h, double alpha, const ddTensorStruct *xd, const void *x,
                             double beta, const ddTensorStruct *yd, void *y) {
  if (h->faultWord && *(volatile int *)h->faultWord)
    DD_FAIL(h, DD_STATUS_EXECUTION_FAILED,
            "ddTransformTensor: an earlier transform/tile-tma kernel gave up waiting for a tile copy; its output is incomplete");
  ddXformPlan pl;
  plan_canon(&pl.canon, xd, yd);
  pl.alpha = alpha;
  pl.beta = beta;
  pl.x = x;
  pl.y = y;
  if (xd->dtype == yd->dtype && alpha == 1.0 && beta == 0.0)
    return dd_xform_raw(h, dd_type_size(xd->dtype), pl);
  switch (xd->dtype) {
    case DD_DATA_FLOAT: return dd_xform_from<float>(h, yd->dtype, pl);
    case DD_DATA_DOUBLE: return dd_xform_from<double>(h, yd->dtype, pl);
    case DD_DATA_HALF: return dd_xform_from<__half>(h, yd->dtype, pl);
    case DD_DATA_INT8: return dd_xform_from<int8_t>(h, yd->dtype, pl);
    case DD_DATA_INT32: return dd_xform_from<int32_t>(h, yd->dtype, pl);
    case DD_DATA_UINT8: return dd_xform_from<uint8_t>(h, yd->dtype, pl);
    case DD_DATA_BFLOAT16: return dd_xform_from<__nv_bfloat16>(h, yd->dtype, pl);
    case DD_DATA_INT64: return dd_xform_from<int64_t>(h, yd->dtype, pl);
  }
  DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddTransformTensor: unknown data type");
}

ddStatus_t dd_gather_transform_impl(ddHandle_t h, int count, const int64_t *srcOff,
                                    const int64_t *dstOff, const ddTensorStruct *xd, const void *x,
                                    const ddTensorStruct *yd, void *y) {
  ddGatherPlan pl;
  plan_canon(&pl.canon, xd, yd);
  pl.x = x;
  pl.y = y;
  pl.count = count;
  pl.so = srcOff;
  pl.do_ = dstOff;
  if (xd->dtype == yd->dtype) return dd_gather_raw(h, dd_type_size(xd->dtype), pl);
  switch (xd->dtype) {
    case DD_DATA_FLOAT: return dd_gather_from<float>(h, yd->dtype, pl);
    case DD_DATA_DOUBLE: return dd_gather_from<double>(h, yd->dtype, pl);
    case DD_DATA_HALF: return dd_gather_from<__half>(h, yd->dtype, pl);
    case DD_DATA_INT8: return dd_gather_from<int8_t>(h, yd->dtype, pl);
    case DD_DATA_INT32: return dd_gather_from<int32_t>(h, yd->dtype, pl);
    case DD_DATA_UINT8: return dd_gather_from<uint8_t>(h, yd->dtype, pl);
    case DD_DATA_BFLOAT16: return dd_gather_from<__nv_bfloat16>(h, yd->dtype, pl);
    case DD_DATA_INT64: return dd_gather_from<int64_t>(h, yd->dtype, pl);
  }
  DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddGatherTransform: unknown data type");
}
