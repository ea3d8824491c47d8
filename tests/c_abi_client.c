/* A plain C client of libdd_b200.so: what a host that is neither Python nor torch (the JVM through
 * FFM, a C++ service) does with the ABI.  Device memory comes from the CUDA runtime, every tensor
 * argument is a raw device pointer plus a descriptor.  Runs a reorder, an activation, a bias add
 * and a reduction on small tensors and checks them against arithmetic done here on the host.
 * Built and run by tests/test_gpu_c_client.py; exits 0 when everything matches. */
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../include/dd_b200.h"

#define CHECK_DD(call)                                                                   \
  do {                                                                                   \
    ddStatus_t st_ = (call);                                                             \
    if (st_ != DD_STATUS_SUCCESS) {                                                      \
      fprintf(stderr, "%s:%d %s -> %s (%s)\n", __FILE__, __LINE__, #call, ddGetErrorString(st_), \
              handle ? ddGetLastErrorMessage(handle) : "");                              \
      return 1;                                                                          \
    }                                                                                    \
  } while (0)
#define CHECK_CUDA(call)                                                                 \
  do {                                                                                   \
    cudaError_t e_ = (call);                                                             \
    if (e_ != cudaSuccess) {                                                             \
      fprintf(stderr, "%s:%d %s -> %s\n", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
      return 1;                                                                          \
    }                                                                                    \
  } while (0)

enum { N = 3, C = 8, H = 4, W = 8, TOTAL = N * C * H * W };

int main(void) {
  ddHandle_t handle = NULL;
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));
  CHECK_DD(ddCreate(&handle));
  CHECK_DD(ddSetStream(handle, stream));

  float *hx = (float *)malloc(sizeof(float) * TOTAL), *hy = (float *)malloc(sizeof(float) * TOTAL);
  for (int i = 0; i < TOTAL; i++) hx[i] = (float)((i * 37) % 101) / 16.0f - 3.0f;
  float *dx, *dy, *dbias, *dsum;
  CHECK_CUDA(cudaMalloc((void **)&dx, sizeof(float) * TOTAL));
  CHECK_CUDA(cudaMalloc((void **)&dy, sizeof(float) * TOTAL));
  CHECK_CUDA(cudaMalloc((void **)&dbias, sizeof(float) * C));
  CHECK_CUDA(cudaMalloc((void **)&dsum, sizeof(float) * C));
  CHECK_CUDA(cudaMemcpyAsync(dx, hx, sizeof(float) * TOTAL, cudaMemcpyHostToDevice, stream));

  ddTensorDescriptor_t nchw, nhwc, bias;
  CHECK_DD(ddCreateTensorDescriptor(&nchw));
  CHECK_DD(ddCreateTensorDescriptor(&nhwc));
  CHECK_DD(ddCreateTensorDescriptor(&bias));
  CHECK_DD(ddSetTensor4dDescriptor(nchw, DD_TENSOR_NCHW, DD_DATA_FLOAT, N, C, H, W));
  CHECK_DD(ddSetTensor4dDescriptor(nhwc, DD_TENSOR_NHWC, DD_DATA_FLOAT, N, C, H, W));
  CHECK_DD(ddSetTensor4dDescriptor(bias, DD_TENSOR_NCHW, DD_DATA_FLOAT, 1, C, 1, 1));
  const float one = 1.0f, zero = 0.0f, half = 0.5f;
  int bad = 0;

  /* 1. reorder nchw -> nhwc */
  CHECK_DD(ddTransformTensor(handle, &one, nchw, dx, &zero, nhwc, dy));
  CHECK_CUDA(cudaMemcpyAsync(hy, dy, sizeof(float) * TOTAL, cudaMemcpyDeviceToHost, stream));
  CHECK_CUDA(cudaStreamSynchronize(stream));
  for (int n = 0; n < N; n++)
    for (int c = 0; c < C; c++)
      for (int h = 0; h < H; h++)
        for (int w = 0; w < W; w++)
          if (hy[((n * H + h) * W + w) * C + c] != hx[((n * C + c) * H + h) * W + w]) bad++;
  printf("reorder: %s (%s)\n", bad ? "MISMATCH" : "ok", ddGetLastKernelName(handle));

  /* 2. relu in place on the nchw tensor, then y = relu(x) + 0.5 * bias[c] */
  ddActivationDescriptor_t relu;
  CHECK_DD(ddCreateActivationDescriptor(&relu));
  CHECK_DD(ddSetActivationDescriptor(relu, DD_ACTIVATION_RELU, DD_PROPAGATE_NAN, 0.0));
  CHECK_DD(ddActivationForward(handle, relu, &one, nchw, dx, &zero, nchw, dx));
  float hbias[C];
  for (int c = 0; c < C; c++) hbias[c] = (float)c - 2.0f;
  CHECK_CUDA(cudaMemcpyAsync(dbias, hbias, sizeof(hbias), cudaMemcpyHostToDevice, stream));
  CHECK_DD(ddAddTensor(handle, &half, bias, dbias, &one, nchw, dx));
  CHECK_CUDA(cudaMemcpyAsync(hy, dx, sizeof(float) * TOTAL, cudaMemcpyDeviceToHost, stream));
  CHECK_CUDA(cudaStreamSynchronize(stream));
  int bad2 = 0;
  for (int i = 0; i < TOTAL; i++) {
    const int c = (i / (H * W)) % C;
    const float want = (hx[i] > 0.0f ? hx[i] : 0.0f) + 0.5f * hbias[c];
    if (hy[i] != want) bad2++;
  }
  printf("relu + bias: %s (%s)\n", bad2 ? "MISMATCH" : "ok", ddGetLastKernelName(handle));

  /* 3. sum over (N, H, W) of what is in dx now */
  ddReduceTensorDescriptor_t red;
  CHECK_DD(ddCreateReduceTensorDescriptor(&red));
  CHECK_DD(ddSetReduceTensorDescriptor(red, DD_REDUCE_TENSOR_ADD, DD_DATA_FLOAT, DD_PROPAGATE_NAN));
  CHECK_DD(ddReduceTensor(handle, red, NULL, 0, NULL, 0, &one, nchw, dx, &zero, bias, dsum));
  float hsum[C];
  CHECK_CUDA(cudaMemcpyAsync(hsum, dsum, sizeof(hsum), cudaMemcpyDeviceToHost, stream));
  CHECK_CUDA(cudaStreamSynchronize(stream));
  int bad3 = 0;
  for (int c = 0; c < C; c++) {
    double want = 0.0, mag = 0.0;
    for (int n = 0; n < N; n++)
      for (int k = 0; k < H * W; k++) {
        want += hy[(n * C + c) * H * W + k];
        mag += fabs(hy[(n * C + c) * H * W + k]);
      }
    if (fabs(hsum[c] - want) > 1e-5 * fabs(want) + 8 * 6e-8 * mag) bad3++;
  }
  printf("reduce: %s (%s)\n", bad3 ? "MISMATCH" : "ok", ddGetLastKernelName(handle));

  /* 4. a bad call is reported, not executed */
  ddStatus_t st = ddTransformTensor(handle, &one, nchw, dx, &zero, bias, dy);
  printf("shape mismatch -> %s\n", ddGetErrorString(st));
  if (st == DD_STATUS_SUCCESS) bad++;

  ddDestroyReduceTensorDescriptor(red);
  ddDestroyActivationDescriptor(relu);
  ddDestroyTensorDescriptor(nchw);
  ddDestroyTensorDescriptor(nhwc);
  ddDestroyTensorDescriptor(bias);
  cudaFree(dx);
  cudaFree(dy);
  cudaFree(dbias);
  cudaFree(dsum);
  ddDestroy(handle);
  cudaStreamDestroy(stream);
  free(hx);
  free(hy);
  return (bad || bad2 || bad3) ? 2 : 0;
}
