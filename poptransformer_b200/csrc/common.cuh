// Shared host/device helpers for libpt_b200 (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pt_b200.h"

namespace pt {

// Records a thread-local message for pt_last_error() and returns `code`.
int set_error(int code, const char *fmt, ...);
void count_launch(int n = 1);
// Streaming multiprocessors of the current device (cached per device; 148 on B200).
int sm_count();

#define PT_REQUIRE(cond, ...)                                \
  do {                                                       \
    if (!(cond)) return pt::set_error(PT_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define PT_LAUNCH_CHECK(name)                                                         \
  do {                                                                                \
    cudaError_t e__ = cudaGetLastError();                                             \
    if (e__ != cudaSuccess)                                                           \
      return pt::set_error(PT_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e__));     \
    pt::count_launch();                                                               \
  } while (0)

#define PT_CUDA(call)                                                                 \
  do {                                                                                \
    cudaError_t e__ = (call);                                                         \
    if (e__ != cudaSuccess)                                                           \
      return pt::set_error(PT_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__));    \
  } while (0)

static inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

#ifdef __CUDACC__
// ---- fp16 arithmetic with the reference's "one rounding per op" semantics -------------
__device__ __forceinline__ __half h_mul(__half a, __half b) { return __hmul_rn(a, b); }
__device__ __forceinline__ __half h_add(__half a, __half b) { return __hadd_rn(a, b); }
__device__ __forceinline__ __half h_sub(__half a, __half b) { return __hsub_rn(a, b); }

// swish as the oracle defines it: x * sigmoid(x) in float32, one rounding to fp16.
__device__ __forceinline__ __half swish_h(__half x) {
  float f = __half2float(x);
  return __float2half_rn(f / (1.0f + expf(-f)));
}
// erf-GELU in float32, one rounding.
__device__ __forceinline__ __half gelu_h(__half x) {
  float f = __half2float(x);
  return __float2half_rn(0.5f * f * (1.0f + erff(f * 0.70710678118654752440f)));
}
__device__ __forceinline__ __half sigmoid_h(__half x) {
  float f = __half2float(x);
  return __float2half_rn(1.0f / (1.0f + expf(-f)));
}

// float -> OCP E4M3 (RNE, saturating to +-448) -> the exactly representable fp16 value.
__device__ __forceinline__ __half e4m3_round_h(float v) {
  __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  __half_raw r = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half(r);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x <= 1024; `red` holds >= 32 floats. All threads get the result.
// Deterministic: fixed shuffle tree, then warp 0 sums the per-warp values in order.
__device__ __forceinline__ float block_sum(float v, float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float block_max(float v, float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
  for (int i = 1; i < nw; ++i) t = fmaxf(t, red[i]);
  return t;
}
#endif  // __CUDACC__

}  // namespace pt
