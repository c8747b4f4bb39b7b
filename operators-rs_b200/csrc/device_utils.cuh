// device_utils.cuh — small device-side helpers shared by the memory-bound kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace ops {

// 8 f16 values held as one 128-bit register quad.
union Pack8 {
  uint4 u;
  __half2 h2[4];
  __half h[8];
};
// The same for either 16-bit float type.
template <class T> union Vec8 {
  uint4 u;
  T h[8];
  __device__ __forceinline__ Vec8() {}
};
union Pack4 {
  uint2 u;
  __half2 h2[2];
  __half h[4];
};

__device__ __forceinline__ uint4 ld_global_16(const void *p) { return *reinterpret_cast<const uint4 *>(p); }
__device__ __forceinline__ void st_global_16(void *p, uint4 v) { *reinterpret_cast<uint4 *>(p) = v; }

// Streaming variants: data touched once should not evict what other kernels keep in L2.
__device__ __forceinline__ uint4 ld_stream_16(const void *p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_16(void *p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
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

// Block-wide reductions; every thread gets the result.  `scratch` holds >= 33 floats of shared memory
// and may be reused right after the call returns.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (nwarps == 1) return v;
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? scratch[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  if (nwarps == 1) return v;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

template <class T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

template <class T> __device__ __forceinline__ T *byte_off(T *p, long long off) {
  return reinterpret_cast<T *>(reinterpret_cast<char *>(p) + off);
}
template <class T> __device__ __forceinline__ const T *byte_off(const T *p, long long off) {
  return reinterpret_cast<const T *>(reinterpret_cast<const char *>(p) + off);
}

}  // namespace ops
