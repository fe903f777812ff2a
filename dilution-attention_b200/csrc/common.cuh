// Shared device helpers for the dilution-attention kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dil {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kCarryRows = 64;  // query rows per demand checkpoint (DILUTION_CARRY_ROWS)

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// 2^x and 1/x on the special-function unit (about 2^-22 relative error).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Geometry of one launch: local query rows [0, tq) sit at absolute positions
// q_off + i and see keys j <= q_off + i, j < tk.
struct Geom {
  int64_t n;      // batch*heads rows
  int tq, tk;     // local queries, keys
  int q_off;      // absolute position of local query 0
  float zscale;   // scale * log2(e): scores are kept in the log2 domain
  float scale;
  float eps;
};

}  // namespace dil
