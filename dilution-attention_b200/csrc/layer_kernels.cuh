// Memory-bound helpers around the attention kernels, for the model's attention layers:
// the head split of the fused q/k/v projection with rotary position embedding applied on the
// way (model.py:59-67 + rope.py:26-44), and its inverse for the backward.
//
// qkv: (B, T, 3, H, D) bf16, the output of c_attn viewed per head.  q, k, v: contiguous
// (B, H, T, D) bf16.  Rotary pairs are adjacent elements (2i, 2i+1); cos/sin come as bf16
// tables (T, D/2) built by the caller exactly as the reference builds them (fp32 angles, cast
// to the activation dtype), and the arithmetic follows the reference's bf16 tensor expression
// x * cos + rotate(x) * sin operation by operation (each product and the sum round to bf16).
// One thread moves 8 consecutive elements (16 bytes) of one head row of q, k and v.
#pragma once

#include "common.cuh"

namespace dil {
namespace layer {

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xffff0000u);
  f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xffff0000u);
  f[4] = __uint_as_float(r.z << 16); f[5] = __uint_as_float(r.z & 0xffff0000u);
  f[6] = __uint_as_float(r.w << 16); f[7] = __uint_as_float(r.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const uint32_t a = __bfloat16_as_ushort(__float2bfloat16_rn(lo));
  const uint32_t b = __bfloat16_as_ushort(__float2bfloat16_rn(hi));
  return a | (b << 16);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}

// x * cos + rotate(x) * sin on 8 elements = 4 pairs; sign = +1 forward, -1 for the inverse
// rotation of the backward (the transpose of a rotation).
__device__ __forceinline__ void rotate8(float* x, const float* c, const float* s, float sign) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float a = x[2 * p], b = x[2 * p + 1];
    const float sn = sign * s[p];
    x[2 * p] = bf16_round(bf16_round(a * c[p]) + bf16_round(-b * sn));
    x[2 * p + 1] = bf16_round(bf16_round(b * c[p]) + bf16_round(a * sn));
  }
}

// SPLIT: qkv -> q, k, v (forward).  !SPLIT: dq, dk, dv -> dqkv (backward).
// cos_t / sin_t may be null: no rotation (layers without position encoding).
template <bool SPLIT, int D>
__global__ void split_heads_rope_kernel(__nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q,
                                        __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v,
                                        const __nv_bfloat16* __restrict__ cos_t,
                                        const __nv_bfloat16* __restrict__ sin_t, int64_t batch, int64_t seq,
                                        int heads, const int* __restrict__ pos_dev,
                                        int64_t table_rows) {
  constexpr int SL = D / 8;                                  // 16-byte slices per head row
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = batch * seq * heads * SL;
  if (idx >= total) return;
  const int sl = (int)(idx % SL);
  const int h = (int)((idx / SL) % heads);
  const int64_t t = (idx / ((int64_t)SL * heads)) % seq;
  const int64_t b = idx / ((int64_t)SL * heads * seq);
  const int64_t in = ((b * seq + t) * 3 * heads + h) * D + sl * 8;          // q part; k: + heads*D; v: + 2*heads*D
  const int64_t out = ((b * heads + h) * seq + t) * D + sl * 8;
  float c[4] = {1.f, 1.f, 1.f, 1.f}, s[4] = {0.f, 0.f, 0.f, 0.f};
  const bool rot = cos_t != nullptr;
  if (rot) {
    // table row = position of the token: its row in this call, plus (a step inside a captured
    // graph, whose arguments are frozen) the first row's position read from device memory
    // (a position outside the table is held at its nearest row: wrong angles, no stray read)
    int64_t tr = t;
    if (pos_dev != nullptr) tr = min(max(t + (int64_t)*pos_dev, (int64_t)0), table_rows - 1);
    const uint2 cr = *reinterpret_cast<const uint2*>(cos_t + tr * (D / 2) + sl * 4);
    const uint2 sr = *reinterpret_cast<const uint2*>(sin_t + tr * (D / 2) + sl * 4);
    c[0] = __uint_as_float(cr.x << 16); c[1] = __uint_as_float(cr.x & 0xffff0000u);
    c[2] = __uint_as_float(cr.y << 16); c[3] = __uint_as_float(cr.y & 0xffff0000u);
    s[0] = __uint_as_float(sr.x << 16); s[1] = __uint_as_float(sr.x & 0xffff0000u);
    s[2] = __uint_as_float(sr.y << 16); s[3] = __uint_as_float(sr.y & 0xffff0000u);
  }
  __nv_bfloat16* heads_ptr[3] = {q, k, v};
#pragma unroll
  for (int part = 0; part < 3; ++part) {
    __nv_bfloat16* a = qkv + in + (int64_t)part * heads * D;
    __nv_bfloat16* o = heads_ptr[part] + out;
    float x[8];
    unpack8(*reinterpret_cast<const uint4*>(SPLIT ? a : o), x);
    if (rot && part < 2) rotate8(x, c, s, SPLIT ? 1.f : -1.f);
    *reinterpret_cast<uint4*>(SPLIT ? o : a) = pack8(x);
  }
}

}  // namespace layer
}  // namespace dil
