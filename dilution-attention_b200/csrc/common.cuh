// Shared device helpers for the dilution-attention kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dil {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kCarryRows = 32;  // query rows per demand checkpoint of the fp32 kernels

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

// 2^x for x <= 0 on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5];
// a minimax polynomial gives 2^f (relative error 2.7e-6 with degree 4, 7.5e-5 with
// degree 3) and n is added to the exponent field.  The special-function unit does 16
// exponentials per clock and SM; kernels bound by it hand a fixed share of their
// exponentials to this routine, whose ten instructions go to otherwise idle issue slots.
template <int DEG>
__device__ __forceinline__ float poly_exp2(float x) {
  static_assert(DEG == 3 || DEG == 4, "degree 3 or 4");
  x = fmaxf(x, -125.f);
  const float r = x + 12582912.f;                 // 1.5 * 2^23: round(x) lands in the low mantissa bits
  const float f = x - (r - 12582912.f);
  float p;
  if (DEG == 4) {
    p = fmaf(f, 0.009570085443556309f, 0.05591784790158272f);
    p = fmaf(p, f, 0.240247443318367f);
    p = fmaf(p, f, 0.6931217908859253f);
    p = fmaf(p, f, 0.9999992847442627f);
  } else {
    p = fmaf(f, 0.05517148599028587f, 0.24261091649532318f);
    p = fmaf(p, f, 0.6932609677314758f);
    p = fmaf(p, f, 0.9999280571937561f);
  }
  return __int_as_float(__float_as_int(p) + (__float_as_int(r) << 23));
}

// Packed fp32 arithmetic (two lanes per instruction, sm_100): halves the issue slots of
// element-wise work on neighbouring values.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 r;
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return r;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 r;
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return r;
}
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
  float2 r;
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "sub.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return r;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 r;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(r.x), "=f"(r.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return r;
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
  int carry_rows; // query rows per demand checkpoint (16, 32 or 64)
  int bid;        // FORM of the bid: kBidSoftmax 2^(z - l), kBidSigmoid 1/(1 + 2^(l - z)), or one of the
                  // four f(a) / rowsum(f) bids (fp32 tile kernels only)
  int share;      // share step (kernels_bid.py:123-127): 1 inclusive, 2 exclusive history, 0 none
  int normalised; // the bid divides by its row sum (softmax, relu, relu2, softplus, minshift): there are
                  // row statistics and the backward has the Jacobian correction ghat; otherwise
                  // l = lshift for every row
  float lshift;   // log2 of the shift of expshift / sigshift (kernels_bid.py:19-26); 0 for the sigmoid
  int ghat_pass;  // reverse pass of an f(a) / rowsum(f) bid, whose Jacobian factor is unbounded (1 / row mass):
                  // 1 = accumulate ghat only, 2 = ghat is known and is subtracted BEFORE the factor
                  // multiplies (kernels_bid.py:718); 0 = one pass, correction afterwards (softmax: jac = p <= 1)
};

// Bid codes of the reference (kernels_bid.py:84) that are built, and the form each one takes:
// expshift = the softmax form without the row sum, sigshift = the sigmoid form, both with l = log2(shift).
constexpr int kBidSoftmax = 0, kBidSigmoid = 5, kBidExpshift = 6, kBidSigshift = 7;
// f(a) / rowsum(f) bids (kernels_bid.py:5-10, 206-225): relu(a), relu(a)^2, softplus(a), a - rowmin(a).
// Row statistics: rmax holds the row minimum for minshift (0 otherwise), rden the row sum of f;
// a row without mass (rden = 0) bids uniformly over its causal window, with a zero Jacobian.
constexpr int kBidRelu = 1, kBidRelu2 = 2, kBidSoftplus = 3, kBidMinshift = 4;
__host__ __device__ constexpr bool row_sum_bid(int bid) { return bid >= kBidRelu && bid <= kBidMinshift; }
__host__ __device__ constexpr int bid_form(int bid) {
  return row_sum_bid(bid) ? bid : (bid == kBidSigmoid || bid == kBidSigshift) ? kBidSigmoid : kBidSoftmax;
}
constexpr int kShareNone = 0, kShareInclusive = 1, kShareExclusive = 2;

// f of the scaled score a for the f(a) / rowsum(f) bids (minshift: the caller subtracts the row minimum).
// FAST: the special-function unit's exponential and logarithm (next to tf32 products; the absolute
// error of log(1 + e^-|a|), ~1e-7, is far below what the rounded products already carry).
template <bool FAST = false>
__device__ __forceinline__ float bid_mass(float a, int bid) {
  if (bid == kBidMinshift) return a;
  const float f = fmaxf(a, 0.f);
  if (bid == kBidRelu) return f;
  if (bid == kBidRelu2) return f * f;
  return f + (FAST ? __logf(1.f + __expf(-fabsf(a))) : log1pf(expf(-fabsf(a))));   // stable softplus
}

}  // namespace dil
