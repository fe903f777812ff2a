// fp32-tile kernels for every pass of dilution attention (forward and backward).
//
// These serve dot_precision "ieee" and "tf32" (the reference's
// tl.dot(input_precision=...), kernels.py:81-92) and every dtype / head_dim the
// tcgen05 path is not built for.  Products run on 64x64 tiles staged in shared
// memory as fp32, either as plain FFMA ("ieee") or as warp-level tf32 tensor-core
// products with fp32 accumulation (everything else); all softmax / cumsum / share
// arithmetic is fp32.
//
// Layout of one CTA: 256 threads, one 64x64 (query x key) tile at a time.
//   FFMA: thread (ty = tid/16, tx = tid%16) owns tile rows ty+16r, columns tx+16c;
//   MMA:  warp w owns rows 16*(w%4).., columns (N/2)*(w/4).. of a [64 x N] result.
// Shared tiles of operands are [64][D+4] fp32 (float4-aligned, conflict-free
// for the access patterns below); score tiles are [64][68].
#pragma once

#include "common.cuh"

namespace dil {
namespace simt {

constexpr int TS = 64;    // tile side
static_assert(TS == 2 * kCarryRows, "two demand checkpoints per tile");
constexpr int NT = 256;   // threads per CTA
constexpr int SL = 68;    // leading dimension of score tiles (4 mod 32: conflict-free MMA fragments)

template <int D> __host__ __device__ constexpr int ld() { return D + 4; }

// Products come in two flavours.  MMA = false: fp32 FMAs, exact (dot_precision "ieee").
// MMA = true: warp-level tensor-core products on tf32 operands with fp32 accumulation
// (mma.sync m16n8k8) — what the reference's "tf32" mode means for fp32 tensors
// (kernels.py:318-325), and exact on bf16 tensors' values, which tf32 holds without loss.
// The eight warps of a CTA tile a [64 x N] result as 4 row groups of 16 x 2 column groups of N/2.
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Element-wise arithmetic follows the product flavour: exact division and exp2f next to the fp32
// FMAs, the special-function unit's approximations (about 2^-22 relative) next to tf32 products.
// An MMA operand is rounded to tf32 once, where it is written to shared memory, so that fragment
// loads are plain loads.
template <bool MMA> __device__ __forceinline__ float op_round(float x) {
  return MMA ? __uint_as_float(to_tf32(x)) : x;
}
template <bool MMA> __device__ __forceinline__ float recip(float x) { return MMA ? fast_rcp(x) : 1.f / x; }
template <bool MMA> __device__ __forceinline__ float ratio(float a, float b) { return MMA ? a * fast_rcp(b) : a / b; }
template <bool MMA> __device__ __forceinline__ float pow2(float x) { return MMA ? fast_exp2(x) : exp2f(x); }

// Which element of a [64 x D] result a thread's accumulator acc[r][c] holds.
template <bool MMA, int D> struct Frag {
  static __device__ __forceinline__ int row(int r, int /*c*/) { return (threadIdx.x >> 4) + 16 * r; }
  static __device__ __forceinline__ int col(int /*r*/, int c) { return (threadIdx.x & 15) + 16 * c; }
};
template <int D> struct Frag<true, D> {
  // r = register of the m16n8 fragment, c = 8-column tile of the warp's D/2 columns
  static __device__ __forceinline__ int row(int r, int /*c*/) {
    return 16 * ((threadIdx.x >> 5) & 3) + ((threadIdx.x & 31) >> 2) + 8 * (r >> 1);
  }
  static __device__ __forceinline__ int col(int r, int c) {
    return (D / 2) * (threadIdx.x >> 7) + 8 * c + 2 * (threadIdx.x & 3) + (r & 1);
  }
};

// Rows [row0, row0+64) of a (rows_total, D) row-major matrix -> fp32 smem tile, 16 bytes per
// load (rows start 16-byte aligned: D is a multiple of 16 elements).  Rows past the end are zero.
// ROUND: fp32 values are rounded to tf32 on the way (bf16 values are tf32 values already).
template <typename T, int D, bool ROUND = false>
__device__ __forceinline__ void load_tile(float* s, const T* __restrict__ g, int row0,
                                          int rows_total) {
  constexpr int LD = ld<D>();
  constexpr int E = 16 / (int)sizeof(T);     // elements per load: 4 fp32 or 8 bf16
  constexpr int PER_ROW = D / E;
  for (int idx = threadIdx.x; idx < TS * PER_ROW; idx += NT) {
    const int r = idx / PER_ROW, c = (idx % PER_ROW) * E;
    const int gr = row0 + r;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (gr < rows_total) raw = *reinterpret_cast<const uint4*>(g + (int64_t)gr * D + c);
    float* dst = s + r * LD + c;
    if (sizeof(T) == 4) {
      if (ROUND) {
        raw.x = to_tf32(__uint_as_float(raw.x));
        raw.y = to_tf32(__uint_as_float(raw.y));
        raw.z = to_tf32(__uint_as_float(raw.z));
        raw.w = to_tf32(__uint_as_float(raw.w));
      }
      *reinterpret_cast<uint4*>(dst) = raw;
    } else {
      // bf16 -> fp32 is a 16-bit shift
      *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                                    __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
      *reinterpret_cast<float4*>(dst + 4) = make_float4(__uint_as_float(raw.z << 16), __uint_as_float(raw.z & 0xffff0000u),
                                                        __uint_as_float(raw.w << 16), __uint_as_float(raw.w & 0xffff0000u));
    }
  }
}

// C[i][j] = sum_d A[i][d] * B[j][d]   (A, B: [64][D+4]; C: [64][SL])
template <int D, bool MMA>
__device__ __forceinline__ void score_tile(const float* A, const float* B, float* C) {
  constexpr int LD = ld<D>();
  if (MMA) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3, r0 = 16 * (warp & 3), c0 = 32 * (warp >> 2);
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
#pragma unroll 2
    for (int k0 = 0; k0 < D; k0 += 8) {
      // both tiles hold tf32 values (load_tile)
      const uint32_t a[4] = {__float_as_uint(A[(r0 + g) * LD + k0 + t]), __float_as_uint(A[(r0 + g + 8) * LD + k0 + t]),
                             __float_as_uint(A[(r0 + g) * LD + k0 + t + 4]),
                             __float_as_uint(A[(r0 + g + 8) * LD + k0 + t + 4])};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float* brow = B + (c0 + 8 * nt + g) * LD + k0 + t;
        const uint32_t b[2] = {__float_as_uint(brow[0]), __float_as_uint(brow[4])};
        mma_tf32(acc[nt], a, b);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float* c = C + (r0 + g) * SL + c0 + 8 * nt + 2 * t;
      c[0] = acc[nt][0];
      c[1] = acc[nt][1];
      c[8 * SL] = acc[nt][2];
      c[8 * SL + 1] = acc[nt][3];
    }
    return;
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
#pragma unroll 4
  for (int d = 0; d < D; d += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const float4*>(&A[(ty + 16 * r) * LD + d]);
#pragma unroll
    for (int c = 0; c < 4; ++c) b[c] = *reinterpret_cast<const float4*>(&B[(tx + 16 * c) * LD + d]);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc[r][c] = fmaf(a[r].x, b[c].x, acc[r][c]);
        acc[r][c] = fmaf(a[r].y, b[c].y, acc[r][c]);
        acc[r][c] = fmaf(a[r].z, b[c].z, acc[r][c]);
        acc[r][c] = fmaf(a[r].w, b[c].w, acc[r][c]);
      }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) C[(ty + 16 * r) * SL + tx + 16 * c] = acc[r][c];
}

// acc[r][c] += sum_j A(i,j) * B[j][col],  (i, col) = Frag<MMA, D>::row / col (r, c).
// A is a [64][SL] score tile, read transposed when TRANS_A (A(i,j) = A[j][i]).  With tf32 products B
// holds tf32 values (load_tile) and so does A unless CVT_A asks for the rounding here.
template <int D, bool TRANS_A, bool MMA, bool CVT_A = false>
__device__ __forceinline__ void accum_tile(const float* A, const float* B, float (&acc)[4][D / 16]) {
  constexpr int LD = ld<D>();
  constexpr int DC = D / 16;
  if (MMA) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3, r0 = 16 * (warp & 3), c0 = (D / 2) * (warp >> 2);
    float c4[DC][4];
#pragma unroll
    for (int nt = 0; nt < DC; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) c4[nt][i] = acc[i][nt];
#pragma unroll 2
    for (int k0 = 0; k0 < TS; k0 += 8) {
      // The eight k of a step are taken in the order 0,2,4,6,1,3,5,7 (fragment index t holds
      // rows k0+2t and k0+2t+1) in A and B alike, which leaves the sum unchanged and makes the
      // loads below fall on distinct banks: row strides are 4 mod 32 words, so 2t rows apart is
      // 8t banks apart and the eight columns g fill the gap.
      float af[4];
      if (TRANS_A) {
        af[0] = A[(k0 + 2 * t) * SL + r0 + g];
        af[1] = A[(k0 + 2 * t) * SL + r0 + g + 8];
        af[2] = A[(k0 + 2 * t + 1) * SL + r0 + g];
        af[3] = A[(k0 + 2 * t + 1) * SL + r0 + g + 8];
      } else {
        const float2 lo = *reinterpret_cast<const float2*>(&A[(r0 + g) * SL + k0 + 2 * t]);
        const float2 hi = *reinterpret_cast<const float2*>(&A[(r0 + g + 8) * SL + k0 + 2 * t]);
        af[0] = lo.x;
        af[1] = hi.x;
        af[2] = lo.y;
        af[3] = hi.y;
      }
      uint32_t a[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = CVT_A ? to_tf32(af[i]) : __float_as_uint(af[i]);
#pragma unroll
      for (int nt = 0; nt < DC; ++nt) {
        const float* bcol = B + (k0 + 2 * t) * LD + c0 + 8 * nt + g;
        const uint32_t b[2] = {__float_as_uint(bcol[0]), __float_as_uint(bcol[LD])};
        mma_tf32(c4[nt], a, b);
      }
    }
#pragma unroll
    for (int nt = 0; nt < DC; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i][nt] = c4[nt][i];
    return;
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll 4
  for (int j = 0; j < TS; ++j) {
    float a[4], b[DC];
#pragma unroll
    for (int r = 0; r < 4; ++r) a[r] = TRANS_A ? A[j * SL + ty + 16 * r] : A[(ty + 16 * r) * SL + j];
#pragma unroll
    for (int c = 0; c < DC; ++c) b[c] = B[j * LD + tx + 16 * c];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
  }
}

// Row statistics of local rows [ib*64, ib*64+64) into shared arrays (rinv = 1/rden;
// both zero for rows past tq so that their p is exactly zero).
// A bid without a row sum has no row statistics (kernels_bid.py:259-262): null pointers, and
// every row's exponent is log2 of the shift.  For the f(a) / rowsum(f) bids sM is the row minimum
// (minshift) or 0, a row without mass gets rinv = 0 and sU = 1 / (keys in its causal window), the
// uniform bid it falls back to (kernels_bid.py:206-225); sU is 0 everywhere else.
__device__ __forceinline__ void load_stats(float* sM, float* sRinv, float* sU, const float* rmax,
                                           const float* rden, int64_t n, int ib, const Geom& g) {
  if (threadIdx.x < TS) {
    const int i = ib * TS + threadIdx.x;
    const bool ok = i < g.tq;
    float m = g.lshift, r = ok ? 1.f : 0.f, u = 0.f;
    if (rmax != nullptr) {
      m = ok ? rmax[n * g.tq + i] : 0.f;
      const float den = ok ? rden[n * g.tq + i] : 0.f;
      if (row_sum_bid(g.bid)) {
        r = den > 0.f ? 1.f / den : 0.f;
        u = (ok && !(den > 0.f)) ? 1.f / (float)(min(g.q_off + i, g.tk - 1) + 1) : 0.f;
      } else {
        r = ok ? 1.f / den : 0.f;
      }
    }
    sM[threadIdx.x] = m;
    sRinv[threadIdx.x] = r;
    sU[threadIdx.x] = u;
  }
}

// The bid of one raw score (kernels_bid.py:191-225): softmax from the row statistics, the
// element-wise sigmoid of the scaled score (m = log2 of the shift, 0 for the plain sigmoid), or
// f(a) * rinv (+ the uniform fall-back of a row without mass).
template <bool MMA>
__device__ __forceinline__ float bid_value(float score, const Geom& g, float m, float rinv, float unif) {
  if (row_sum_bid(g.bid)) {
    const float a = score * g.scale;
    const float f = g.bid == kBidMinshift ? fmaxf(a - m, 0.f) : bid_mass<MMA>(a, g.bid);
    return fmaf(f, rinv, unif);
  }
  const float z = score * g.zscale;
  return g.bid == kBidSigmoid ? recip<MMA>(1.f + pow2<MMA>(m - z)) : pow2<MMA>(z - m) * rinv;
}

// jac, the diagonal factor of dp/da (da = jac * (dp - ghat), kernels_bid.py:187-225), from the bid
// itself (the tile no longer holds the score): relu p > 0 <=> a > 0; relu2 p = f^2 r so
// 2 f r = 2 sqrt(p r); softplus f = p / r and sigmoid(a) = 1 - e^-f; minshift r inside the causal
// window (`inside`).  A row without mass has rinv = 0 and with it a zero Jacobian.
template <bool MMA>
__device__ __forceinline__ float bid_jac_of_bid(float p, const Geom& g, float rinv, bool inside) {
  if (g.bid == kBidSoftmax) return p;
  if (g.bid == kBidSigmoid) return p * (1.f - p);
  if (g.bid == kBidRelu) return p > 0.f ? rinv : 0.f;
  if (g.bid == kBidRelu2) return 2.f * sqrtf(p * rinv);
  if (g.bid == kBidSoftplus) {
    if (!(rinv > 0.f)) return 0.f;
    return MMA ? (1.f - __expf(-p * fast_rcp(rinv))) * rinv : -expm1f(-p / rinv) * rinv;
  }
  return inside ? rinv : 0.f;
}

__device__ __forceinline__ int first_query_block(int jb, int q_off) {
  const int k0 = jb * TS;
  return k0 > q_off ? (k0 - q_off) / TS : 0;
}

// ---------------------------------------------------------------- pass 1
// grid = n * ceil(tq/64), longest rows first.
template <typename T, int D, bool MMA>
__global__ void __launch_bounds__(NT) rowstats_kernel(const T* __restrict__ q,
                                                      const T* __restrict__ k, Geom g,
                                                      float* __restrict__ rmax,
                                                      float* __restrict__ rden) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = ld<D>();
  float* sQ = smem;
  float* sK = sQ + TS * LD;
  float* sS = sK + TS * LD;
  const int nqb = (g.tq + TS - 1) / TS;
  const int64_t n = blockIdx.x % g.n;
  const int ib = nqb - 1 - (int)(blockIdx.x / g.n);
  load_tile<T, D, MMA>(sQ, q + n * g.tq * D, ib * TS, g.tq);

  const int r = threadIdx.x >> 2, part = threadIdx.x & 3;
  const int ia = g.q_off + ib * TS + r;
  const bool mass = row_sum_bid(g.bid);          // f(a) / rowsum(f): the sum of f, and the row minimum
  float m = mass ? INFINITY : -INFINITY, s = 0.f;
  const int last_key = min(g.tk - 1, g.q_off + ib * TS + TS - 1);
  const int njb = last_key / TS + 1;
  for (int jb = 0; jb < njb; ++jb) {
    __syncthreads();
    load_tile<T, D, MMA>(sK, k + n * g.tk * D, jb * TS, g.tk);
    __syncthreads();
    score_tile<D, MMA>(sQ, sK, sS);
    __syncthreads();
    if (mass) {                                  // kernels_bid.py:326-338
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const int ja = jb * TS + part * 16 + c;
        if (ja > ia || ja >= g.tk) continue;
        const float a = sS[r * SL + part * 16 + c] * g.scale;
        s += bid_mass<MMA>(a, g.bid);
        m = fminf(m, a);
      }
      continue;
    }
    float z[16];
    float tmax = -INFINITY;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const int ja = jb * TS + part * 16 + c;
      float val = sS[r * SL + part * 16 + c] * g.zscale;
      if (ja > ia || ja >= g.tk) val = -INFINITY;
      z[c] = val;
      tmax = fmaxf(tmax, val);
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const float nm = fmaxf(m, tmax);
    float ps = 0.f;
    if (nm > -INFINITY) {
#pragma unroll
      for (int c = 0; c < 16; ++c) ps += pow2<MMA>(z[c] - nm);
    }
    ps += __shfl_xor_sync(0xffffffffu, ps, 1);
    ps += __shfl_xor_sync(0xffffffffu, ps, 2);
    if (nm > -INFINITY) {
      s = s * pow2<MMA>(m - nm) + ps;
      m = nm;
    }
  }
  const int i = ib * TS + r;
  if (mass) {
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    m = fminf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fminf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    if (g.bid == kBidMinshift) {
      // sum(a - rmin) over the window (kernels_bid.py:338-340); the rmax buffer holds rmin
      s = fmaxf(s - (float)(min(ia, g.tk - 1) + 1) * m, 0.f);
    } else {
      m = 0.f;
    }
  }
  if (part == 0 && i < g.tq) {
    rmax[n * g.tq + i] = m;
    rden[n * g.tq + i] = s;
  }
}

// ---------------------------------------------------------------- pass 2
// Key-stationary: one CTA per (row n, 64-key block), query blocks in causal
// order; the running per-key demand is the exclusive scan, written as a
// checkpoint before each query block.  grid = n * ceil(tk/64).
template <typename T, int D, bool MMA>
__global__ void __launch_bounds__(NT) colsum_scan_kernel(
    const T* __restrict__ q, const T* __restrict__ k, Geom g, const float* __restrict__ rmax,
    const float* __restrict__ rden, const float* __restrict__ carry_base,
    float* __restrict__ carry, float* __restrict__ total) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = ld<D>();
  float* sK = smem;
  float* sQ = sK + TS * LD;
  float* sS = sQ + TS * LD;
  float* sM = sS + TS * SL;
  float* sRinv = sM + TS;
  float* sU = sRinv + TS;
  float* sPart = sU + TS;  // [4][64]
  const int nqb = (g.tq + TS - 1) / TS;
  const int ncb = (g.tq + kCarryRows - 1) / kCarryRows;
  const int64_t n = blockIdx.x % g.n;
  const int jb = (int)(blockIdx.x / g.n);
  load_tile<T, D, MMA>(sK, k + n * g.tk * D, jb * TS, g.tk);

  const int col = threadIdx.x & 63, seg = threadIdx.x >> 6;
  const int ja = jb * TS + col;
  const float base = (seg == 0 && carry_base != nullptr && ja < g.tk) ? carry_base[n * g.tk + ja] : 0.f;
  float local = 0.f;
  for (int ib = first_query_block(jb, g.q_off); ib < nqb; ++ib) {
    __syncthreads();
    load_tile<T, D, MMA>(sQ, q + n * g.tq * D, ib * TS, g.tq);
    load_stats(sM, sRinv, sU, rmax, rden, n, ib, g);
    __syncthreads();
    score_tile<D, MMA>(sQ, sK, sS);
    __syncthreads();
    float part = 0.f;
#pragma unroll 4
    for (int rr = 0; rr < 16; ++rr) {
      const int i = seg * 16 + rr;
      const int il = ib * TS + i, ia = g.q_off + il;
      part += (ja <= ia && ja < g.tk && il < g.tq) ? bid_value<MMA>(sS[i * SL + col], g, sM[i], sRinv[i], sU[i]) : 0.f;
    }
    sPart[seg * TS + col] = part;
    __syncthreads();
    if (seg == 0) {
      // two checkpoints per tile: in front of its first and of its 33rd query row
      const float half0 = sPart[col] + sPart[TS + col];
      if (ja < g.tk) {
        carry[(n * ncb + 2 * ib) * (int64_t)g.tk + ja] = base + local;
        if (2 * ib + 1 < ncb) carry[(n * ncb + 2 * ib + 1) * (int64_t)g.tk + ja] = base + local + half0;
      }
      local += half0 + (sPart[2 * TS + col] + sPart[3 * TS + col]);
    }
  }
  if (seg == 0 && ja < g.tk) total[n * g.tk + ja] = local;
}

// ---------------------------------------------------------------- pass 3
// Query-stationary main pass.  grid = n * ceil(tq/64), longest rows first.
template <typename T, int D, bool PK, bool MMA>
__global__ void __launch_bounds__(NT) main_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, Geom g,
    const float* __restrict__ rmax, const float* __restrict__ rden,
    const float* __restrict__ carry, const float* __restrict__ carry_base,
    float* __restrict__ out, float* __restrict__ ssum, float* __restrict__ pk) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = ld<D>();
  constexpr int DC = D / 16;
  float* sQ = smem;
  float* sK = sQ + TS * LD;
  float* sV = sK + TS * LD;
  float* sP = sV + TS * LD;   // scores, then bids, then shares, in place
  float* sM = sP + TS * SL;
  float* sRinv = sM + TS;
  float* sRow = sRinv + TS;
  float* sSeg = sRow + TS;   // [4][64] segment sums of the bids
  float* sU = sSeg + 4 * TS;
  const int nqb = (g.tq + TS - 1) / TS;
  const int64_t n = blockIdx.x % g.n;
  const int ib = nqb - 1 - (int)(blockIdx.x / g.n);
  load_tile<T, D, MMA>(sQ, q + n * g.tq * D, ib * TS, g.tq);
  load_stats(sM, sRinv, sU, rmax, rden, n, ib, g);

  float acc_o[4][DC], acc_pk[4][DC];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < DC; ++c) acc_o[r][c] = acc_pk[r][c] = 0.f;
  float my_ssum = 0.f;
  const int row = threadIdx.x >> 2, part = threadIdx.x & 3;

  const int last_key = min(g.tk - 1, g.q_off + ib * TS + TS - 1);
  const int njb = last_key / TS + 1;
  const int ncb = (g.tq + kCarryRows - 1) / kCarryRows;
  const float* carry_row = carry + (n * ncb + 2 * ib) * (int64_t)g.tk;
  for (int jb = 0; jb < njb; ++jb) {
    __syncthreads();
    load_tile<T, D, MMA>(sK, k + n * g.tk * D, jb * TS, g.tk);
    load_tile<T, D, MMA>(sV, v + n * g.tk * D, jb * TS, g.tk);
    __syncthreads();
    score_tile<D, MMA>(sQ, sK, sP);
    __syncthreads();
    {
      // thread = (key column, 16-query segment): bids in place and their segment sums, then the
      // demand in front of the segment (checkpoint + earlier segments) and the shares
      const int col = threadIdx.x & 63, seg = threadIdx.x >> 6;
      const int ja = jb * TS + col;
      float seg_sum = 0.f;
#pragma unroll 4
      for (int rr = 0; rr < 16; ++rr) {
        const int i = seg * 16 + rr, il = ib * TS + i, ia = g.q_off + il;
        const float p =
            (ja <= ia && ja < g.tk && il < g.tq) ? bid_value<MMA>(sP[i * SL + col], g, sM[i], sRinv[i], sU[i]) : 0.f;
        sP[i * SL + col] = p;
        seg_sum += p;
      }
      sSeg[seg * TS + col] = seg_sum;
      __syncthreads();
      if (PK) {                 // pk = p K while the tile still holds the bids
        accum_tile<D, false, MMA, true>(sP, sK, acc_pk);
        __syncthreads();
      }
      float c = 0.f;
      if (g.share != kShareNone) {                  // no share step: no demand is read
        c = (ja < g.tk) ? carry_row[ja] : 0.f;
        if (carry_base != nullptr && ja < g.tk) c += carry_base[n * g.tk + ja];
        for (int s2 = 0; s2 < seg; ++s2) c += sSeg[s2 * TS + col];
      }
      if (g.share == kShareInclusive) {
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const int i = seg * 16 + rr;
          const float p = sP[i * SL + col];
          sP[i * SL + col] = op_round<MMA>(ratio<MMA>(p, c + p + g.eps));
          c += p;
        }
      } else if (g.share == kShareExclusive) {      // earlier queries' demand only
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const int i = seg * 16 + rr;
          const float p = sP[i * SL + col];
          sP[i * SL + col] = op_round<MMA>(ratio<MMA>(p, c + g.eps));
          c += p;
        }
      } else if (MMA) {                             // no share step: the bids themselves
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr)
          sP[(seg * 16 + rr) * SL + col] = op_round<MMA>(sP[(seg * 16 + rr) * SL + col]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 16; ++c) my_ssum += sP[row * SL + part * 16 + c];
    accum_tile<D, false, MMA>(sP, sV, acc_o);
  }
  my_ssum += __shfl_xor_sync(0xffffffffu, my_ssum, 1);
  my_ssum += __shfl_xor_sync(0xffffffffu, my_ssum, 2);
  __syncthreads();
  if (part == 0) {
    sRow[row] = my_ssum;
    const int i = ib * TS + row;
    if (i < g.tq) ssum[n * g.tq + i] = my_ssum;
  }
  __syncthreads();
  using F = Frag<MMA, D>;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int il = F::row(r, 0), i = ib * TS + il;
    if (i >= g.tq) continue;
    const float den = sRow[il] + g.eps;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int64_t o = (n * g.tq + i) * D + F::col(r, c);
      out[o] = acc_o[r][c] / den;
      if (PK) pk[o] = acc_pk[r][c] * g.scale;
    }
  }
}

// ---------------------------------------------------------------- backward
// dbar_i = dout_i . out_i ; one warp per row.  Also zeroes the atomics targets.
template <int D>
__global__ void dbar_kernel(const float* __restrict__ dout, const float* __restrict__ out,
                            int64_t rows, float* __restrict__ dbar, float* __restrict__ ghat,
                            float* __restrict__ dq_main) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int c = lane; c < D; c += 32) {
    s += dout[row * D + c] * out[row * D + c];
    dq_main[row * D + c] = 0.f;
  }
  s = warp_sum(s);
  if (lane == 0) {
    dbar[row] = s;
    ghat[row] = 0.f;
  }
}

// Heavy reverse pass (the reference's BA, kernels.py:677-775): key-stationary,
// query blocks from last to first so the per-key suffix of dk_share is a
// running sum.  grid = n * ceil(t/64).
template <typename T, int D, bool MMA>
__global__ void __launch_bounds__(NT) backward_main_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, Geom g,
    const float* __restrict__ dout, const float* __restrict__ dbar,
    const float* __restrict__ ssum, const float* __restrict__ rmax,
    const float* __restrict__ rden, const float* __restrict__ carry,
    float* __restrict__ dq_main, float* __restrict__ dk_main, T* __restrict__ dv,
    float* __restrict__ ghat) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = ld<D>();
  constexpr int DC = D / 16;
  float* sK = smem;
  float* sV = sK + TS * LD;
  float* sQ = sV + TS * LD;
  float* sDO = sQ + TS * LD;
  float* sP = sDO + TS * LD;
  float* sDS = sP + TS * SL;
  float* sM = sDS + TS * SL;
  float* sRinv = sM + TS;
  float* sDbar = sRinv + TS;
  float* sSinv = sDbar + TS;
  float* sSeg = sSinv + TS;   // [8][64] segment sums: bids, then dk_share
  float* sU = sSeg + 8 * TS;
  float* sGh = sU + TS;       // f(a) / rowsum(f) bids: the tile's part of ghat_i (pass 1), or ghat_i (pass 2)
  const int nqb = (g.tq + TS - 1) / TS;
  const int ncb = (g.tq + kCarryRows - 1) / kCarryRows;
  const int64_t n = blockIdx.x % g.n;
  const int jb = (int)(blockIdx.x / g.n);
  load_tile<T, D, MMA>(sK, k + n * g.tk * D, jb * TS, g.tk);
  load_tile<T, D, MMA>(sV, v + n * g.tk * D, jb * TS, g.tk);

  float acc_dk[4][DC], acc_dv[4][DC];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < DC; ++c) acc_dk[r][c] = acc_dv[r][c] = 0.f;
  float sufk = 0.f;
  const int row = threadIdx.x >> 2, part = threadIdx.x & 3;
  using F = Frag<MMA, D>;

  for (int ib = nqb - 1; ib >= first_query_block(jb, g.q_off); --ib) {
    __syncthreads();
    load_tile<T, D, MMA>(sQ, q + n * g.tq * D, ib * TS, g.tq);
    load_tile<float, D, MMA>(sDO, dout + n * g.tq * D, ib * TS, g.tq);
    load_stats(sM, sRinv, sU, rmax, rden, n, ib, g);
    if (threadIdx.x < TS) {
      const int i = ib * TS + threadIdx.x;
      const bool ok = i < g.tq;
      sGh[threadIdx.x] = (g.ghat_pass == 2 && ok) ? ghat[n * g.tq + i] : 0.f;
      sDbar[threadIdx.x] = ok ? dbar[n * g.tq + i] : 0.f;
      sSinv[threadIdx.x] = ok ? 1.f / (ssum[n * g.tq + i] + g.eps) : 0.f;
    }
    __syncthreads();
    score_tile<D, MMA>(sQ, sK, sP);
    score_tile<D, MMA>(sDO, sV, sDS);
    __syncthreads();
    {
      // thread = (key column, 16-query segment), three phases separated by barriers:
      //  1. bids and ds in place, segment sums of the bids;
      //  2. the demand in front of every query (checkpoint + earlier segments + running sum) and
      //     the segment sums of dk_share;
      //  3. the same walk again with the suffix of dk_share over later queries (as
      //     kernels_bid.py:749: total minus prefix), the element-wise terms of kernels.py:757-765 /
      //     kernels_bid.py:735-754 by share step and bid, pdp and attn in place.
      const int col = threadIdx.x & 63, seg = threadIdx.x >> 6;
      const int ja = jb * TS + col;
      float seg_sum = 0.f;
#pragma unroll 4
      for (int rr = 0; rr < 16; ++rr) {
        const int i = seg * 16 + rr, il = ib * TS + i, ia = g.q_off + il;
        const bool ok = ja <= ia && ja < g.tk && il < g.tq;
        const float p = ok ? bid_value<MMA>(sP[i * SL + col], g, sM[i], sRinv[i], sU[i]) : 0.f;
        sP[i * SL + col] = p;
        seg_sum += p;
        sDS[i * SL + col] = ok ? (sDS[i * SL + col] - sDbar[i]) * sSinv[i] : 0.f;   // kernels.py:463-464
      }
      sSeg[seg * TS + col] = seg_sum;
      __syncthreads();
      float c0 = 0.f;
      if (g.share != kShareNone) {                  // no share step: no demand is read
        c0 = (ja < g.tk) ? carry[(n * ncb + 2 * ib) * (int64_t)g.tk + ja] : 0.f;
        for (int s2 = 0; s2 < seg; ++s2) c0 += sSeg[s2 * TS + col];
      }
      // first walk: the segment's sum of dk_share
      float c = c0, dk_sum = 0.f;
      if (g.share != kShareNone) {
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const int i = seg * 16 + rr;
          const float p = sP[i * SL + col], ds = sDS[i * SL + col];
          const float inv = recip<MMA>(g.share == kShareInclusive ? c + p + g.eps : c + g.eps);
          dk_sum -= ds * p * inv * inv;                    // :761
          c += p;
        }
      }
      sSeg[(4 + seg) * TS + col] = dk_sum;
      __syncthreads();
      // second walk, same order (the demand of every query is rebuilt bit for bit): the suffix of
      // dk_share over later queries = later tiles + later segments + this segment - prefix
      float r = sufk + dk_sum;
      for (int s2 = 3; s2 > seg; --s2) r += sSeg[(4 + s2) * TS + col];
      c = c0;
#pragma unroll 4
      for (int rr = 0; rr < 16; ++rr) {
        const int i = seg * 16 + rr;
        const float p = sP[i * SL + col], ds = sDS[i * SL + col];
        float inv = 1.f, direct = ds;
        if (g.share == kShareInclusive) {
          inv = recip<MMA>(c + p + g.eps);
          const float inv2 = inv * inv;
          r += ds * p * inv2;                              // minus this query's dk_share
          direct = ds * (c + g.eps) * inv2;                // :765
        } else if (g.share == kShareExclusive) {
          inv = recip<MMA>(c + g.eps);
          r += ds * p * inv * inv;
          direct = ds * inv;
        }
        const int il = ib * TS + i;
        const float jac = bid_jac_of_bid<MMA>(p, g, sRinv[i], ja <= g.q_off + il && ja < g.tk && il < g.tq);
        float dp = direct + r;
        if (g.ghat_pass == 1) {
          // ghat_i = sum_j p_ij dp_ij (not the row sum of the tile below: jac != p): the 32 columns
          // of a warp are summed here, two shared atomics per query row and tile
          const float part_g = warp_sum(p * dp);
          if ((threadIdx.x & 31) == 0) atomicAdd(&sGh[i], part_g);
        } else if (g.ghat_pass == 2) {
          dp -= sGh[i];
        }
        sDS[i * SL + col] = op_round<MMA>(jac * dp);                      // pdp
        sP[i * SL + col] = op_round<MMA>(p * inv * sSinv[i]);             // attn, :757
        c += p;
      }
      sufk += (sSeg[4 * TS + col] + sSeg[5 * TS + col]) + (sSeg[6 * TS + col] + sSeg[7 * TS + col]);
    }
    __syncthreads();
    if (g.normalised && g.ghat_pass != 2) {   // ghat: the row-normalised bid's Jacobian term
      float gs = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) gs += sDS[row * SL + part * 16 + c];
      gs += __shfl_xor_sync(0xffffffffu, gs, 1);
      gs += __shfl_xor_sync(0xffffffffu, gs, 2);
      if (g.ghat_pass == 1) gs = sGh[row];
      const int i = ib * TS + row;
      if (part == 0 && i < g.tq) atomicAdd(&ghat[n * g.tq + i], gs);
    }
    if (g.ghat_pass == 1) continue;           // this pass is for ghat alone
    accum_tile<D, true, MMA>(sP, sDO, acc_dv);
    accum_tile<D, true, MMA>(sDS, sQ, acc_dk);
    float dqp[4][DC];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < DC; ++c) dqp[r][c] = 0.f;
    accum_tile<D, false, MMA>(sDS, sK, dqp);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = ib * TS + F::row(r, 0);
      if (i >= g.tq) continue;
#pragma unroll
      for (int c = 0; c < DC; ++c)
        atomicAdd(&dq_main[(n * g.tq + i) * D + F::col(r, c)], dqp[r][c] * g.scale);
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int j = jb * TS + F::row(r, 0);
    if (j >= g.tk) continue;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int64_t o = (n * g.tk + j) * D + F::col(r, c);
      dk_main[o] = acc_dk[r][c] * g.scale;
      dv[o] = from_f32<T>(acc_dv[r][c]);
    }
  }
}

// Softmax-Jacobian correction for dk (the reference's BC, kernels.py:777-809):
// dk = dk_main - scale * p^T (ghat q).  grid = n * ceil(t/64).
template <typename T, int D, bool MMA>
__global__ void __launch_bounds__(NT) backward_dk_correction_kernel(
    const T* __restrict__ q, const T* __restrict__ k, Geom g, const float* __restrict__ rmax,
    const float* __restrict__ rden, const float* __restrict__ ghat,
    const float* __restrict__ dk_main, T* __restrict__ dk) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LD = ld<D>();
  constexpr int DC = D / 16;
  float* sK = smem;
  float* sQ = sK + TS * LD;
  float* sP = sQ + TS * LD;
  float* sM = sP + TS * SL;
  float* sRinv = sM + TS;
  float* sG = sRinv + TS;
  float* sU = sG + TS;
  const int nqb = (g.tq + TS - 1) / TS;
  const int64_t n = blockIdx.x % g.n;
  const int jb = (int)(blockIdx.x / g.n);
  load_tile<T, D, MMA>(sK, k + n * g.tk * D, jb * TS, g.tk);
  float acc[4][DC];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[r][c] = 0.f;
  for (int ib = first_query_block(jb, g.q_off); ib < nqb; ++ib) {
    __syncthreads();
    load_tile<T, D, MMA>(sQ, q + n * g.tq * D, ib * TS, g.tq);
    load_stats(sM, sRinv, sU, rmax, rden, n, ib, g);
    if (threadIdx.x < TS) {
      const int i = ib * TS + threadIdx.x;
      sG[threadIdx.x] = i < g.tq ? ghat[n * g.tq + i] : 0.f;
    }
    __syncthreads();
    score_tile<D, MMA>(sQ, sK, sP);
    __syncthreads();
    for (int idx = threadIdx.x; idx < TS * TS; idx += NT) {
      const int i = idx >> 6, j = idx & 63;
      const int ja = jb * TS + j, ia = g.q_off + ib * TS + i;
      // (softmax only: jac = p; the f(a) / rowsum(f) bids subtract ghat inside their second sweep)
      sP[i * SL + j] = (ja <= ia && ja < g.tk) ? op_round<MMA>(bid_value<MMA>(sP[i * SL + j], g, sM[i], sRinv[i], 0.f) * sG[i]) : 0.f;
    }
    __syncthreads();
    accum_tile<D, true, MMA>(sP, sQ, acc);
  }
  using F = Frag<MMA, D>;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int j = jb * TS + F::row(r, 0);
    if (j >= g.tk) continue;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int64_t o = (n * g.tk + j) * D + F::col(r, c);
      dk[o] = from_f32<T>(dk_main[o] - acc[r][c] * g.scale);
    }
  }
}

// dq = dq_main - ghat * pk  (kernels.py:814-826), stored in the input dtype.  Without pk
// (a bid with no row normalisation has no such term) a plain store in the input dtype.
template <typename T>
__global__ void dq_epilogue_kernel(const float* __restrict__ dq_main,
                                   const float* __restrict__ ghat, const float* __restrict__ pk,
                                   int64_t total, int d, T* __restrict__ dq) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  dq[idx] = from_f32<T>(pk != nullptr ? dq_main[idx] - ghat[idx / d] * pk[idx] : dq_main[idx]);
}

// Shared-memory sizes (bytes) of the kernels above.
template <int D> constexpr size_t smem_rowstats() { return sizeof(float) * (2 * TS * ld<D>() + TS * SL); }
template <int D> constexpr size_t smem_colsum() { return sizeof(float) * (2 * TS * ld<D>() + TS * SL + 3 * TS + 4 * TS); }
template <int D> constexpr size_t smem_main() { return sizeof(float) * (3 * TS * ld<D>() + TS * SL + 8 * TS); }
template <int D> constexpr size_t smem_bwd_main() { return sizeof(float) * (4 * TS * ld<D>() + 2 * TS * SL + 14 * TS); }
template <int D> constexpr size_t smem_bwd_dk() { return sizeof(float) * (2 * TS * ld<D>() + TS * SL + 4 * TS); }

}  // namespace simt
}  // namespace dil
