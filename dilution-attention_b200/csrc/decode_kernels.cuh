// Cached decode step (the reference's _dilution_decode, kernels.py:936-991),
// re-cut for HBM bandwidth: every (batch, head) row is split into key chunks so
// that the grid fills the machine at any batch size, and the step is three
// launches with no device-side waiting:
//   scores_kernel  : stream K once; z_j = q.k_j (log2 domain) -> scratch, and
//                    (max, sum) of each chunk;
//   sweep_kernel   : combine the chunk statistics, p_j, share_j = p/(c+p+eps) (or the
//                    selected bid / share variant), c_j += p_j in place, stream V once,
//                    partial share@V;
//   finalize_kernel: out = sum(partials) / (sum(share) + eps).
// Optionally the step also appends the new token (the model's _append_kv,
// model.py:85-93): given its k and v rows, the CTA that owns position len-1 takes
// them from there and writes them into the caches on the way.
// A warp reads cache rows 16 bytes per lane, so one load instruction covers
// 32/TPK whole rows (TPK = lanes per row) and every 128-byte line is consumed
// by the instruction that fetched it.
#pragma once

#include "common.cuh"

namespace dil {
namespace decode {

constexpr int NT = 256;
constexpr int WARPS = NT / 32;
constexpr int ROUND = 32 * WARPS;   // keys one CTA covers per round
constexpr int MAX_CHUNKS = 128;

template <typename T, int D> struct Cfg {
  static constexpr int E = 16 / (int)sizeof(T);   // elements per 16-byte slice
  static constexpr int TPK = D / E;                // lanes per cache row
  static_assert(TPK >= 1 && TPK <= 32, "row must fit a warp");
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

template <typename T> struct Unpack;
template <> struct Unpack<float> {
  static __device__ __forceinline__ void run(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
};
template <> struct Unpack<__nv_bfloat16> {
  static __device__ __forceinline__ void run(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xffff0000u);
    f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xffff0000u);
    f[4] = __uint_as_float(r.z << 16); f[5] = __uint_as_float(r.z & 0xffff0000u);
    f[6] = __uint_as_float(r.w << 16); f[7] = __uint_as_float(r.w & 0xffff0000u);
  }
};

// Layout of the caller-provided scratch for n rows and `stride` keys per row.
struct Scratch {
  float* aff;    // (n, stride)
  float2* part;  // (n, MAX_CHUNKS)  chunk (max, sum)
  float* pout;   // (n, MAX_CHUNKS, d)
  float* psum;   // (n, MAX_CHUNKS)
};

// grid = (chunks, n)
// MASS: an f(a) / rowsum(f) bid (kernels_bid.py:880-911) — the chunk statistics are (minimum of
// the scaled scores, sum of f) instead of the softmax's (maximum, sum of exponentials).
template <typename T, int D, bool MASS = false>
__global__ void __launch_bounds__(NT) scores_kernel(const T* __restrict__ q1,
                                                    const T* __restrict__ kc, int64_t cap,
                                                    int len_arg, int chunk, float zscale,
                                                    int64_t stride, float* __restrict__ aff,
                                                    float2* __restrict__ part,
                                                    const T* __restrict__ knew, T* __restrict__ kc_out,
                                                    const int* __restrict__ pos_dev, int bid = kBidSoftmax) {
  constexpr int E = Cfg<T, D>::E, TPK = Cfg<T, D>::TPK;
  // the number of valid keys: a launch argument, or (a step inside a captured graph, whose
  // arguments are frozen) the new token's position read from device memory, plus one
  // (held inside the cache: a position past the capacity rewrites the last row instead of
  // writing behind the cache; the caller owns the count)
  const int len = pos_dev != nullptr ? min(max(*pos_dev + 1, 1), (int)cap) : len_arg;
  const int64_t n = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = lane % TPK, grp = lane / TPK;
  float qf[E];
  {
    const uint4 raw = *reinterpret_cast<const uint4*>(q1 + n * D + t * E);
    Unpack<T>::run(raw, qf);
#pragma unroll
    for (int e = 0; e < E; ++e) qf[e] *= zscale;
  }
  const int k0 = blockIdx.x * chunk;
  // with an append, position len-1 (the last key of the last chunk) is not read from the cache:
  // the streaming loop stops in front of it and warp 0 takes its row from knew afterwards
  // (a grid sized for the capacity has chunks behind the last key: they write neutral statistics)
  const bool appends = knew != nullptr && len - 1 >= k0 && len - 1 < k0 + chunk;
  const int k1 = min(len, k0 + chunk) - (appends ? 1 : 0);
  const T* krow = kc + n * cap * D + t * E;
  float m = MASS ? INFINITY : -INFINITY, s = 0.f;
  for (int base = k0 + warp * 32; base < k1; base += ROUND) {
    float mine = -INFINITY;
    uint4 raw[TPK];
#pragma unroll
    for (int u = 0; u < TPK; ++u) {
      const int key = base + grp * TPK + u;
      raw[u] = key < k1 ? ld_stream(krow + (int64_t)key * D) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < TPK; ++u) {
      float kf[E];
      Unpack<T>::run(raw[u], kf);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) dot = fmaf(qf[e], kf[e], dot);
#pragma unroll
      for (int o = TPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (u == t) mine = dot;
    }
    const int key = base + lane;   // == base + grp*TPK + t
    if (key < k1) {
      aff[n * stride + key] = mine;
      if (MASS) {
        const float a = mine * kLn2;             // the scores are kept in the log2 domain
        s += bid_mass(a, bid);
        m = fminf(m, a);
      } else {
        const float nm = fmaxf(m, mine);
        s = s * exp2f(m - nm) + exp2f(mine - nm);
        m = nm;
      }
    }
  }
  if (appends && warp == 0) {
    // the new token's key: into the cache, and its score from registers
    float dot = 0.f;
    if (lane < TPK) {
      const uint4 raw = *reinterpret_cast<const uint4*>(knew + n * D + lane * E);
      *reinterpret_cast<uint4*>(kc_out + n * cap * D + (int64_t)(len - 1) * D + lane * E) = raw;
      float kf[E];
      Unpack<T>::run(raw, kf);
#pragma unroll
      for (int e = 0; e < E; ++e) dot = fmaf(qf[e], kf[e], dot);
    }
#pragma unroll
    for (int o = TPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) {
      aff[n * stride + len - 1] = dot;
      if (MASS) {
        s += bid_mass(dot * kLn2, bid);
        m = fminf(m, dot * kLn2);
      } else {
        const float nm = fmaxf(m, dot);
        s = s * exp2f(m - nm) + exp2f(dot - nm);
        m = nm;
      }
    }
  }
  // chunk statistics
  __shared__ float sm[WARPS], ss[WARPS];
  if (MASS) {
    const float wmin = -warp_max(-m), wsum = warp_sum(s);
    if (lane == 0) { sm[warp] = wmin; ss[warp] = wsum; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float cm = INFINITY, cs = 0.f;
      for (int w = 0; w < WARPS; ++w) { cm = fminf(cm, sm[w]); cs += ss[w]; }
      part[n * MAX_CHUNKS + blockIdx.x] = make_float2(cm, cs);
    }
    return;
  }
  const float wm = warp_max(m);
  const float ws = warp_sum(wm > -INFINITY ? s * exp2f(m - wm) : 0.f);
  if (lane == 0) { sm[warp] = wm; ss[warp] = ws; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float cm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) cm = fmaxf(cm, sm[w]);
    float cs = 0.f;
    for (int w = 0; w < WARPS; ++w) cs += sm[w] > -INFINITY ? ss[w] * exp2f(sm[w] - cm) : 0.f;
    part[n * MAX_CHUNKS + blockIdx.x] = make_float2(cm, cs);
  }
}

// The share of one key (kernels_bid.py:925-945) and its demand advanced in place.
//   MODE kSweepDilution: softmax bid, share = p / (c + p + eps)            (the operator)
//   MODE kSweepSoftmax : share = p, no demand read or written: plain softmax attention of the
//                        new token over the cache, the cached step of the reference's softmax
//                        layers (model.py:112-117)
//   MODE kSweepVariant : bid (any of the eight) and share step (inclusive / exclusive / none)
//                        chosen at run time; the demand advances by p in every case.  For an
//                        f(a) / rowsum(f) bid gmax is the row minimum (minshift) or 0, rinv the
//                        reciprocal of the row's mass (0 for a row without mass, which bids unif).
constexpr int kSweepSoftmax = 0, kSweepDilution = 1, kSweepVariant = 2;

template <int MODE>
__device__ __forceinline__ float key_share(float a, float gmax, float rinv, float eps, float* c_ptr,
                                           bool fresh, int bid, int share_step, float lshift, float unif = 0.f) {
  float p = exp2f(a - gmax) * rinv;
  if (MODE == kSweepSoftmax) return p;
  if (MODE == kSweepVariant && row_sum_bid(bid)) {
    const float an = a * kLn2;
    p = fmaf(bid == kBidMinshift ? fmaxf(an - gmax, 0.f) : bid_mass(an, bid), rinv, unif);
  } else if (MODE == kSweepVariant && bid != kBidSoftmax) {      // bids without a row sum
    p = bid_form(bid) == kBidSigmoid ? 1.f / (1.f + exp2f(lshift - a)) : exp2f(a - lshift);
  }
  const float c = fresh ? 0.f : *c_ptr;     // a fresh key: no demand yet, whatever the buffer holds
  *c_ptr = c + p;
  if (MODE == kSweepDilution || share_step == kShareInclusive) return p / (c + p + eps);
  return share_step == kShareExclusive ? p / (c + eps) : p;
}

// grid = (chunks, n)
template <typename T, int D, int MODE = kSweepDilution>
__global__ void __launch_bounds__(NT) sweep_kernel(const T* __restrict__ vc, int64_t cap, int len_arg,
                                                   int chunk, float eps, int64_t stride,
                                                   const float* __restrict__ aff,
                                                   const float2* __restrict__ part,
                                                   float* __restrict__ committed,
                                                   float* __restrict__ pout,
                                                   float* __restrict__ psum,
                                                   const T* __restrict__ vnew, T* __restrict__ vc_out,
                                                   int bid, int share_step, float lshift,
                                                   const int* __restrict__ pos_dev) {
  constexpr int E = Cfg<T, D>::E, TPK = Cfg<T, D>::TPK;
  const int len = pos_dev != nullptr ? min(max(*pos_dev + 1, 1), (int)cap) : len_arg;   // as in scores_kernel
  const int64_t n = blockIdx.y;
  const int nch = gridDim.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = lane % TPK, grp = lane / TPK;
  __shared__ float sred[WARPS];
  __shared__ float sacc[WARPS][D];
  __shared__ float sstat[3];

  // combine the per-chunk statistics of this row (nch <= MAX_CHUNKS <= NT)
  if (MODE == kSweepVariant && row_sum_bid(bid)) {
    // (minimum, mass) per chunk -> the row's minimum, 1 / mass and the uniform fall-back
    float2 pr = make_float2(INFINITY, 0.f);
    if (threadIdx.x < nch) pr = part[n * MAX_CHUNKS + threadIdx.x];
    const float wmin = -warp_max(-pr.x), wsum = warp_sum(pr.y);
    if (lane == 0) { sred[warp] = wmin; sacc[0][warp] = wsum; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float rmin = INFINITY, mass = 0.f;
      for (int w = 0; w < WARPS; ++w) { rmin = fminf(rmin, sred[w]); mass += sacc[0][w]; }
      if (bid == kBidMinshift) mass = fmaxf(mass - (float)len * rmin, 0.f);   // sum(a - rmin)
      else rmin = 0.f;
      sstat[0] = rmin;
      sstat[1] = mass > 0.f ? 1.f / mass : 0.f;
      sstat[2] = mass > 0.f ? 0.f : 1.f / (float)len;
    }
    __syncthreads();
  } else {
    float2 pr = make_float2(-INFINITY, 0.f);
    if (threadIdx.x < nch) pr = part[n * MAX_CHUNKS + threadIdx.x];
    const float wm = warp_max(pr.x);
    if (lane == 0) sred[warp] = wm;
    __syncthreads();
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) gm = fmaxf(gm, sred[w]);
    __syncthreads();
    const float ws = warp_sum(pr.x > -INFINITY ? pr.y * exp2f(pr.x - gm) : 0.f);
    if (lane == 0) sred[warp] = ws;
    __syncthreads();
    if (threadIdx.x == 0) {
      float den = 0.f;
      for (int w = 0; w < WARPS; ++w) den += sred[w];
      sstat[0] = gm;
      sstat[1] = 1.f / den;
      sstat[2] = 0.f;
    }
    __syncthreads();
  }
  const float gmax = sstat[0], rinv = sstat[1], unif = sstat[2];

  const int k0 = blockIdx.x * chunk;
  const bool appends = vnew != nullptr && len - 1 >= k0 && len - 1 < k0 + chunk;     // as in scores_kernel
  const int k1 = min(len, k0 + chunk) - (appends ? 1 : 0);
  const T* vrow = vc + n * cap * D + t * E;
  float acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  float ssh = 0.f;
  for (int base = k0 + warp * 32; base < k1; base += ROUND) {
    uint4 raw[TPK];
#pragma unroll
    for (int u = 0; u < TPK; ++u) {
      const int key = base + grp * TPK + u;
      raw[u] = key < k1 ? ld_stream(vrow + (int64_t)key * D) : make_uint4(0, 0, 0, 0);
    }
    const int key = base + lane;
    float share = 0.f;
    if (key < k1) {
      share = key_share<MODE>(aff[n * stride + key], gmax, rinv, eps, committed + n * cap + key, false, bid,
                              share_step, lshift, unif);
      ssh += share;
    }
#pragma unroll
    for (int u = 0; u < TPK; ++u) {
      const float sh = __shfl_sync(0xffffffffu, share, grp * TPK + u);
      float vf[E];
      Unpack<T>::run(raw[u], vf);
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = fmaf(sh, vf[e], acc[e]);
    }
  }
  if (appends && warp == 0) {
    // the new token: no demand on it yet (whatever the buffer holds), its value row from vnew
    float share = 0.f;
    if (lane == 0) {
      share = key_share<MODE>(aff[n * stride + len - 1], gmax, rinv, eps, committed + n * cap + len - 1, true,
                              bid, share_step, lshift, unif);
      ssh += share;
    }
    share = __shfl_sync(0xffffffffu, share, 0);
    if (lane < TPK) {
      const uint4 raw = *reinterpret_cast<const uint4*>(vnew + n * D + lane * E);
      *reinterpret_cast<uint4*>(vc_out + n * cap * D + (int64_t)(len - 1) * D + lane * E) = raw;
      float vf[E];
      Unpack<T>::run(raw, vf);
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = fmaf(share, vf[e], acc[e]);
    }
  }
  // lanes with the same slice t hold partial sums of the same output elements
#pragma unroll
  for (int o = TPK; o < 32; o <<= 1) {
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
  }
  ssh = warp_sum(ssh);
  if (lane < TPK) {
#pragma unroll
    for (int e = 0; e < E; ++e) sacc[warp][lane * E + e] = acc[e];
  }
  if (lane == 0) sred[warp] = ssh;
  __syncthreads();
  const int64_t slot = n * MAX_CHUNKS + blockIdx.x;
  if (threadIdx.x < D) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) o += sacc[w][threadIdx.x];
    pout[slot * D + threadIdx.x] = o;
  }
  if (threadIdx.x == 0) {
    float o = 0.f;
    for (int w = 0; w < WARPS; ++w) o += sred[w];
    psum[slot] = o;
  }
}

// grid = n, block = D
template <typename T, int D>
__global__ void finalize_kernel(const float* __restrict__ pout, const float* __restrict__ psum,
                                int nch, float eps, T* __restrict__ out) {
  const int64_t n = blockIdx.x;
  float o = 0.f, s = 0.f;
  for (int c = 0; c < nch; ++c) {
    o += pout[(n * MAX_CHUNKS + c) * D + threadIdx.x];
    s += psum[n * MAX_CHUNKS + c];
  }
  out[n * D + threadIdx.x] = from_f32<T>(o / (s + eps));
}

}  // namespace decode
}  // namespace dil
