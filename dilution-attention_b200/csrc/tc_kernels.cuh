// bf16 tensor-core path (dot_precision "bf16", bf16 inputs, head_dim 64):
// tcgen05.mma with accumulators in TMEM, operands staged by TMA, 128x128 tiles.
//
// Which axis sits on the TMEM lanes decides what is cheap per thread:
//   pass 1 (row statistics)   S  = Q K^T : lane = query, so row max / row sum
//                                          are private to a thread;
//   passes 2-4 (column work)  S^T = K Q^T: lane = key, so the cumulative demand
//                                          of a key is a running sum in ONE
//                                          register while the thread walks the
//                                          queries of the tile in order; the
//                                          per-query statistics it needs are
//                                          warp-uniform and come from shared
//                                          memory as broadcasts.
// A training forward runs passes 2 and 3 as one key-stationary sweep (tc_fused_forward.cuh);
// forward-only calls, sequence-parallel prefill and the bid / share variants run them separately.
// Warp w of a CTA reads TMEM lanes 32*(w%4)..32*(w%4)+31.  The forward passes and the
// correction pass run 256 threads (two warpgroups that split a tile's columns), thread 0
// issuing TMA and MMA, two to four CTAs per SM hiding each other's MMA/TMA latency; the
// main reverse pass runs 384 threads, one CTA per SM, with a dedicated issuing warpgroup.
#pragma once

#include <mutex>
#include <type_traits>

#include "tc_common.cuh"

namespace dil {
namespace tc {

__device__ int g_status = 0;   // first bounded wait that ran out (0 = none)

inline bool supported(int dtype, int precision, int d, int64_t q_offset) {
  return dtype == 1 && precision == 2 && d == kHeadDim && (q_offset % kTileRows) == 0;
}

// ---------------------------------------------------------------- host: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// cuTensorMapEncodeTiled is a driver entry point and wants a current context.  A thread that
// has only selected the device (an autograd engine thread calling the backward first) may
// not have one yet: a runtime call that touches the device binds the primary context.
inline void ensure_context() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

// Encoded maps are kept: a map depends only on (base, n, t, element type, box), and the same
// tensors come back on every step of a training loop or every pass of a forward.
struct MapKey {
  const void* base;
  int64_t n, t;
  int kind;      // 0: bf16 box {64, rows, 1}; 1: fp32 box {32, 128, 1}
  int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && n == o.n && t == o.t && kind == o.kind && box_rows == o.box_rows;
  }
};
struct MapCache {
  static constexpr int kSlots = 64;
  std::mutex mu;
  MapKey keys[kSlots];
  CUtensorMap maps[kSlots];
  int used = 0, next = 0;
  bool find(const MapKey& k, CUtensorMap* out) {
    std::lock_guard<std::mutex> lk(mu);
    for (int i = 0; i < used; ++i)
      if (keys[i] == k) { *out = maps[i]; return true; }
    return false;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    std::lock_guard<std::mutex> lk(mu);
    const int i = used < kSlots ? used++ : (next = (next + 1) % kSlots);
    keys[i] = k;
    maps[i] = m;
  }
};
inline MapCache& map_cache() {
  static MapCache c;
  return c;
}

// (n, t, 64) bf16 row-major -> 3-D map {64, t, n}, box {64, 128, 1}, 128-byte swizzle.
// Rows past t read as zero, and a box never crosses into the next (batch, head) row.
inline int make_map(CUtensorMap* map, const void* base, int64_t n, int64_t t, char* err, size_t errlen,
                    int box_rows = kTileRows) {
  const MapKey key{base, n, t, 0, box_rows};
  if (map_cache().find(key, map)) return 0;
  ensure_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    snprintf(err, errlen, "cuTensorMapEncodeTiled is not available from the driver");
    return 3;
  }
  if ((uintptr_t)base & 15) {
    snprintf(err, errlen, "bf16 tensor-core path needs 16-byte aligned q/k/v");
    return 1;
  }
  const cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)t, (cuuint64_t)n};
  const cuuint64_t strides[2] = {(cuuint64_t)kHeadDim * 2, (cuuint64_t)t * kHeadDim * 2};
  const cuuint32_t box[3] = {(cuuint32_t)kHeadDim, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(err, errlen, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return 3;
  }
  map_cache().put(key, *map);
  return 0;
}

// (n, t, 64) fp32 row-major -> 3-D map {64, t, n}, box {32, 128, 1} (128 bytes wide),
// 128-byte swizzle: the target of the dQ tile reductions.
inline int make_map_f32(CUtensorMap* map, const void* base, int64_t n, int64_t t, char* err, size_t errlen) {
  const MapKey key{base, n, t, 1, kTileRows};
  if (map_cache().find(key, map)) return 0;
  ensure_context();
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    snprintf(err, errlen, "cuTensorMapEncodeTiled is not available from the driver");
    return 3;
  }
  const cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)t, (cuuint64_t)n};
  const cuuint64_t strides[2] = {(cuuint64_t)kHeadDim * 4, (cuuint64_t)t * kHeadDim * 4};
  const cuuint32_t box[3] = {32, (cuuint32_t)kTileRows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(err, errlen, "cuTensorMapEncodeTiled (fp32) failed (%d)", (int)r);
    return 3;
  }
  map_cache().put(key, *map);
  return 0;
}

// ---------------------------------------------------------------- forward kernels
// Common shape of passes 1-3: 256 threads = two warpgroups.  Warp w reads TMEM
// lanes 32*(w%4).., so both warpgroups see all 128 lanes of a 128x128 score tile
// and split its COLUMNS: warpgroup 0 takes columns 0-63, warpgroup 1 columns 64-127.
// Thread 0 issues TMA and MMA.  One score buffer in TMEM per CTA; several CTAs per
// SM overlap each other's MMA/TMA latency.

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Byte offset of the 16-byte chunk holding queries [q, q+8) of `key` in an
// MN-major [128 keys][128 queries] bf16 tile (q a multiple of 8): two 64-query
// sub-tiles of 16 KB, rows of 128 B, 16-byte chunks XOR-swizzled by the row.
__device__ __forceinline__ uint32_t share_chunk_offset(int key, int q) {
  return (uint32_t)((q >> 6) * (int)kTileBytes + key * 128 + ((((q & 63) >> 3) ^ (key & 7)) << 4));
}

// log2-domain log-sum-exp of query i (+inf past the end, so that its p is 0).  The sigmoid bid
// and the shifted bids have no row statistics: their "lse" is log2 of the shift (0 for the plain
// sigmoid) for a query that exists and +inf past the end.
template <int BID = kBidSoftmax>
__device__ __forceinline__ float load_lse(const float* __restrict__ rmax, const float* __restrict__ rden,
                                          int64_t row_base, int i, int tq, float lshift = 0.f) {
  if (BID == kBidSigmoid || rmax == nullptr) return i < tq ? lshift : INFINITY;   // no row statistics
  return i < tq ? rmax[row_base + i] + log2f(rden[row_base + i]) : INFINITY;
}

// The bid of one raw score s (kernels_bid.py:191-204) given the row's lse l:
// softmax 2^(s*zscale - l); sigmoid 1 / (1 + 2^(l - s*zscale)), which is 0 for l = +inf.
template <int BID, bool POLY = false>
__device__ __forceinline__ float bid_p(float s, float zscale, float l) {
  if (BID == kBidSigmoid) return fast_rcp(1.f + fast_exp2(fmaf(s, -zscale, l)));
  // POLY: the exponential on the FMA pipe (a share of them, where the special-function unit binds)
  return POLY ? poly_exp2<4>(fmaf(s, zscale, -l)) : fast_exp2(fmaf(s, zscale, -l));
}

// ---------------------------------------------------------------- pass 1: row statistics
// grid = n * ceil(tq/128), longest rows first.  S = Q K^T, lane = query: each
// thread reduces its 64 key columns of the tile with an online max / sum; the two
// halves of a row are merged once at the end.  TMEM: 128 columns; 4 CTAs per SM.
constexpr int kRowstatsSmem = 3 * kTileBytes + 1024 + 1024 + 256;

__global__ void __launch_bounds__(256, 4) rowstats_kernel(const __grid_constant__ CUtensorMap map_q,
                                                          const __grid_constant__ CUtensorMap map_k,
                                                          Geom g, float* __restrict__ rmax,
                                                          float* __restrict__ rden) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sQ = smem_u32(smem), sK0 = sQ + kTileBytes;
  float2* sMerge = reinterpret_cast<float2*>(smem + 3 * kTileBytes);          // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes + 1024);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t kfull = smem_u32(bars), sdone = smem_u32(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int n = (int)(blockIdx.x % g.n);
  const int ib = nqb - 1 - (int)(blockIdx.x / g.n);
  const int q0 = g.q_off + ib * kTileRows;
  const int njb = min(g.tk - 1, q0 + kTileRows - 1) / kTileRows + 1;

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 3; ++i) mbar_init(kfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;

  if (tid == 0) {
    mbar_expect_tx(kfull, 2 * kTileBytes);
    tma_load_tile(sQ, &map_q, ib * kTileRows, n, kfull);
    tma_load_tile(sK0, &map_k, 0, n, kfull);
    if (njb > 1) {
      mbar_expect_tx(kfull + 8, kTileBytes);
      tma_load_tile(sK0 + kTileBytes, &map_k, kTileRows, n, kfull + 8);
    }
  }
  float m = -INFINITY, s = 0.f;
  const int ia = q0 + row;
  const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 64 * wg;
  for (int jb = 0; jb < njb; ++jb) {
    const int b = jb & 1;
    if (tid == 0) {
      mbar_wait(kfull + 8 * b, (jb >> 1) & 1, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      mma_scores(tmem, sQ, sK0 + kTileBytes * b, 128);
      mma_commit(sdone);
    }
    __syncwarp();
    mbar_wait(sdone, jb & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && jb + 2 < njb) {     // this K stage is free again
      mbar_expect_tx(kfull + 8 * b, kTileBytes);
      tma_load_tile(sK0 + kTileBytes * b, &map_k, (jb + 2) * kTileRows, n, kfull + 8 * b);
    }
    __syncwarp();
    const bool edge = (jb * kTileRows + kTileRows - 1 > q0) || ((jb + 1) * kTileRows > g.tk);
    // the mask arithmetic exists only in the instantiation used for edge tiles
    auto tile = [&](auto edge_tag) {
      constexpr bool EDGE = decltype(edge_tag)::value;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_ld32(taddr + 32 * c, v);
        tmem_ld_wait(v);
        float cmax = -INFINITY;          // max of the raw scores (zscale > 0 keeps the order)
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (EDGE) {
            const int ja = jb * kTileRows + wg * 64 + c * 32 + e;
            if (ja > ia || ja >= g.tk) v[e] = -INFINITY;
          }
          cmax = fmaxf(cmax, v[e]);
        }
        const float nm = fmaxf(m, cmax * g.zscale);
        if (nm > -INFINITY) {
          float ps = 0.f;
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            // the pass is bound by the special-function unit: every fourth exponential
            // is a polynomial on the FMA pipe instead
            const float z = fmaf(v[e], g.zscale, -nm);
            ps += (e & 3) == 3 ? poly_exp2<4>(z) : fast_exp2(z);
          }
          s = s * fast_exp2(m - nm) + ps;
          m = nm;
        }
      }
    };
    if (edge) tile(std::true_type{}); else tile(std::false_type{});
    tc_fence_before();
    __syncthreads();
  }
  if (wg == 1) sMerge[row] = make_float2(m, s);
  __syncthreads();
  const int i = ib * kTileRows + row;
  if (wg == 0 && i < g.tq) {
    const float2 o = sMerge[row];
    const float nm = fmaxf(m, o.x);          // finite: the first tile always holds key 0
    const float tot = s * fast_exp2(m - nm) + o.y * fast_exp2(o.x - nm);
    rmax[(int64_t)n * g.tq + i] = nm;
    rden[(int64_t)n * g.tq + i] = tot;
  }
  drain_if_aborted(ctl);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 128);
}

// ---------------------------------------------------------------- pass 2: column sums + scan
// grid = n * ceil(tk/128), key blocks with the most query blocks first.
// S^T = K Q^T, lane = key.  The CTA keeps its K tile and walks the query blocks
// in causal order.  Each warpgroup sums p over its 64 queries of the tile, 32 at a
// time; the thread of warpgroup 0 owns the key's running sum — the exclusive scan —
// and stores one checkpoint per CR query rows, one tile behind the sums.  CR = 32 when
// a backward will read the checkpoints (two threads per key there, 32 queries each),
// 64 for forward-only calls (the main forward pass starts its two warpgroups at queries
// 0 and 64 of a tile): half the scratch and half the checkpoint stores.
constexpr int kColsumSmem = 3 * kTileBytes + 1024 + 2048 + 1024 + 256;

template <int CR, int BID = kBidSoftmax>
__global__ void __launch_bounds__(256, 4) colsum_scan_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, Geom g,
    const float* __restrict__ rmax, const float* __restrict__ rden,
    const float* __restrict__ carry_base, float* __restrict__ carry, float* __restrict__ total) {
  static_assert(CR == 32 || CR == 64, "checkpoints every 32 or 64 query rows");
  constexpr int kPerTile = kTileRows / CR;                                      // 4 or 2
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem), sQ0 = sK + kTileBytes;
  float* sL = reinterpret_cast<float*>(smem + 3 * kTileBytes);                 // [2][128]
  float2* sCs = reinterpret_cast<float2*>(smem + 3 * kTileBytes + 1024);       // [2][128] the two sums of warpgroup 1
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes + 3072);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t qfull = smem_u32(bars), sdone = smem_u32(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int ncb = (g.tq + CR - 1) / CR;
  const int n = (int)(blockIdx.x % g.n);
  const int jb = (int)(blockIdx.x / g.n);
  const int k0 = jb * kTileRows;
  const int ib0 = k0 > g.q_off ? (k0 - g.q_off) / kTileRows : 0;     // first block that sees these keys
  const int nib = nqb - ib0;                                          // may be <= 0
  const int64_t row_base = (int64_t)n * g.tq;

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 3; ++i) mbar_init(qfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 128);
  if (nib > 0 && wg == 0) sL[row] = load_lse<BID>(rmax, rden, row_base, ib0 * kTileRows + row, g.tq, g.lshift);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;

  if (tid == 0 && nib > 0) {
    mbar_expect_tx(qfull, 2 * kTileBytes);
    tma_load_tile(sK, &map_k, k0, n, qfull);
    tma_load_tile(sQ0, &map_q, ib0 * kTileRows, n, qfull);
    if (nib > 1) {
      mbar_expect_tx(qfull + 8, kTileBytes);
      tma_load_tile(sQ0 + kTileBytes, &map_q, (ib0 + 1) * kTileRows, n, qfull + 8);
    }
  }
  const int ja = k0 + row;
  const bool live = ja < g.tk;
  const float base = (carry_base != nullptr && live) ? carry_base[(int64_t)n * g.tk + ja] : 0.f;
  float local = 0.f, prev0 = 0.f, prev1 = 0.f;   // warpgroup 0: scan state, its two sums of the previous tile
  // the checkpoints of 128-row tile `tile` (in front of its queries 0, 32, 64, 96 — or 0 and 64),
  // and the scan moved past it
  auto store_checkpoints = [&](int tile, float2 w1) {
    const int rb = tile * kPerTile;
    const float c0 = base + local, c1 = c0 + prev0, c2 = c1 + prev1, c3 = c2 + w1.x;
    if (live) {
      const int64_t o = ((int64_t)n * ncb + rb) * g.tk + ja;
      if (CR == 32) {
        if (rb < ncb) carry[o] = c0;
        if (rb + 1 < ncb) carry[o + g.tk] = c1;
        if (rb + 2 < ncb) carry[o + 2 * (int64_t)g.tk] = c2;
        if (rb + 3 < ncb) carry[o + 3 * (int64_t)g.tk] = c3;
      } else {
        if (rb < ncb) carry[o] = c0;
        if (rb + 1 < ncb) carry[o + g.tk] = c2;
      }
    }
    local += (prev0 + prev1) + (w1.x + w1.y);
  };
  const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + 64 * wg;
  for (int it = 0; it < nib; ++it) {
    const int ib = ib0 + it, b = it & 1;
    if (tid == 0) {
      mbar_wait(qfull + 8 * b, (it >> 1) & 1, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      mma_scores(tmem, sK, sQ0 + kTileBytes * b, 128);
      mma_commit(sdone);
    }
    __syncwarp();
    // while the MMA runs: next tile's statistics, and the checkpoints of the previous tile
    float lse_next = 0.f;
    if (wg == 1 && it + 1 < nib) lse_next = load_lse<BID>(rmax, rden, row_base, (ib + 1) * kTileRows + row, g.tq, g.lshift);
    if (wg == 0 && it > 0) store_checkpoints(ib - 1, sCs[((it - 1) & 1) * 128 + row]);
    mbar_wait(sdone, it & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && it + 2 < nib) {
      mbar_expect_tx(qfull + 8 * b, kTileBytes);
      tma_load_tile(sQ0 + kTileBytes * b, &map_q, (ib + 2) * kTileRows, n, qfull + 8 * b);
    }
    __syncwarp();
    const int i0 = g.q_off + ib * kTileRows + 64 * wg;   // absolute position of this half's first query
    const bool edge = i0 < k0 + kTileRows - 1;            // part of the diagonal tile
    const float4* L4 = reinterpret_cast<const float4*>(sL + 128 * b + 64 * wg);
    float colsum0 = 0.f, colsum1 = 0.f;      // queries 0-31 and 32-63 of this warpgroup's half
    auto tile = [&](auto edge_tag) {
      constexpr bool EDGE = decltype(edge_tag)::value;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_ld32(taddr + 32 * c, v);
        tmem_ld_wait(v);
        float part[4] = {0.f, 0.f, 0.f, 0.f};     // four independent sums
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l = L4[c * 8 + e4];
          const float ls[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float p = bid_p<BID>(v[e4 * 4 + u], g.zscale, ls[u]);
            if (EDGE && ja > i0 + c * 32 + e4 * 4 + u) p = 0.f;
            part[u] += p;
          }
        }
        const float cs = (part[0] + part[1]) + (part[2] + part[3]);
        if (c == 0) colsum0 = cs; else colsum1 = cs;
      }
    };
    if (edge) tile(std::true_type{}); else tile(std::false_type{});
    if (wg == 0) {
      prev0 = colsum0;
      prev1 = colsum1;
    } else {
      sCs[b * 128 + row] = make_float2(colsum0, colsum1);
    }
    if (wg == 1 && it + 1 < nib) sL[128 * (b ^ 1) + row] = lse_next;
    tc_fence_before();
    __syncthreads();
  }
  if (wg == 0 && live) {
    if (nib > 0) store_checkpoints(nqb - 1, sCs[((nib - 1) & 1) * 128 + row]);
    total[(int64_t)n * g.tk + ja] = local;
  }
  drain_if_aborted(ctl);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 128);
}

// ---------------------------------------------------------------- pass 3: main pass
// grid = n * ceil(tq/128), longest rows first.  S^T = K Q^T, lane = key.
// Each thread walks 64 queries of the tile in order (warpgroup 1 starts from the
// mid-block checkpoint) with its key's demand in one register:
//     den += p;  share = p / den          (den = committed + p + eps)
// and writes its half of the bf16 share tile to shared memory as an MN-major
// operand ([key][query]).  Two MMAs consume the tile:
//   O   [query x d ] += share * V      (A = share MN-major, B = V MN-major)
//   rs  [query x 16] += share * ones   (row sums of the SAME bf16 shares)
// so the final divide out = O / (rs + eps) normalises exactly what was summed.
// TMEM: S^T 128 columns, O 64, rs 16 (256 allocated; two CTAs per SM).
constexpr int kMainSmem = 7 * kTileBytes + 512 + 128;   // exact: the base must already be 1024-aligned

// BID / SHARE select the ablations of kernels_bid.py (sigmoid bid; exclusive or absent share step,
// :254-262); the default instantiation is the operator.
template <int BID = kBidSoftmax, int SHARE = kShareInclusive>
__global__ void __launch_bounds__(256, 2) forward_main_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, Geom g, const float* __restrict__ rmax,
    const float* __restrict__ rden, const float* __restrict__ carry,
    const float* __restrict__ carry_base, float* __restrict__ out, float* __restrict__ ssum) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {                      // no slack is requested: refuse instead of overrunning
    if (threadIdx.x == 0) atomicCAS(&g_status, 0, kErrAlign);
    return;
  }
  const uint32_t sQ = smem_u32(smem), sK0 = sQ + kTileBytes, sV = sQ + 3 * kTileBytes;
  // a [128 keys][64] bf16 tile of ones right behind V: the second 64-column group of the B
  // operand of share @ [V | ones] (N = 80), so the row sums come out of the same MMA
  const uint32_t sOnes = sQ + 4 * kTileBytes, sSh = sQ + 5 * kTileBytes;
  uint8_t* ones_ptr = smem + 4 * kTileBytes;
  float* sL = reinterpret_cast<float*>(smem + 7 * kTileBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * kTileBytes + 512);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t kfull = smem_u32(bars), vfull = smem_u32(bars + 2), sdone = smem_u32(bars + 3);

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int ncb = (g.tq + g.carry_rows - 1) / g.carry_rows;
  const int n = (int)(blockIdx.x % g.n);
  const int ib = nqb - 1 - (int)(blockIdx.x / g.n);
  const int q0 = g.q_off + ib * kTileRows;
  const int njb = min(g.tk - 1, q0 + kTileRows - 1) / kTileRows + 1;

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 4; ++i) mbar_init(kfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 256);
  if (wg == 0) sL[row] = load_lse<BID>(rmax, rden, (int64_t)n * g.tq, ib * kTileRows + row, g.tq, g.lshift);
  else {
#pragma unroll
    for (int c = 0; c < 8; ++c)
      reinterpret_cast<uint4*>(ones_ptr)[row * 8 + c] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;
  const uint32_t tS = tmem, tO = tmem + 128, tR = tmem + 192;   // O (64) and row sums (16): one N = 80 tile

  if (tid == 0) {
    mbar_expect_tx(kfull, 2 * kTileBytes);
    tma_load_tile(sQ, &map_q, ib * kTileRows, n, kfull);
    tma_load_tile(sK0, &map_k, 0, n, kfull);
    mbar_expect_tx(vfull, kTileBytes);
    tma_load_tile(sV, &map_v, 0, n, vfull);
    if (njb > 1) {
      mbar_expect_tx(kfull + 8, kTileBytes);
      tma_load_tile(sK0 + kTileBytes, &map_k, kTileRows, n, kfull + 8);
    }
    mbar_wait(kfull, 0, ctl, &g_status, kErrWaitTma);
    tc_fence_after();
    mma_scores(tS, sK0, sQ, 128);
    mma_commit(sdone);
  }
  __syncwarp();

  // the checkpoint row this warpgroup starts from: the one in front of query 0 / query 64 of the block
  const int rb = (ib * kTileRows + 64 * wg) / g.carry_rows;
  const bool have_rows = rb < ncb;                 // false only for a ragged last half block
  const int64_t carry_row = ((int64_t)n * ncb + (have_rows ? rb : 0)) * g.tk;
  const float4* L4 = reinterpret_cast<const float4*>(sL + 64 * wg);
  const uint32_t taddr = tS + ((uint32_t)((warp & 3) * 32) << 16) + 64 * wg;
  const int qh = q0 + 64 * wg;                     // absolute position of this half's first query
  auto load_den = [&](int jbx) {
    const int jx = jbx * kTileRows + row;
    float d = g.eps;
    if (SHARE != kShareNone && jx < g.tk && have_rows) {      // no share step: no demand is read
      d += carry[carry_row + jx];
      if (carry_base != nullptr) d += carry_base[(int64_t)n * g.tk + jx];
    }
    return d;
  };
  float den_next = load_den(0);
  for (int jb = 0; jb < njb; ++jb) {
    const int b = jb & 1;
    const int ja = jb * kTileRows + row;
    float den = den_next;
    mbar_wait(sdone, jb & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0) {
      if (jb >= 1) {                      // the V buffer is free: the previous share*V finished
        mbar_expect_tx(vfull, kTileBytes);
        tma_load_tile(sV, &map_v, jb * kTileRows, n, vfull);
      }
      if (jb >= 1 && jb + 1 < njb) {      // K stage of tile jb-1 is free
        mbar_expect_tx(kfull + 8 * (b ^ 1), kTileBytes);
        tma_load_tile(sK0 + kTileBytes * (b ^ 1), &map_k, (jb + 1) * kTileRows, n, kfull + 8 * (b ^ 1));
      }
    }
    __syncwarp();
    if (jb + 1 < njb) den_next = load_den(jb + 1);   // lands while this tile is processed
    const bool diag = jb * kTileRows + kTileRows - 1 > qh;
    const bool dead = ja >= g.tk;
    auto tile = [&](auto mask_tag) {
    constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float v[32];
      tmem_ld32(taddr + 32 * c, v);
      tmem_ld_wait(v);
      // the statistics of group e8+1 are read before group e8 is stored: shared-memory
      // loads cannot be hoisted above the stores by the compiler
      float4 lnext[2] = {L4[c * 8], L4[c * 8 + 1]};
#pragma unroll
      for (int e8 = 0; e8 < 4; ++e8) {
        uint32_t packed[4];
        const float4 lcur[2] = {lnext[0], lnext[1]};
        if (e8 < 3) {
          lnext[0] = L4[c * 8 + e8 * 2 + 2];
          lnext[1] = L4[c * 8 + e8 * 2 + 3];
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float ls[4] = {lcur[h].x, lcur[h].y, lcur[h].z, lcur[h].w};
          float sh[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e8 * 8 + h * 4 + u;
            // two special-function ops per score bind this pass: every fourth exponential of the
            // softmax bid is a polynomial on the FMA pipe (79.7 -> 75.3 ms at the 128K prefill shape)
            float p = u == 3 ? bid_p<BID, true>(v[e], g.zscale, ls[u]) : bid_p<BID>(v[e], g.zscale, ls[u]);
            if (MASK && (dead || ja > qh + c * 32 + e)) p = 0.f;
            if (SHARE == kShareInclusive) {
              den += p;
              sh[u] = p * fast_rcp(den);
            } else if (SHARE == kShareExclusive) {     // earlier queries' demand only
              sh[u] = p * fast_rcp(den);
              den += p;
            } else {                                   // no share step
              sh[u] = p;
            }
          }
          packed[h * 2 + 0] = pack_bf16(sh[0], sh[1]);
          packed[h * 2 + 1] = pack_bf16(sh[2], sh[3]);
        }
        const uint32_t dst = sSh + share_chunk_offset(row, wg * 64 + c * 32 + e8 * 8);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]),
                     "r"(packed[1]), "r"(packed[2]), "r"(packed[3])
                     : "memory");
      }
    }
    };
    if (diag || dead) tile(std::true_type{}); else tile(std::false_type{});
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      mbar_wait(vfull, jb & 1, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      constexpr uint32_t id_o = instr_desc(128, 80, 1, 1);
      // descriptors are built once per tile; a k-step is a constant 2048 B (128 units) further
      const Desc dSh = make_desc(sSh, kTileBytes, 1024), dVm = make_desc(sV, sOnes - sV, 1024);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) mma_ss(tO, dSh, 128 * kk, dVm, 128 * kk, id_o, (jb > 0 || kk > 0));
      if (jb + 1 < njb) {
        mbar_wait(kfull + 8 * (b ^ 1), ((jb + 1) >> 1) & 1, ctl, &g_status, kErrWaitTma);
        tc_fence_after();
        mma_scores(tS, sK0 + kTileBytes * (b ^ 1), sQ, 128);
      }
      mma_commit(sdone);
    }
    __syncwarp();
  }
  mbar_wait(sdone, njb & 1, ctl, &g_status, kErrWaitMma);
  tc_fence_after();
  {
    // lane = query now: each warpgroup stores 32 of the 64 output columns of row `row`
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    float o[32], r[32];
    tmem_ld32(tO + lane_base + 32 * wg, o);
    tmem_ld32(tR + lane_base, r);
    tmem_ld_wait(o);
    tmem_ld_wait(r);
    const int i = ib * kTileRows + row;
    if (i < g.tq) {
      const float inv = 1.f / (r[0] + g.eps);
      float4* dst = reinterpret_cast<float4*>(out + ((int64_t)n * g.tq + i) * kHeadDim + 32 * wg);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        dst[c] = make_float4(o[4 * c] * inv, o[4 * c + 1] * inv, o[4 * c + 2] * inv, o[4 * c + 3] * inv);
      if (wg == 0) ssum[(int64_t)n * g.tq + i] = r[0];
    }
  }
  drain_if_aborted(ctl);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// ---------------------------------------------------------------- pass 4: backward
// Pre-pass, one warp per query row: sinv = 1/(ssum+eps); dbar' = sinv * (dout . out);
// do' = bf16(sinv * dout); zeroes the dq / ghat accumulators.  Folding sinv into dO
// turns  ds = (do.v - dbar) * sinv  into  do'.v - dbar'  and  dv = attn^T do  into
// share^T do', so the main pass never multiplies by sinv per element.
template <typename TD>
__global__ void backward_prep_kernel(const TD* __restrict__ dout, const float* __restrict__ out,
                                     const float* __restrict__ ssum, float eps, int64_t rows,
                                     float* __restrict__ dbarp, __nv_bfloat16* __restrict__ dop,
                                     float* __restrict__ ghat, float* __restrict__ dq_main) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float2 a;
  if (std::is_same<TD, float>::value) {
    a = reinterpret_cast<const float2*>(dout + row * kHeadDim)[lane];
  } else {
    const uint32_t raw = reinterpret_cast<const uint32_t*>(dout + row * kHeadDim)[lane];
    a = make_float2(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u));
  }
  const float2 b = reinterpret_cast<const float2*>(out + row * kHeadDim)[lane];
  const float sinv = 1.f / (ssum[row] + eps);
  const float dot = warp_sum(a.x * b.x + a.y * b.y);
  reinterpret_cast<uint32_t*>(dop + row * kHeadDim)[lane] = pack_bf16(a.x * sinv, a.y * sinv);
  reinterpret_cast<float2*>(dq_main + row * kHeadDim)[lane] = make_float2(0.f, 0.f);
  if (lane == 0) {
    dbarp[row] = dot * sinv;
    ghat[row] = 0.f;
  }
}

// Main reverse pass (the reference's BA, kernels.py:677-775).  grid = n * ceil(t/128),
// key blocks with the most query blocks first; one CTA per SM, three warpgroups: two of
// compute warps and one whose first thread issues every TMA copy and every MMA and whose
// four warps move the finished dQ tiles out.
// TMEM (496 of 512 columns): two stages of S^T (64 columns each) | two stages of dOV^T
// (64 each) | dV 64 | dK 64 | dQ 64 + ghat 16 as one 80-column tile | the V tile as a
// bf16 A operand (32).
// The CTA keeps K (shared memory) and V (TMEM) of 128 keys and walks the queries from
// last to first in half-steps of 64: S^T = K Q^T and (dO' V^T)^T = V dO'^T are
// [128 keys x 64 queries], lane = key.  Two threads share a key and take 32 queries of a
// half-step each; the key's demand is stored every 32 query rows, so each starts from a
// stored checkpoint.  Each thread sweeps its 32 queries twice:
//   forwards for p and 1/(committed + p + eps), the demand accumulated from the checkpoint
//     exactly as the forward pass did (walking it backwards by subtraction cancels
//     catastrophically once attention is peaked);
//   backwards for the suffix sum of dk_share (kernels.py:763-764), in the reference's order:
//     its terms grow towards a key's first bidders, so a forward prefix would lose the small
//     ones.  Warpgroup 0 (queries 63..32) starts from the suffix behind the half-step;
//     warpgroup 1 (31..0) starts from zero, keeps p and pdp = p * dp in registers, and after
//     one barrier of the compute warps adds p * (the suffix warpgroup 0 ended with): dp is
//     linear in the suffix.
// Per half-step each thread writes 32 shares and 32 pdp values as bf16 pairs over TMEM
// columns it has already read: lane = key is the M index, so they are the A operands of
// dV += share^T dO' and dK += pdp^T Q without passing through shared memory.  pdp also goes
// to shared memory as the MN-major A operand (M = queries) of one N = 80 MMA per 128
// queries against B = [K | ones], which yields dQ = pdp K in 64 columns and ghat = pdp 1
// in the next 16.
// The issuing thread runs two half-steps ahead of the arithmetic: when the tiles of
// half-step h are complete it issues dV, dK (and dQ | ghat after the second half) of h and
// the score MMAs of h + 2 into the stage h has just left, so the tensor pipe works under
// the arithmetic of h + 1.  Q and dO' tiles are triple-buffered.  After setup the third
// warpgroup gives registers up (setmaxnreg) and the compute warpgroups take them.
constexpr int kBwdThreads = 384;
constexpr int kBwdSmem = 12 * kTileBytes + 2048 + 2048 + 256 + 1024;

template <int BID = kBidSoftmax, int SHARE = kShareInclusive>
__global__ void __launch_bounds__(kBwdThreads, 1) backward_main_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_dq, Geom g,
    const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ rmax, const float* __restrict__ rden, const float* __restrict__ dbarp,
    const float* __restrict__ carry, const float* __restrict__ total, float* __restrict__ dq_main,
    float* __restrict__ dk_main, __nv_bfloat16* __restrict__ dv, float* __restrict__ ghat) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem);
  // a [128 keys][64] bf16 tile of ones: the second 64-column group of the dQ MMA's B operand
  // (N = 80 = 64 columns of K + 16 of ones), so ghat comes out of the same instruction
  const uint32_t sOnes = sK + kTileBytes;
  uint8_t* ones_ptr = smem + kTileBytes;
  const uint32_t sQ0 = sK + 2 * kTileBytes, sD0 = sK + 5 * kTileBytes;        // [3] each
  const uint32_t sPd = sK + 8 * kTileBytes;                                    // 32 KB
  const uint32_t sDq = sK + 10 * kTileBytes;                                   // 32 KB: fp32 dQ staging
  float* sLse = reinterpret_cast<float*>(smem + 12 * kTileBytes);              // [2][128] log-sum-exp of a step's queries
  float* sDbar = sLse + 256;                                                   // [2][128] their dbar'
  float* sG = reinterpret_cast<float*>(smem + 12 * kTileBytes + 2048);         // [2][2][128] sums of dk_share
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 12 * kTileBytes + 4096);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 12);
  const uint32_t kfull = smem_u32(bars), qfull = smem_u32(bars + 1);           // qfull[3]
  const uint32_t sdone = smem_u32(bars + 4), tiles = smem_u32(bars + 6);       // [2] each
  const uint32_t dqdone = smem_u32(bars + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int ncb = (g.tq + kCarryRows - 1) / kCarryRows;
  const int n = (int)(blockIdx.x % g.n);
  const int jb = (int)(blockIdx.x / g.n);
  const int k0 = jb * kTileRows;
  const int nsteps = nqb - jb;                     // query blocks jb .. nqb-1, visited in reverse
  const int nhalf = 2 * nsteps;
  const int64_t row_base = (int64_t)n * g.tq;
  const int ja = k0 + row;
  const bool dead = ja >= g.tk;

  auto load_stats = [&](int ib) {
    const int i = ib * kTileRows + row;
    float2 st = make_float2(INFINITY, 0.f);
    if (i < g.tq) st = make_float2(load_lse<BID>(rmax, rden, row_base, i, g.tq, g.lshift), dbarp[row_base + i]);
    return st;
  };

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 6; ++i) mbar_init(kfull + 8 * i, 1);      // kfull, qfull[3], sdone[2]
    mbar_init(tiles, 8);
    mbar_init(tiles + 8, 8);
    mbar_init(dqdone, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 512);
  if (wg == 0) {
    const float2 st = load_stats(nqb - 1);
    sLse[row] = st.x;
    sDbar[row] = st.y;
  }
  else if (wg == 1) {
#pragma unroll
    for (int c = 0; c < 8; ++c)
      reinterpret_cast<uint4*>(ones_ptr)[row * 8 + c] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;
  const uint32_t tS0 = tmem, tDOV0 = tmem + 128, tDV = tmem + 256, tDK = tmem + 320, tDQ = tmem + 384,
                 tG = tmem + 448, tV = tmem + 464;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

  if (wg == 0) {
    // this key's V row as an A operand: two head-dim elements per 32-bit column
    uint32_t w[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (!dead) x = reinterpret_cast<const uint4*>(v + ((int64_t)n * g.tk + ja) * kHeadDim)[c];
      w[4 * c] = x.x; w[4 * c + 1] = x.y; w[4 * c + 2] = x.z; w[4 * c + 3] = x.w;
    }
    tmem_st16(tV + lane_base, w);
    tmem_st16(tV + lane_base + 16, w + 16);
  }
  if (wg < 2) {
    // dV and dK start from zero, so that every MMA into them accumulates
    uint32_t z[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) z[c] = 0u;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      tmem_st16(tDV + lane_base + 32 * wg + 16 * c, z);
      tmem_st16(tDK + lane_base + 32 * wg + 16 * c, z);
    }
    tmem_st_wait();
  }
  if (tid == 256) {
    mbar_expect_tx(kfull, kTileBytes);
    tma_load_tile(sK, &map_k, k0, n, kfull);
    for (int s = 0; s < 3 && s < nsteps; ++s) {
      mbar_expect_tx(qfull + 8 * s, 2 * kTileBytes);
      tma_load_tile(sQ0 + kTileBytes * s, &map_q, (nqb - 1 - s) * kTileRows, n, qfull + 8 * s);
      tma_load_tile(sD0 + kTileBytes * s, &map_do, (nqb - 1 - s) * kTileRows, n, qfull + 8 * s);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (wg == 2) {
    // ------------------------------------------------------------ warpgroup 2: issue and dQ read-out
    // Thread 256 issues every MMA and TMA copy.  After the second half-step of a step all
    // four warps (lane = query) move the finished dQ | ghat tile out, so that the compute
    // warps never touch it.  The warpgroup hands most of its registers to the other two.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 128;");
    constexpr uint32_t id_s = instr_desc(128, 64, 0, 0);     // scores: both operands K-major
    constexpr uint32_t id_kd = instr_desc(128, 64, 0, 1);    // dV, dK: A from TMEM (M = keys), B MN-major
    constexpr uint32_t id_qd = instr_desc(128, 80, 1, 1);    // dQ | ghat: A MN-major (M = queries)
    // every descriptor is built once; inside the loop tile, stage and k-step are constant
    // offsets (in 16-byte units: a tile is 1024, an MN-major k-step 128, a K-major one 2)
    const Desc dKk = make_desc(sK, 16, 1024);                 // K, K-major: A of the scores
    const Desc dKm = make_desc(sK, sOnes - sK, 1024);         // [K | ones], MN-major: B of dQ | ghat
    const Desc dPm = make_desc(sPd, kTileBytes, 1024);        // pdp, MN-major: A of dQ | ghat
    const Desc dQk = make_desc(sQ0, 16, 1024), dQm = make_desc(sQ0, kTileBytes, 1024);
    const Desc dDk = make_desc(sD0, 16, 1024), dDm = make_desc(sD0, kTileBytes, 1024);
    // scores of a half-step in stage ST of Q and dO'; even half-steps take queries 64..127
    auto issue_scores = [&](auto odd_c, auto st_c) {
      constexpr int ODD = decltype(odd_c)::value, ST = decltype(st_c)::value;
      constexpr uint32_t off = ST * 1024 + (ODD ? 0 : 512);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) mma_ss(tS0 + 64 * ODD, dKk, 2 * kk, dQk, off + 2 * kk, id_s, kk > 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) mma_ts(tDOV0 + 64 * ODD, tV + 8 * kk, dDk, off + 2 * kk, id_s, kk > 0);
    };
    if (tid == 256) {
      mbar_wait(kfull, 0, ctl, &g_status, kErrWaitTma);
      mbar_wait(qfull, 0, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      issue_scores(std::integral_constant<int, 0>{}, std::integral_constant<int, 0>{});
      mma_commit(sdone);
      issue_scores(std::integral_constant<int, 1>{}, std::integral_constant<int, 0>{});
      mma_commit(sdone + 8);
    }
    __syncwarp();
    // half-step h = 2s + ODD of step s, whose Q and dO' tiles sit in stage ST = s % 3
    auto half = [&](auto odd_c, auto st_c, int s) {
      constexpr int ODD = decltype(odd_c)::value, ST = decltype(st_c)::value;
      constexpr int ST1 = (ST + 1) % 3, ST2 = (ST + 2) % 3;
      if (tid == 256) {
        mbar_wait(tiles + 8 * ODD, s & 1, ctl, &g_status, kErrWaitTile);
        tc_fence_after();
#pragma unroll
        for (int kq = 0; kq < 4; ++kq) {                    // contraction over the 64 queries
          // queries [16kq, 16kq+16) of the half-step: 8 columns at the start of the owning
          // warpgroup's 32-column range (warpgroup 1 owns queries 0..31)
          constexpr uint32_t base = ST * 1024 + (ODD ? 0 : 4) * 128;
          const uint32_t col = 64 * ODD + 32 * (kq >> 1) + 8 * (kq & 1);
          mma_ts(tDV, tS0 + col, dDm, base + 128 * kq, id_kd, 1);
          mma_ts(tDK, tDOV0 + col, dQm, base + 128 * kq, id_kd, 1);
        }
        if (ODD) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)                    // contraction over the 128 keys
            mma_ss(tDQ, dPm, 128 * kk, dKm, 128 * kk, id_qd, kk > 0);
          mma_commit(dqdone);
        }
        if (s + 1 < nsteps) {                               // half-step h + 2 belongs to step s + 1
          if (!ODD) {
            mbar_wait(qfull + 8 * ST1, ((s + 1) / 3) & 1, ctl, &g_status, kErrWaitTma);
            tc_fence_after();
          }
          issue_scores(odd_c, std::integral_constant<int, ST1>{});
        }
        mma_commit(sdone + 8 * ODD);
        if (!ODD && s >= 1 && s + 2 < nsteps) {
          // every MMA of step s-1 has completed once the commit of its second half-step has:
          // its Q and dO' stage takes step s+2
          mbar_wait(sdone + 8, s & 1, ctl, &g_status, kErrWaitMma);
          mbar_expect_tx(qfull + 8 * ST2, 2 * kTileBytes);
          tma_load_tile(sQ0 + kTileBytes * ST2, &map_q, (nqb - 3 - s) * kTileRows, n, qfull + 8 * ST2);
          tma_load_tile(sD0 + kTileBytes * ST2, &map_do, (nqb - 3 - s) * kTileRows, n, qfull + 8 * ST2);
        }
      }
      __syncwarp();
      if (ODD) {
        // dQ and ghat of the step's 128 queries: lane = query.  The fp32 tile is staged in
        // shared memory in the copy engine's swizzled layout and added to dq_main by two
        // tensor reductions of 32 columns.
        if (lane == 0) mbar_wait(dqdone, s & 1, ctl, &g_status, kErrWaitMma);
        __syncwarp();
        tc_fence_after();
        if (tid == 256) tma_wait_read_all();            // the previous reductions have read the staging buffer
        asm volatile("bar.sync 2, 128;" ::: "memory");
        const uint32_t stage = sDq + row * 128;
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {                   // 16 columns at a time
          float dq[16];
          tmem_ld16(tDQ + lane_base + 16 * j, dq);
          tmem_ld_wait16(dq);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage + kTileBytes * (j >> 1) + (((4 * (j & 1) + c) ^ (row & 7)) << 4)),
                         "f"(dq[4 * c] * g.scale), "f"(dq[4 * c + 1] * g.scale), "f"(dq[4 * c + 2] * g.scale),
                         "f"(dq[4 * c + 3] * g.scale)
                         : "memory");
        }
        float gh;
        tmem_ld1(tG + lane_base, &gh);
        tmem_ld_wait();
        fence_async_smem();
        tc_fence_before();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        const int ibq = nqb - 1 - s;
        if (tid == 256) {
          tc_fence_after();
          tma_reduce_add_tile(&map_dq, sDq, 0, ibq * kTileRows, n);
          tma_reduce_add_tile(&map_dq, sDq + kTileBytes, 32, ibq * kTileRows, n);
        }
        const int i = ibq * kTileRows + row;
        if (i < g.tq) atomicAdd(ghat + row_base + i, gh);
      }
    };
    using C0 = std::integral_constant<int, 0>;
    using C1 = std::integral_constant<int, 1>;
    using C2 = std::integral_constant<int, 2>;
    for (int s = 0; s < nsteps; s += 3) {
      half(C0{}, C0{}, s);
      half(C1{}, C0{}, s);
      if (s + 1 < nsteps) {
        half(C0{}, C1{}, s + 1);
        half(C1{}, C1{}, s + 1);
      }
      if (s + 2 < nsteps) {
        half(C0{}, C2{}, s + 2);
        half(C1{}, C2{}, s + 2);
      }
    }
    if (tid == 256) tma_wait_read_all();
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
    // ------------------------------------------------------------ the compute warps
    const int cw = 32 * (1 - wg);                    // this warpgroup's columns of a stage
    // demand of this thread's key in front of its 32 queries of half-step h (exclusive of the
    // first): the stored checkpoint of that 32-row block (past the end: any value, p is 0 there)
    auto load_edge = [&](int h) {
      if (dead || SHARE == kShareNone) return 0.f;         // no share step: no demand is read
      const int rb = 4 * (nqb - 1 - (h >> 1)) + ((h & 1) ? 0 : 2) + (wg == 0 ? 1 : 0);
      return rb < ncb ? carry[((int64_t)n * ncb + rb) * g.tk + ja] : total[(int64_t)n * g.tk + ja];
    };
    float sigma = 0.f;                               // suffix of dk_share behind the half-step
    // the checkpoints are read once from a buffer far larger than L2: each load is issued two
    // half-steps before its value is used
    float incl = load_edge(0);
    float incl_next = nhalf > 1 ? load_edge(1) : 0.f;
    for (int h = 0; h < nhalf; ++h) {
      const int s = h >> 1, odd = h & 1, ib = nqb - 1 - s, b = s & 1;
      // fetch what the coming half-steps need before waiting for this one
      float incl_next2 = 0.f;
      float st_max = INFINITY, st_den = 1.f, st_dbar = 0.f;
      if (h + 2 < nhalf) incl_next2 = load_edge(h + 2);
      const bool fetch_stats = !odd && wg == 0 && s + 1 < nsteps;
      if (fetch_stats) {
        const int i = (ib - 1) * kTileRows + row;     // ib >= 1 here, so i < tq
        if (BID == kBidSoftmax && rmax != nullptr) {
          st_max = rmax[row_base + i];
          st_den = rden[row_base + i];
        } else {
          st_max = g.lshift;                          // no row statistics: lse = log2(shift) + log2(1)
        }
        st_dbar = dbarp[row_base + i];
      }
      mbar_wait(sdone + 8 * odd, s & 1, ctl, &g_status, kErrWaitMma);
      tc_fence_after();
      float vs[32], vd[32];
      const uint32_t tcol = lane_base + 64 * odd + cw;
      tmem_ld32(tS0 + tcol, vs);
      tmem_ld32(tDOV0 + tcol, vd);
      tmem_ld_wait(vs);
      tmem_ld_wait(vd);
      const int qc = (odd ? 0 : 64) + cw;             // first query column of this thread in the step's tile
      const int iq0 = ib * kTileRows + qc;            // its position (q_off == 0 here)
      const bool masked_tile = dead || (ib * kTileRows + (odd ? 0 : 64) < k0 + kTileRows - 1);
      const float4* Lse4 = reinterpret_cast<const float4*>(sLse + b * 128 + qc);
      const float4* Dbar4 = reinterpret_cast<const float4*>(sDbar + b * 128 + qc);
      uint32_t shp[16];                                // 32 shares as bf16 pairs
      // warpgroup 0 (queries 32..63) knows the suffix of dk_share behind its queries; warpgroup 1
      // starts from zero and adds p * (the suffix warpgroup 0 ends with) afterwards: dp is linear in it
      float R = wg == 0 ? sigma : 0.f;
      float incle = incl + g.eps;                      // demand + eps at the walk's position

      // Two sweeps over the thread's 32 queries.  Forwards: p and 1/(committed+p+eps), the demand
      // accumulated from the checkpoint in front exactly as the forward pass did.  Backwards: the
      // suffix of dk_share (kernels.py:763-764), accumulated from the last query to the first as
      // the reference does — its terms grow towards a key's first bidders, so the other order
      // loses the small ones.  Afterwards vs holds p and vd holds p * dp.
      auto chunk = [&](auto mask_tag) {
        constexpr bool MASK = decltype(mask_tag)::value;
        float inv[32];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l4 = Lse4[e4];
          const float lse[4] = {l4.x, l4.y, l4.z, l4.w};
          // softmax: z = s*zscale - lse, p = 2^z;  sigmoid: z = lse - s*zscale, p = 1/(1 + 2^z)
          const float zsign = BID == kBidSigmoid ? -g.zscale : g.zscale;
          const float lsign = BID == kBidSigmoid ? 1.f : -1.f;
          const float2 zs = make_float2(zsign, zsign);
          const float2 z01 = fma2(make_float2(vs[e4 * 4], vs[e4 * 4 + 1]), zs, make_float2(lsign * lse[0], lsign * lse[1]));
          const float2 z23 = fma2(make_float2(vs[e4 * 4 + 2], vs[e4 * 4 + 3]), zs, make_float2(lsign * lse[2], lsign * lse[3]));
          const float z[4] = {z01.x, z01.y, z23.x, z23.y};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e4 * 4 + u;
            float p = fast_exp2(z[u]);
            if (BID == kBidSigmoid) p = fast_rcp(1.f + p);
            if (MASK) {
              if (dead || ja > iq0 + e) p = 0.f;
            }
            if (SHARE == kShareInclusive) {
              incle += p;
              inv[e] = fast_rcp(incle);
            } else if (SHARE == kShareExclusive) {     // the demand of earlier queries only
              inv[e] = fast_rcp(incle);
              incle += p;
            } else {
              inv[e] = 1.f;
            }
            vs[e] = p;
          }
        }
#pragma unroll
        for (int e4 = 7; e4 >= 0; --e4) {
          const float4 d4 = Dbar4[e4];
          const float dbr[4] = {d4.x, d4.y, d4.z, d4.w};
          // with inv = 1/(committed+p+eps), share = p*inv and w = ds*inv:
          //   ds*(committed+eps)*inv^2 = w*(1-share),  dk_share = -w*share,
          //   dp = w - w*share + (suffix before this query) = w + (suffix after it)
          // (element-wise parts two queries per instruction; the suffix itself is serial).
          // Exclusive share step (inv = 1/(committed+eps)): the direct term is w itself, so
          // dp = w + (suffix BEFORE this query); no share step: dp = ds, no suffix at all.
          // The Jacobian factor is p for the softmax bid and p(1-p) for the sigmoid
          // (kernels_bid.py:196-204, 735-754); vs keeps it for the later suffix fix-up.
#pragma unroll
          for (int h = 1; h >= 0; --h) {
            const int e = e4 * 4 + 2 * h;
            const float2 p2 = make_float2(vs[e], vs[e + 1]), i2 = make_float2(inv[e], inv[e + 1]);
            const float2 w2 = mul2(sub2(make_float2(vd[e], vd[e + 1]), make_float2(dbr[2 * h], dbr[2 * h + 1])), i2);
            const float2 s2 = mul2(p2, i2);
            float2 jac2 = p2;
            if (BID == kBidSigmoid) jac2 = mul2(p2, sub2(make_float2(1.f, 1.f), p2));
            float2 pd2;
            if (SHARE == kShareInclusive) {
              const float r1 = fmaf(-w2.y, s2.y, R);
              R = fmaf(-w2.x, s2.x, r1);
              pd2 = mul2(jac2, add2(w2, make_float2(R, r1)));
            } else if (SHARE == kShareExclusive) {
              const float r1 = fmaf(-w2.y, s2.y, R);
              pd2 = mul2(jac2, add2(w2, make_float2(r1, R)));
              R = fmaf(-w2.x, s2.x, r1);
            } else {
              pd2 = mul2(jac2, w2);
            }
            vd[e] = pd2.x;
            vd[e + 1] = pd2.y;
            if (BID == kBidSigmoid) {
              vs[e] = jac2.x;
              vs[e + 1] = jac2.y;
            }
            shp[e4 * 2 + h] = pack_bf16(s2.x, s2.y);
          }
        }
      };
      if (masked_tile) chunk(std::true_type{}); else chunk(std::false_type{});
      // warpgroup 0: the suffix behind query 32; warpgroup 1: minus its own sum of -dk_share
      sG[(odd * 2 + wg) * 128 + row] = R;
      // the shares stay in TMEM, over score columns this thread has consumed
      tmem_st16(tS0 + tcol, shp);
      asm volatile("bar.sync 1, 256;" ::: "memory");   // the compute warps
      const float rother = sG[(odd * 2 + (1 - wg)) * 128 + row];
      const float fix = wg == 1 ? rother : 0.f;
      sigma = R + rother;                              // the suffix behind the next half-step
      // the dQ MMAs of the previous 128 queries read the pdp buffer that is written next
      if (!odd && s >= 1) {
        mbar_wait(dqdone, (s - 1) & 1, ctl, &g_status, kErrWaitMma);
      }
      {
        uint32_t pdt[16];                              // 32 pdp values as bf16 pairs
#pragma unroll
        for (int e8 = 0; e8 < 4; ++e8) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e8 * 8 + 2 * u;
            const float2 f2 = fma2(make_float2(vs[e], vs[e + 1]), make_float2(fix, fix), make_float2(vd[e], vd[e + 1]));
            pdt[e8 * 4 + u] = pack_bf16(f2.x, f2.y);
          }
          // shared memory: the MN-major A operand of dQ | ghat (M = queries)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sPd + share_chunk_offset(row, qc + e8 * 8)),
                       "r"(pdt[e8 * 4]), "r"(pdt[e8 * 4 + 1]), "r"(pdt[e8 * 4 + 2]), "r"(pdt[e8 * 4 + 3])
                       : "memory");
        }
        // TMEM, over consumed dOV^T columns: the A operand of dK (M = keys)
        tmem_st16(tDOV0 + tcol, pdt);
      }
      if (fetch_stats) {
        sLse[(b ^ 1) * 128 + row] = st_max + log2f(st_den);
        sDbar[(b ^ 1) * 128 + row] = st_dbar;
      }
      incl = incl_next;
      incl_next = incl_next2;
      tmem_st_wait();
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tiles + 8 * odd);
    }
  }
  mbar_wait(sdone + 8, nsteps & 1, ctl, &g_status, kErrWaitMma);
  tc_fence_after();
  if (warp < 8) {
    // lane = key: each warpgroup stores 32 of the 64 columns of dk_main and dv
    float a[32];
    const int64_t o = ((int64_t)n * g.tk + ja) * kHeadDim + 32 * wg;
    tmem_ld32(tDK + lane_base + 32 * wg, a);
    tmem_ld_wait(a);
    if (!dead) {
#pragma unroll
      for (int e = 0; e < 32; e += 4)
        *reinterpret_cast<float4*>(dk_main + o + e) =
            make_float4(a[e] * g.scale, a[e + 1] * g.scale, a[e + 2] * g.scale, a[e + 3] * g.scale);
    }
    tmem_ld32(tDV + lane_base + 32 * wg, a);
    tmem_ld_wait(a);
    if (!dead) {
#pragma unroll
      for (int e = 0; e < 32; e += 8)
        *reinterpret_cast<uint4*>(dv + o + e) =
            make_uint4(pack_bf16(a[e], a[e + 1]), pack_bf16(a[e + 2], a[e + 3]),
                       pack_bf16(a[e + 4], a[e + 5]), pack_bf16(a[e + 6], a[e + 7]));
    }
  }
  drain_if_aborted(ctl);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 512);
}

// Barrier of the 128 threads of one warpgroup (named barriers 1 and 2).
__device__ __forceinline__ void wg_barrier(int wg) {
  if (wg == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
  else asm volatile("bar.sync 2, 128;" ::: "memory");
}

// Softmax-Jacobian corrections (the reference's BC + dq epilogue, kernels.py:777-826):
//   dk = dk_main - scale * P^T (ghat * Q)        (accumulated here per key block)
//   dq = dq_main - scale * ghat * (P K)          (added to dq_main with vector reductions;
//                                                 the reference reads a saved pk instead)
// One bf16 tile W[key][query] = p * ghat serves both products: K-major it is the A
// operand with M = keys, MN-major the A operand with M = queries.
// grid = n * ceil(t/128); 256 threads, the two warpgroups split the tile's query
// columns; TMEM: S^T 128, dKc 64, dQc 64 (256; two CTAs per SM).
constexpr int kCorrSmem = 3 * kTileBytes + 2 * kTileBytes + 2048 + 1024 + 256;

__global__ void __launch_bounds__(256, 2) backward_correction_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_dq, Geom g, const float* __restrict__ rmax,
    const float* __restrict__ rden, const float* __restrict__ ghat, const float* __restrict__ dk_main,
    __nv_bfloat16* __restrict__ dk) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem), sQ0 = sK + kTileBytes, sW = sK + 3 * kTileBytes;
  float2* sStat = reinterpret_cast<float2*>(smem + 5 * kTileBytes);           // [2][128] (lse, ghat)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 5 * kTileBytes + 2048);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t qfull = smem_u32(bars), sdone = smem_u32(bars + 2), dqdone = smem_u32(bars + 3);

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int n = (int)(blockIdx.x % g.n);
  const int jb = (int)(blockIdx.x / g.n);
  const int k0 = jb * kTileRows;
  const int nsteps = nqb - jb;
  const int64_t row_base = (int64_t)n * g.tq;

  auto load_stats = [&](int ib) {
    const int i = ib * kTileRows + row;
    float2 st = make_float2(INFINITY, 0.f);
    if (i < g.tq) st = make_float2(rmax[row_base + i] + log2f(rden[row_base + i]), ghat[row_base + i]);
    return st;
  };

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 4; ++i) mbar_init(qfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 256);
  if (wg == 1) sStat[row] = load_stats(jb);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;
  const uint32_t tS = tmem, tDK = tmem + 128, tDQ = tmem + 192;

  if (tid == 0) {
    mbar_expect_tx(qfull, 2 * kTileBytes);
    tma_load_tile(sK, &map_k, k0, n, qfull);
    tma_load_tile(sQ0, &map_q, jb * kTileRows, n, qfull);
    if (nsteps > 1) {
      mbar_expect_tx(qfull + 8, kTileBytes);
      tma_load_tile(sQ0 + kTileBytes, &map_q, (jb + 1) * kTileRows, n, qfull + 8);
    }
    mbar_wait(qfull, 0, ctl, &g_status, kErrWaitTma);
    tc_fence_after();
    mma_scores(tS, sK, sQ0, 128);
    mma_commit(sdone);
  }
  __syncwarp();

  const int ja = k0 + row;
  const bool dead = ja >= g.tk;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  for (int t = 0; t < nsteps; ++t) {
    const int ib = jb + t, b = t & 1;
    // next step's statistics as raw values: they are combined at the store below, when the
    // loads have long returned, so that no instruction waits for them here
    float nx_max = INFINITY, nx_den = 1.f, nx_gh = 0.f;
    if (wg == 1 && t + 1 < nsteps && (ib + 1) * kTileRows + row < g.tq) {
      const int64_t i = row_base + (ib + 1) * kTileRows + row;
      nx_max = rmax[i];
      nx_den = rden[i];
      nx_gh = ghat[i];
    }
    mbar_wait(sdone, t & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && t >= 1 && t + 1 < nsteps) {      // the Q stage of step t-1 is free
      mbar_expect_tx(qfull + 8 * (b ^ 1), kTileBytes);
      tma_load_tile(sQ0 + kTileBytes * (b ^ 1), &map_q, (ib + 1) * kTileRows, n, qfull + 8 * (b ^ 1));
    }
    __syncwarp();
    // this warpgroup's half of the W buffer doubled as its dQ staging area: the previous
    // step's reduction must have read it before it is written again
    if (row == 0) tma_wait_read_all();
    wg_barrier(wg);
    const int i0 = ib * kTileRows + 64 * wg;
    const bool masked_tile = dead || t == 0;
    const float4* St4 = reinterpret_cast<const float4*>(sStat + b * 128 + 64 * wg);
    auto tile = [&](auto mask_tag) {
    constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float vs[32];
      uint32_t wt[16];                                 // this chunk's 32 W values as bf16 pairs
      tmem_ld32(tS + lane_base + 64 * wg + 32 * c, vs);
      tmem_ld_wait(vs);
      float4 snext[4];
#pragma unroll
      for (int u2 = 0; u2 < 4; ++u2) snext[u2] = St4[(c * 32) / 2 + u2];
#pragma unroll
      for (int e8 = 0; e8 < 4; ++e8) {
        float w8[8];
        float4 scur[4];
#pragma unroll
        for (int u2 = 0; u2 < 4; ++u2) scur[u2] = snext[u2];
        if (e8 < 3) {      // next group's statistics, read before this group's store
#pragma unroll
          for (int u2 = 0; u2 < 4; ++u2) snext[u2] = St4[(c * 32 + (e8 + 1) * 8) / 2 + u2];
        }
#pragma unroll
        for (int u2 = 0; u2 < 4; ++u2) {
          const float4 st = scur[u2];
          const float lse[2] = {st.x, st.z}, gh[2] = {st.y, st.w};
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            const int u = u2 * 2 + w, e = e8 * 8 + u;
            float p = fast_exp2(fmaf(vs[e], g.zscale, -lse[w]));
            if (MASK && (dead || ja > i0 + c * 32 + e)) p = 0.f;
            w8[u] = p * gh[w];
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) wt[e8 * 4 + u] = pack_bf16(w8[2 * u], w8[2 * u + 1]);
        // shared memory: the MN-major A operand of dQc (M = queries)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sW + share_chunk_offset(row, wg * 64 + c * 32 + e8 * 8)),
                     "r"(wt[e8 * 4]), "r"(wt[e8 * 4 + 1]), "r"(wt[e8 * 4 + 2]), "r"(wt[e8 * 4 + 3])
                     : "memory");
      }
      // TMEM, over the score columns just consumed: the A operand of dKc (M = keys)
      tmem_st16(tS + lane_base + 64 * wg + 32 * c, wt);
    }
    };
    if (masked_tile) tile(std::true_type{}); else tile(std::false_type{});
    if (wg == 1 && t + 1 < nsteps) sStat[(b ^ 1) * 128 + row] = make_float2(nx_max + log2f(nx_den), nx_gh);
    tmem_st_wait();
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t id_kd = instr_desc(128, 64, 0, 1), id_qd = instr_desc(128, 64, 1, 1);
      // descriptors are built once per tile; a k-step is a constant 2048 B (128 units) further
      const Desc dQm = make_desc(sQ0 + kTileBytes * b, kTileBytes, 1024);
      const Desc dWm = make_desc(sW, kTileBytes, 1024), dKm = make_desc(sK, kTileBytes, 1024);
      // dQc first: its tile is what the threads read out next, and only it reads the shared-
      // memory W tile (the staging area of that read-out); dKc takes W from TMEM and runs,
      // with the next scores, under the read-out
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) mma_ss(tDQ, dWm, 128 * kk, dKm, 128 * kk, id_qd, kk > 0);
      mma_commit(dqdone);
#pragma unroll
      for (int kq = 0; kq < 8; ++kq)
        mma_ts(tDK, tS + 64 * (kq >> 2) + 32 * ((kq & 3) >> 1) + 8 * (kq & 1), dQm, 128 * kq, id_kd,
               (t > 0 || kq > 0));
      if (t + 1 < nsteps) {
        mbar_wait(qfull + 8 * (b ^ 1), ((t + 1) >> 1) & 1, ctl, &g_status, kErrWaitTma);
        tc_fence_after();
        mma_scores(tS, sK, sQ0 + kTileBytes * (b ^ 1), 128);
      }
      mma_commit(sdone);
    }
    __syncwarp();
    mbar_wait(dqdone, t & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    {
      // lane = query: each warpgroup owns 32 of the 64 columns.  The fp32 tile is staged in
      // the (now free) W buffer in the copy engine's swizzled layout and added to dq_main
      // by ONE tensor reduction per warpgroup: 128 B per row instead of eight scattered
      // 16-byte reductions per thread.
      float dq[32];
      tmem_ld32(tDQ + lane_base + 32 * wg, dq);
      tmem_ld_wait(dq);
      const float ns = -g.scale;
      const uint32_t stage = sW + kTileBytes * wg + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage + ((c ^ (row & 7)) << 4)),
                     "f"(dq[4 * c] * ns), "f"(dq[4 * c + 1] * ns), "f"(dq[4 * c + 2] * ns), "f"(dq[4 * c + 3] * ns)
                     : "memory");
      fence_async_smem();
      tc_fence_before();
      wg_barrier(wg);
      if (row == 0) tma_reduce_add_tile(&map_dq, sW + kTileBytes * wg, 32 * wg, ib * kTileRows, n);
    }
    tc_fence_before();
  }
  if (row == 0) tma_wait_read_all();
  mbar_wait(sdone, nsteps & 1, ctl, &g_status, kErrWaitMma);
  tc_fence_after();
  {
    // lane = key: each warpgroup finishes 32 of the 64 columns of dk
    float a[32];
    const int64_t o = ((int64_t)n * g.tk + ja) * kHeadDim + 32 * wg;
    tmem_ld32(tDK + lane_base + 32 * wg, a);
    tmem_ld_wait(a);
    if (!dead) {
      float m[32];
#pragma unroll
      for (int e = 0; e < 32; e += 4) {
        const float4 x = *reinterpret_cast<const float4*>(dk_main + o + e);
        m[e] = x.x - g.scale * a[e];
        m[e + 1] = x.y - g.scale * a[e + 1];
        m[e + 2] = x.z - g.scale * a[e + 2];
        m[e + 3] = x.w - g.scale * a[e + 3];
      }
#pragma unroll
      for (int e = 0; e < 32; e += 8)
        *reinterpret_cast<uint4*>(dk + o + e) =
            make_uint4(pack_bf16(m[e], m[e + 1]), pack_bf16(m[e + 2], m[e + 3]),
                       pack_bf16(m[e + 4], m[e + 5]), pack_bf16(m[e + 6], m[e + 7]));
    }
  }
  drain_if_aborted(ctl);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// dq = bf16(dq_main)
__global__ void cast_dq_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n4) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 x = reinterpret_cast<const float4*>(src)[i];
  reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w));
}

// ---------------------------------------------------------------- host launchers
#define DILUTION_TC_HAS_MAIN 1
#define DILUTION_TC_HAS_BACKWARD 1

// The opt-in to more than 48 KB of dynamic shared memory is per kernel and per device: it is
// made on the first launch of that kernel on that device and remembered.
inline int set_smem_attr(const void* fn, int bytes, char* err, size_t errlen) {
  constexpr int kKernels = 16, kDevices = 64;
  static std::mutex mu;
  static const void* fns[kKernels];
  static bool done[kKernels][kDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kDevices) dev = -1;
  int slot = -1;
  if (dev >= 0) {
    std::lock_guard<std::mutex> lk(mu);
    for (int i = 0; i < kKernels && slot < 0; ++i) {
      if (fns[i] == fn) slot = i;
      else if (fns[i] == nullptr) { fns[i] = fn; slot = i; }
    }
    if (slot >= 0 && done[slot][dev]) return 0;
  }
  const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    snprintf(err, errlen, "cudaFuncSetAttribute(%d): %s", bytes, cudaGetErrorString(e));
    return 3;
  }
  if (slot >= 0) {
    std::lock_guard<std::mutex> lk(mu);
    done[slot][dev] = true;
  }
  return 0;
}

inline int launch_status(const char* what, char* err, size_t errlen) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(err, errlen, "%s: %s", what, cudaGetErrorString(e));
    return 3;
  }
  return 0;
}

// Shared memory of the 256-column kernels is padded so that at most two CTAs share
// an SM (an SM has 512 TMEM columns); the 128-column kernels fit four by themselves.
constexpr int kTwoPerSm = 100 * 1024;
static_assert(5 * (kRowstatsSmem + 1024) > 233472 && 5 * (kColsumSmem + 1024) > 233472,
              "at most four CTAs of a 128-column kernel may share an SM");

// Compile-time bid / share of a launch from the run-time fields of its geometry.
#define DIL_TC_SHARE(g, ...)                                                                       \
  if ((g).share == kShareInclusive) { constexpr int SHARE = kShareInclusive; __VA_ARGS__; }        \
  else if ((g).share == kShareExclusive) { constexpr int SHARE = kShareExclusive; __VA_ARGS__; }   \
  else { constexpr int SHARE = kShareNone; __VA_ARGS__; }
#define DIL_TC_BID(g, ...)                                                     \
  if ((g).bid == kBidSigmoid) { constexpr int BID = kBidSigmoid; __VA_ARGS__; } \
  else { constexpr int BID = kBidSoftmax; __VA_ARGS__; }

inline int rowstats(const void* q, const void* k, const Geom& g, float* rmax, float* rden,
                    cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  constexpr int smem = kRowstatsSmem;
  if (int rc = set_smem_attr((const void*)rowstats_kernel, smem, err, errlen)) return rc;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  rowstats_kernel<<<(unsigned)(g.n * nqb), 256, smem, st>>>(mq, mk, g, rmax, rden);
  return launch_status("tc rowstats", err, errlen);
}

inline int colsum_scan(const void* q, const void* k, const Geom& g, const float* rmax,
                       const float* rden, const float* carry_base, float* carry, float* total,
                       cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  constexpr int smem = kColsumSmem;
  const int nkb = (g.tk + kTileRows - 1) / kTileRows;
  const unsigned grid = (unsigned)(g.n * nkb);
  if (g.carry_rows == 32) {
    DIL_TC_BID(g, {
      if (int rc = set_smem_attr((const void*)colsum_scan_kernel<32, BID>, smem, err, errlen)) return rc;
      colsum_scan_kernel<32, BID><<<grid, 256, smem, st>>>(mq, mk, g, rmax, rden, carry_base, carry, total);
    })
  } else {
    DIL_TC_BID(g, {
      if (int rc = set_smem_attr((const void*)colsum_scan_kernel<64, BID>, smem, err, errlen)) return rc;
      colsum_scan_kernel<64, BID><<<grid, 256, smem, st>>>(mq, mk, g, rmax, rden, carry_base, carry, total);
    })
  }
  return launch_status("tc colsum_scan", err, errlen);
}

inline int forward_main(const void* q, const void* k, const void* v, const Geom& g, const float* rmax,
                        const float* rden, const float* carry, const float* carry_base, float* out,
                        float* ssum, cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk, mv;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  if (int rc = make_map(&mv, v, g.n, g.tk, err, errlen)) return rc;
  constexpr int smem = kMainSmem;
  static_assert(2 * (smem + 1024) <= 233472 && 3 * (smem + 1024) > 233472, "exactly two CTAs of the main pass fit one SM");
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const unsigned grid = (unsigned)(g.n * nqb);
  DIL_TC_BID(g, DIL_TC_SHARE(g, {
    if (int rc = set_smem_attr((const void*)forward_main_kernel<BID, SHARE>, smem, err, errlen)) return rc;
    forward_main_kernel<BID, SHARE><<<grid, 256, smem, st>>>(mq, mk, mv, g, rmax, rden, carry, carry_base, out, ssum);
  }))
  return launch_status("tc forward_main", err, errlen);
}

int backward_tail_with_pk(const CUtensorMap& mq, const CUtensorMap& mk, const Geom& g, const float* rmax,
                          const float* rden, const float* ghat, const float* dk_main, const float* dq_main,
                          const float* pk, void* dq, void* dk, cudaStream_t st, char* err, size_t errlen,
                          void (*mark)(const char*, cudaStream_t, int));

// dop: (n, t, 64) bf16 scratch for the pre-scaled dout.  pk: the query correction saved by the
// forward (rowstats_pk), or null: the correction pass then recomputes it.
inline int backward(const void* q, const void* k, const void* v, const Geom& g, const void* dout,
                    int dout_dtype, const float* out, const float* rmax, const float* rden, const float* carry,
                    const float* total, const float* ssum, const float* pk, float* dq_main, float* dk_main,
                    float* ghat,
                    float* dbarp, void* dop, void* dq, void* dk, void* dv, cudaStream_t st, char* err,
                    size_t errlen, void (*mark)(const char*, cudaStream_t, int)) {
  CUtensorMap mq, mk;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  CUtensorMap md;
  if (int rc = make_map(&md, dop, g.n, g.tq, err, errlen)) return rc;
  const int64_t rows = g.n * g.tq;
  const int nkb = (g.tk + kTileRows - 1) / kTileRows;
  mark("tc_backward_prep", st, 0);
  if (dout_dtype == 0)
    backward_prep_kernel<float><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(
        (const float*)dout, out, ssum, g.eps, rows, dbarp, (__nv_bfloat16*)dop, ghat, dq_main);
  else
    backward_prep_kernel<__nv_bfloat16><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(
        (const __nv_bfloat16*)dout, out, ssum, g.eps, rows, dbarp, (__nv_bfloat16*)dop, ghat, dq_main);
  mark("tc_backward_prep", st, 1);
  if (int rc = launch_status("tc backward_prep", err, errlen)) return rc;
  CUtensorMap mdq;
  if (int rc = make_map_f32(&mdq, dq_main, g.n, g.tq, err, errlen)) return rc;
  if (g.carry_rows == 32) {
    constexpr int smem_bwd = kBwdSmem;
    static_assert(smem_bwd <= 232448 && 2 * smem_bwd > 233472, "the backward main pass runs one CTA per SM");
    mark("tc_backward_main", st, 0);
    const unsigned grid = (unsigned)(g.n * nkb);
    DIL_TC_BID(g, DIL_TC_SHARE(g, {
      if (int rc = set_smem_attr((const void*)backward_main_kernel<BID, SHARE>, smem_bwd, err, errlen)) return rc;
      backward_main_kernel<BID, SHARE><<<grid, kBwdThreads, smem_bwd, st>>>(
          mq, mk, md, mdq, g, (const __nv_bfloat16*)v, rmax, rden, dbarp, carry, total, dq_main, dk_main,
          (__nv_bfloat16*)dv, ghat);
    }))
  } else {
    snprintf(err, errlen, "the tensor-core backward needs checkpoints every 32 query rows (got %d)", g.carry_rows);
    return 1;
  }
  mark("tc_backward_main", st, 1);
  if (int rc = launch_status("tc backward_main", err, errlen)) return rc;
  if (!g.normalised || g.share == kShareNone) {
    // no row normalisation in the bid: no Jacobian correction, dk and dq are dk_main and dq_main.
    // Without a share step the correction of the softmax bid vanishes identically:
    // ghat_i = sum_j p_ij (do_i.v_j - do_i.out_i) = do_i.out_i - do_i.out_i = 0 (out_i = sum_j p_ij v_j).
    const int64_t n4 = rows * kHeadDim / 4;
    mark("tc_cast_dk_dq", st, 0);
    cast_dq_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dk_main, (__nv_bfloat16*)dk, n4);
    cast_dq_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dq_main, (__nv_bfloat16*)dq, n4);
    mark("tc_cast_dk_dq", st, 1);
    return launch_status("tc cast_dk_dq", err, errlen);
  }
  if (pk != nullptr)
    return backward_tail_with_pk(mq, mk, g, rmax, rden, ghat, dk_main, dq_main, pk, dq, dk, st, err, errlen, mark);
  constexpr int smem = kCorrSmem > kTwoPerSm ? kCorrSmem : kTwoPerSm;
  if (int rc = set_smem_attr((const void*)backward_correction_kernel, smem, err, errlen)) return rc;
  mark("tc_backward_correction", st, 0);
  backward_correction_kernel<<<(unsigned)(g.n * nkb), 256, smem, st>>>(mq, mk, mdq, g, rmax, rden, ghat,
                                                                     dk_main, (__nv_bfloat16*)dk);
  mark("tc_backward_correction", st, 1);
  if (int rc = launch_status("tc backward_correction", err, errlen)) return rc;
  const int64_t n4 = rows * kHeadDim / 4;
  mark("tc_cast_dq", st, 0);
  cast_dq_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dq_main, (__nv_bfloat16*)dq, n4);
  mark("tc_cast_dq", st, 1);
  return launch_status("tc cast_dq", err, errlen);
}

// Self-test of the bounded wait: one CTA waits on an mbarrier phase that nothing will
// ever complete, with a short limit (about a millisecond).  The wait must give up,
// record kErrSelfTest and let the kernel return normally; nothing faults or hangs.
__global__ void selftest_wait_kernel(long long limit_cycles, int* __restrict__ gave_up) {
  __shared__ uint64_t bar;
  __shared__ Ctl ctl;
  if (threadIdx.x == 0) {
    ctl.abort = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  const bool ok = mbar_wait(smem_u32(&bar), 0, &ctl, &g_status, kErrSelfTest, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}

inline int selftest_wait(int* gave_up_dev, cudaStream_t st, char* err, size_t errlen) {
  selftest_wait_kernel<<<1, 64, 0, st>>>(2000000LL, gave_up_dev);
  return launch_status("selftest_wait", err, errlen);
}

// Reads (and clears) the device status word; synchronises the device.
inline int read_status(int* out) {
  int v = 0;
  // kernels on non-blocking streams are not ordered before a copy on the default stream
  if (cudaDeviceSynchronize() != cudaSuccess) return 3;
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return 3;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  }
  *out = v;
  return 0;
}

}  // namespace tc
}  // namespace dil
