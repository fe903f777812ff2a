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
// All kernels: 128 threads (warp w owns TMEM lanes 32w..32w+31), thread 0 issues
// TMA and MMA, two CTAs per SM overlap one CTA's MMA/TMA latency with the
// other's arithmetic.
#pragma once

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

// (n, t, 64) bf16 row-major -> 3-D map {64, t, n}, box {64, 128, 1}, 128-byte swizzle.
// Rows past t read as zero, and a box never crosses into the next (batch, head) row.
inline int make_map(CUtensorMap* map, const void* base, int64_t n, int64_t t, char* err, size_t errlen,
                    int box_rows = kTileRows) {
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
  return 0;
}

// (n, t, 64) fp32 row-major -> 3-D map {64, t, n}, box {32, 128, 1} (128 bytes wide),
// 128-byte swizzle: the target of the dQ tile reductions.
inline int make_map_f32(CUtensorMap* map, const void* base, int64_t n, int64_t t, char* err, size_t errlen) {
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

// log2-domain log-sum-exp of query i (+inf past the end, so that its p is 0)
__device__ __forceinline__ float load_lse(const float* __restrict__ rmax, const float* __restrict__ rden,
                                          int64_t row_base, int i, int tq) {
  return i < tq ? rmax[row_base + i] + log2f(rden[row_base + i]) : INFINITY;
}

// ---------------------------------------------------------------- pass 1: row statistics
// grid = n * ceil(tq/128), longest rows first.  S = Q K^T, lane = query: each
// thread reduces its 64 key columns of the tile with an online max / sum; the two
// halves of a row are merged once at the end.  TMEM: 128 columns; 4 CTAs per SM.
constexpr int kRowstatsSmem = 3 * kTileBytes + 1024 + 1024 + 256;

__global__ void __launch_bounds__(256, 3) rowstats_kernel(const __grid_constant__ CUtensorMap map_q,
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
#pragma unroll 1
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
          for (int e = 0; e < 32; ++e) ps += fast_exp2(fmaf(v[e], g.zscale, -nm));
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
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 128);
}

// ---------------------------------------------------------------- pass 2: column sums + scan
// grid = n * ceil(tk/128), key blocks with the most query blocks first.
// S^T = K Q^T, lane = key.  The CTA keeps its K tile and walks the query blocks
// in causal order.  Each warpgroup sums p over its 64 queries of the tile; the
// thread of warpgroup 0 owns the key's running sum — the exclusive scan — and
// stores one checkpoint per 64 query rows, one tile behind the sums.
constexpr int kColsumSmem = 3 * kTileBytes + 1024 + 1024 + 1024 + 256;

__global__ void __launch_bounds__(256, 3) colsum_scan_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, Geom g,
    const float* __restrict__ rmax, const float* __restrict__ rden,
    const float* __restrict__ carry_base, float* __restrict__ carry, float* __restrict__ total) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem), sQ0 = sK + kTileBytes;
  float* sL = reinterpret_cast<float*>(smem + 3 * kTileBytes);                 // [2][128]
  float* sCs = reinterpret_cast<float*>(smem + 3 * kTileBytes + 1024);         // [2][128] sums of warpgroup 1
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes + 2048);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t qfull = smem_u32(bars), sdone = smem_u32(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int ncb = (g.tq + kCarryRows - 1) / kCarryRows;
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
  if (nib > 0 && wg == 0) sL[row] = load_lse(rmax, rden, row_base, ib0 * kTileRows + row, g.tq);
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
  float local = 0.f, prev = 0.f;      // warpgroup 0: scan state and its own sum of the previous tile
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
    if (wg == 1 && it + 1 < nib) lse_next = load_lse(rmax, rden, row_base, (ib + 1) * kTileRows + row, g.tq);
    if (wg == 0 && it > 0) {
      const int rb = (ib - 1) * 2;
      if (live) {
        if (rb < ncb) carry[((int64_t)n * ncb + rb) * g.tk + ja] = base + local;
        if (rb + 1 < ncb) carry[((int64_t)n * ncb + rb + 1) * g.tk + ja] = base + local + prev;
      }
      local += prev + sCs[((it - 1) & 1) * 128 + row];
    }
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
    float colsum = 0.f;
    auto tile = [&](auto edge_tag) {
      constexpr bool EDGE = decltype(edge_tag)::value;
#pragma unroll 1
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
            float p = fast_exp2(fmaf(v[e4 * 4 + u], g.zscale, -ls[u]));
            if (EDGE && ja > i0 + c * 32 + e4 * 4 + u) p = 0.f;
            part[u] += p;
          }
        }
        colsum += (part[0] + part[1]) + (part[2] + part[3]);
      }
    };
    if (edge) tile(std::true_type{}); else tile(std::false_type{});
    if (wg == 0) prev = colsum; else sCs[b * 128 + row] = colsum;
    if (wg == 1 && it + 1 < nib) sL[128 * (b ^ 1) + row] = lse_next;
    tc_fence_before();
    __syncthreads();
  }
  if (wg == 0 && live) {
    if (nib > 0) {
      const int rb = (nqb - 1) * 2;
      if (rb < ncb) carry[((int64_t)n * ncb + rb) * g.tk + ja] = base + local;
      if (rb + 1 < ncb) carry[((int64_t)n * ncb + rb + 1) * g.tk + ja] = base + local + prev;
      local += prev + sCs[((nib - 1) & 1) * 128 + row];
    }
    total[(int64_t)n * g.tk + ja] = local;
  }
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
  const int ncb = (g.tq + kCarryRows - 1) / kCarryRows;
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
  if (wg == 0) sL[row] = load_lse(rmax, rden, (int64_t)n * g.tq, ib * kTileRows + row, g.tq);
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

  // the checkpoint row this warpgroup starts from: rows 2*ib (queries 0-63) and 2*ib+1 (64-127)
  const int rb = 2 * ib + wg;
  const bool have_rows = rb < ncb;                 // false only for a ragged last half block
  const int64_t carry_row = ((int64_t)n * ncb + (have_rows ? rb : 0)) * g.tk;
  const float4* L4 = reinterpret_cast<const float4*>(sL + 64 * wg);
  const uint32_t taddr = tS + ((uint32_t)((warp & 3) * 32) << 16) + 64 * wg;
  const int qh = q0 + 64 * wg;                     // absolute position of this half's first query
  auto load_den = [&](int jbx) {
    const int jx = jbx * kTileRows + row;
    float d = g.eps;
    if (jx < g.tk && have_rows) {
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
#pragma unroll 1
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
            float p = fast_exp2(fmaf(v[e], g.zscale, -ls[u]));
            if (MASK && (dead || ja > qh + c * 32 + e)) p = 0.f;
            den += p;
            sh[u] = p * fast_rcp(den);
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
      const uint32_t id_o = instr_desc(128, 80, 1, 1);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        mma_ss(tO, smem_desc(sSh + 2048 * kk, kTileBytes, 1024), smem_desc(sV + 2048 * kk, sOnes - sV, 1024), id_o,
               (jb > 0 || kk > 0));
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
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// ---------------------------------------------------------------- pass 4: backward
// Pre-pass, one warp per query row: sinv = 1/(ssum+eps); dbar' = sinv * (dout . out);
// do' = bf16(sinv * dout); zeroes the dq / ghat accumulators.  Folding sinv into dO
// turns  ds = (do.v - dbar) * sinv  into  do'.v - dbar'  and  dv = attn^T do  into
// share^T do', so the main pass never multiplies by sinv per element.
__global__ void backward_prep_kernel(const float* __restrict__ dout, const float* __restrict__ out,
                                     const float* __restrict__ ssum, float eps, int64_t rows,
                                     float* __restrict__ dbarp, __nv_bfloat16* __restrict__ dop,
                                     float* __restrict__ ghat, float* __restrict__ dq_main) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float2 a = reinterpret_cast<const float2*>(dout + row * kHeadDim)[lane];
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

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Main reverse pass (the reference's BA, kernels.py:677-775).  grid = n * ceil(t/128),
// key blocks with the most query blocks first; 256 threads, one CTA per SM (464 TMEM
// columns: S^T 128 | dOV^T 128 | dV 64 | dK 64 | dQ 64 + ghat 16 as one 80-column tile).
// The CTA keeps the K and V tiles of 128 keys and walks the 128-row query blocks from
// last to first.  S^T = K Q^T and (dO' V^T)^T = V dO'^T are [128 keys x 128 queries],
// lane = key.  Two threads share a key: warpgroup 0 walks queries 127..64 of the tile,
// warpgroup 1 queries 63..0, both backwards, each with two registers:
//   incl   : demand of the key including the current query.  It starts from the stored
//            checkpoint of the next 64-row block and is walked backwards by subtracting
//            p, so committed + p + eps = incl + eps needs no forward sweep and the two
//            halves are independent;
//   suffix : running sum of dk_share over later queries (kernels.py:763-764).  Warpgroup
//            1 does not yet know the sum G0 of warpgroup 0's half; dp is linear in the
//            suffix, so pdp (fp32) and p (bf16) stay in registers, and after one
//            block-wide barrier p * G0 is added before the pdp tile is stored.  Both
//            warpgroups run this same instruction stream (warpgroup 0 adds zero): two
//            unrolled variants did not fit the instruction cache with 8 warps.
// Per step the CTA writes two bf16 tiles [key][query]: share and pdp = p * dp.  Read as
// K-major they are A operands with M = keys (dV += share^T dO', dK += pdp^T Q); pdp read
// as MN-major is the A operand with M = queries: one MMA with N = 80 against
// B = [K | ones] yields dQ = pdp K in 64 columns and ghat = pdp 1 in the next 16.  dQ has
// its own columns, so the next step's score MMAs are issued right behind this step's
// and the dQ read-out runs under them.
constexpr int kBwdSmem = 11 * kTileBytes + 2048 + 1024 + 1024 + 256;

__global__ void __launch_bounds__(256, 1) backward_main_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, Geom g,
    const float* __restrict__ rmax, const float* __restrict__ rden, const float* __restrict__ dbarp,
    const float* __restrict__ carry, const float* __restrict__ total, float* __restrict__ dq_main,
    float* __restrict__ dk_main, __nv_bfloat16* __restrict__ dv, float* __restrict__ ghat) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem), sV = sK + kTileBytes;
  const uint32_t sQ0 = sK + 2 * kTileBytes, sD0 = sK + 4 * kTileBytes;     // [2] each
  const uint32_t sSh = sK + 6 * kTileBytes, sPd = sK + 8 * kTileBytes;      // 32 KB each
  // a [128 keys][64] bf16 tile of ones: the second 64-column group of the dQ MMA's B operand
  // (N = 80 = 64 columns of K + 16 of ones), so ghat comes out of the same instruction
  const uint32_t sOnes = sK + 10 * kTileBytes;
  uint8_t* ones_ptr = smem + 10 * kTileBytes;
  float2* sStat = reinterpret_cast<float2*>(smem + 11 * kTileBytes);          // [2][128] (lse, dbar')
  float* sG = reinterpret_cast<float*>(smem + 11 * kTileBytes + 2048);        // [2][128] half sums of dk_share
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 11 * kTileBytes + 3072);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t kvfull = smem_u32(bars), qfull = smem_u32(bars + 1);         // qfull[2]
  const uint32_t sdone = smem_u32(bars + 3), dqdone = smem_u32(bars + 4);

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int half = 1 - wg;                          // warpgroup 0 owns the later 64 queries
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int ncb = (g.tq + kCarryRows - 1) / kCarryRows;
  const int n = (int)(blockIdx.x % g.n);
  const int jb = (int)(blockIdx.x / g.n);
  const int k0 = jb * kTileRows;
  const int nsteps = nqb - jb;                     // query blocks jb .. nqb-1, visited in reverse
  const int64_t row_base = (int64_t)n * g.tq;
  const int ja = k0 + row;
  const bool dead = ja >= g.tk;

  auto load_stats = [&](int ib) {
    const int i = ib * kTileRows + row;
    float2 st = make_float2(INFINITY, 0.f);
    if (i < g.tq) st = make_float2(rmax[row_base + i] + log2f(rden[row_base + i]), dbarp[row_base + i]);
    return st;
  };
  // demand of this thread's key through the last query of its half of block ib
  auto load_incl = [&](int ib) {
    const int rb = 2 * ib + half + 1;
    if (dead) return 0.f;
    return rb < ncb ? carry[((int64_t)n * ncb + rb) * g.tk + ja] : total[(int64_t)n * g.tk + ja];
  };

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 5; ++i) mbar_init(kvfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 512);
  if (wg == 0) sStat[row] = load_stats(nqb - 1);
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
  const uint32_t tS = tmem, tDOV = tmem + 128, tDV = tmem + 256, tDK = tmem + 320, tDQ = tmem + 384,
                 tG = tmem + 448;

  if (tid == 0) {
    mbar_expect_tx(kvfull, 2 * kTileBytes);
    tma_load_tile(sK, &map_k, k0, n, kvfull);
    tma_load_tile(sV, &map_v, k0, n, kvfull);
    mbar_expect_tx(qfull, 2 * kTileBytes);
    tma_load_tile(sQ0, &map_q, (nqb - 1) * kTileRows, n, qfull);
    tma_load_tile(sD0, &map_do, (nqb - 1) * kTileRows, n, qfull);
    mbar_wait(kvfull, 0, ctl, &g_status, kErrWaitTma);
    mbar_wait(qfull, 0, ctl, &g_status, kErrWaitTma);
    tc_fence_after();
    mma_scores(tS, sK, sQ0, 128);
    mma_scores(tDOV, sV, sD0, 128);
    mma_commit(sdone);
  }
  __syncwarp();

  float suffix_in = 0.f;                            // suffix entering the tile (same in both warpgroups)
  float incl = load_incl(nqb - 1);
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const int qbase = 64 * half;                      // first query column of this warpgroup
  for (int t = 0; t < nsteps; ++t) {
    const int ib = nqb - 1 - t, b = t & 1;
    // fetch what the next tile needs before waiting for this one
    float2 stat_next = make_float2(INFINITY, 0.f);
    float incl_next = 0.f;
    if (t + 1 < nsteps) {
      if (wg == 0) stat_next = load_stats(ib - 1);
      incl_next = load_incl(ib - 1);
    }
    mbar_wait(sdone, t & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && t + 1 < nsteps) {               // buffers of step t-1 are free
      mbar_expect_tx(qfull + 8 * (b ^ 1), 2 * kTileBytes);
      tma_load_tile(sQ0 + kTileBytes * (b ^ 1), &map_q, (ib - 1) * kTileRows, n, qfull + 8 * (b ^ 1));
      tma_load_tile(sD0 + kTileBytes * (b ^ 1), &map_do, (ib - 1) * kTileRows, n, qfull + 8 * (b ^ 1));
    }
    __syncwarp();
    const int i0 = ib * kTileRows;                   // first query of the tile (q_off == 0 here)
    const bool masked_tile = dead || (i0 < k0 + kTileRows - 1);
    const float4* St4 = reinterpret_cast<const float4*>(sStat + b * 128);
    float suffix = suffix_in;
    float pdk[64];                                   // warpgroup 1: pdp without warpgroup 0's half sum
    uint32_t pk2[32];                                // warpgroup 1: p as bf16 pairs

    // one chunk = 32 queries [qc, qc+32) of the tile, visited from the last to the first
    auto chunk = [&](auto mask_tag, auto keep_tag, const float* vs, const float* vd, int qc, int slot) {
      constexpr bool MASK = decltype(mask_tag)::value;
      constexpr bool KEEP = decltype(keep_tag)::value;
      uint32_t shp[16];                              // this chunk's 32 shares as bf16 pairs
#pragma unroll
      for (int e8 = 3; e8 >= 0; --e8) {
        float sh[8], pd[8], pp[8];
#pragma unroll
        for (int u2 = 3; u2 >= 0; --u2) {
          const float4 st = St4[(qc + e8 * 8) / 2 + u2];       // two queries: (lse, dbar') x2
          const float lse[2] = {st.x, st.z}, dbr[2] = {st.y, st.w};
#pragma unroll
          for (int w = 1; w >= 0; --w) {
            const int u = u2 * 2 + w, e = e8 * 8 + u;
            float p = fast_exp2(fmaf(vs[e], g.zscale, -lse[w]));
            bool off = false;
            if (MASK) {
              off = dead || ja > i0 + qc + e;
              if (off) p = 0.f;
            }
            // with inv = 1/(committed+p+eps), share = p*inv and w = ds*inv:
            //   ds*(committed+eps)*inv^2 = w*(1-share),  dk_share = -w*share
            const float den = MASK ? fmaxf(incl + g.eps, g.eps) : incl + g.eps;
            const float inv = fast_rcp(den);
            const float wv = (vd[e] - dbr[w]) * inv;
            const float share = p * inv;
            const float gneg = wv * share;                     // -dk_share
            pd[u] = p * ((wv - gneg) + suffix);                // p * dp
            sh[u] = share;
            pp[u] = p;
            if (!MASK || !off) {
              suffix -= gneg;
              incl -= p;
            }
          }
        }
        const uint32_t off8 = share_chunk_offset(row, qc + e8 * 8);
#pragma unroll
        for (int u = 0; u < 4; ++u) shp[e8 * 4 + u] = pack_bf16(sh[2 * u], sh[2 * u + 1]);
        if (KEEP) {
#pragma unroll
          for (int u = 0; u < 8; ++u) pdk[slot * 32 + e8 * 8 + u] = pd[u];
#pragma unroll
          for (int u = 0; u < 4; ++u) pk2[slot * 16 + e8 * 4 + u] = pack_bf16(pp[2 * u], pp[2 * u + 1]);
        } else {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sPd + off8),
                       "r"(pack_bf16(pd[0], pd[1])), "r"(pack_bf16(pd[2], pd[3])),
                       "r"(pack_bf16(pd[4], pd[5])), "r"(pack_bf16(pd[6], pd[7]))
                       : "memory");
        }
      }
      // the shares stay in TMEM, over score columns this warpgroup has already consumed (the
      // upper half of its own 64-column range): lane = key is the M index of
      // dV += share^T dO', two queries per 32-bit column
      tmem_st16(tS + lane_base + qbase + 32 + 16 * slot, shp);
    };
    auto run = [&](auto keep_tag) {
#pragma unroll
      for (int c = 1; c >= 0; --c) {
        float vs[32], vd[32];
        tmem_ld32(tS + lane_base + qbase + 32 * c, vs);
        tmem_ld32(tDOV + lane_base + qbase + 32 * c, vd);
        tmem_ld_wait(vs);
        tmem_ld_wait(vd);
        if (masked_tile) chunk(std::true_type{}, keep_tag, vs, vd, qbase + 32 * c, c);
        else chunk(std::false_type{}, keep_tag, vs, vd, qbase + 32 * c, c);
      }
    };
    run(std::true_type{});                           // one instruction stream for both warpgroups
    const float gsum = suffix - suffix_in;           // this half's sum of dk_share
    if (wg == 0) sG[row] = gsum;
    __syncthreads();                                 // warpgroup 0's half sums are visible
    float g0 = gsum, g1 = gsum;
    if (wg == 1) {
      g0 = sG[row];
      sG[128 + row] = gsum;
    }
    {
      const float fix = wg == 1 ? g0 : 0.f;          // warpgroup 0 started from the exact suffix
#pragma unroll
      for (int c = 1; c >= 0; --c) {
        uint32_t pdt[16];                              // this chunk's 32 pdp values as bf16 pairs
#pragma unroll
        for (int e8 = 3; e8 >= 0; --e8) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint32_t pr = pk2[c * 16 + e8 * 4 + u];
            const float plo = __uint_as_float(pr << 16), phi = __uint_as_float(pr & 0xffff0000u);
            pdt[e8 * 4 + u] = pack_bf16(fmaf(plo, fix, pdk[c * 32 + e8 * 8 + 2 * u]),
                                        fmaf(phi, fix, pdk[c * 32 + e8 * 8 + 2 * u + 1]));
          }
          // shared memory: the MN-major A operand of dQ | ghat (M = queries)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sPd + share_chunk_offset(row, qbase + 32 * c + e8 * 8)),
                       "r"(pdt[e8 * 4]), "r"(pdt[e8 * 4 + 1]), "r"(pdt[e8 * 4 + 2]), "r"(pdt[e8 * 4 + 3])
                       : "memory");
        }
        // TMEM, over consumed dOV^T columns: the A operand of dK (M = keys)
        tmem_st16(tDOV + lane_base + qbase + 32 + 16 * c, pdt);
      }
    }
    if (wg == 0 && t + 1 < nsteps) sStat[(b ^ 1) * 128 + row] = stat_next;
    incl = incl_next;
    tmem_st_wait();
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (wg == 0) g1 = sG[128 + row];
    suffix_in += g0 + g1;
    if (tid == 0) {
      tc_fence_after();
      const uint32_t id_kd = instr_desc(128, 64, 0, 1);   // A K-major (M = keys), B MN-major
      const uint32_t id_qd = instr_desc(128, 80, 1, 1);   // A MN-major (M = queries); B = [K | ones]
      const uint32_t sQ = sQ0 + kTileBytes * b, sD = sD0 + kTileBytes * b;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {                    // contraction over the 128 keys
        const uint64_t a = smem_desc(sPd + 2048 * kk, kTileBytes, 1024);
        mma_ss(tDQ, a, smem_desc(sK + 2048 * kk, sOnes - sK, 1024), id_qd, kk > 0);
      }
      mma_commit(dqdone);
#pragma unroll
      for (int kq = 0; kq < 8; ++kq) {                    // contraction over the 128 queries
        // queries [16kq, 16kq+16): 8 columns in the upper half of the owning warpgroup's score range
        const uint32_t a_sh = tS + 64 * (kq >> 2) + 32 + 16 * ((kq & 3) >> 1) + 8 * (kq & 1);
        mma_ts(tDV, a_sh, smem_desc(sD + 2048 * kq, kTileBytes, 1024), id_kd, (t > 0 || kq > 0));
        mma_ts(tDK, a_sh - tS + tDOV, smem_desc(sQ + 2048 * kq, kTileBytes, 1024), id_kd, (t > 0 || kq > 0));
      }
      if (t + 1 < nsteps) {
        mbar_wait(qfull + 8 * (b ^ 1), ((t + 1) >> 1) & 1, ctl, &g_status, kErrWaitTma);
        tc_fence_after();
        mma_scores(tS, sK, sQ0 + kTileBytes * (b ^ 1), 128);
        mma_scores(tDOV, sV, sD0 + kTileBytes * (b ^ 1), 128);
      }
      mma_commit(sdone);
    }
    __syncwarp();
    // dQ and ghat of this tile: lane = query, each warpgroup takes 32 of the 64 columns.
    // Runs under the remaining MMAs.
    mbar_wait(dqdone, t & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    {
      float dq[32], gh[32];
      tmem_ld32(tDQ + lane_base + 32 * wg, dq);
      if (wg == 0) tmem_ld32(tG + lane_base, gh);
      tmem_ld_wait(dq);
      const int i = i0 + row;
      if (i < g.tq) {
        float* dst = dq_main + (row_base + i) * kHeadDim + 32 * wg;
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4)
          red_add_v4(dst + 4 * c4, dq[4 * c4] * g.scale, dq[4 * c4 + 1] * g.scale,
                     dq[4 * c4 + 2] * g.scale, dq[4 * c4 + 3] * g.scale);
      }
      if (wg == 0) {
        tmem_ld_wait(gh);
        if (i < g.tq) atomicAdd(ghat + row_base + i, gh[0]);
      }
    }
    tc_fence_before();
  }
  mbar_wait(sdone, nsteps & 1, ctl, &g_status, kErrWaitMma);
  tc_fence_after();
  {
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
    float2 stat_next = make_float2(INFINITY, 0.f);
    if (wg == 1 && t + 1 < nsteps) stat_next = load_stats(ib + 1);
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
#pragma unroll 1
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
    if (wg == 1 && t + 1 < nsteps) sStat[(b ^ 1) * 128 + row] = stat_next;
    tmem_st_wait();
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t id_kd = instr_desc(128, 64, 0, 1), id_qd = instr_desc(128, 64, 1, 1);
      const uint32_t sQ = sQ0 + kTileBytes * b;
#pragma unroll
      for (int kq = 0; kq < 8; ++kq)
        mma_ts(tDK, tS + 64 * (kq >> 2) + 32 * ((kq & 3) >> 1) + 8 * (kq & 1),
               smem_desc(sQ + 2048 * kq, kTileBytes, 1024), id_kd, (t > 0 || kq > 0));
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        mma_ss(tDQ, smem_desc(sW + 2048 * kk, kTileBytes, 1024), smem_desc(sK + 2048 * kk, kTileBytes, 1024),
               id_qd, kk > 0);
      mma_commit(dqdone);                                // both products have read the W tile
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

inline int set_smem_attr(const void* fn, int bytes, char* err, size_t errlen) {
  const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    snprintf(err, errlen, "cudaFuncSetAttribute(%d): %s", bytes, cudaGetErrorString(e));
    return 3;
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
  if (int rc = set_smem_attr((const void*)colsum_scan_kernel, smem, err, errlen)) return rc;
  const int nkb = (g.tk + kTileRows - 1) / kTileRows;
  colsum_scan_kernel<<<(unsigned)(g.n * nkb), 256, smem, st>>>(mq, mk, g, rmax, rden, carry_base, carry,
                                                             total);
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
  if (int rc = set_smem_attr((const void*)forward_main_kernel, smem, err, errlen)) return rc;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  forward_main_kernel<<<(unsigned)(g.n * nqb), 256, smem, st>>>(mq, mk, mv, g, rmax, rden, carry, carry_base,
                                                              out, ssum);
  return launch_status("tc forward_main", err, errlen);
}

// dop: (n, t, 64) bf16 scratch for the pre-scaled dout.
inline int backward(const void* q, const void* k, const void* v, const Geom& g, const float* dout,
                    const float* out, const float* rmax, const float* rden, const float* carry,
                    const float* total, const float* ssum, float* dq_main, float* dk_main, float* ghat,
                    float* dbarp, void* dop, void* dq, void* dk, void* dv, cudaStream_t st, char* err,
                    size_t errlen, void (*mark)(const char*, cudaStream_t, int)) {
  CUtensorMap mq, mk, mv;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  if (int rc = make_map(&mv, v, g.n, g.tk, err, errlen)) return rc;
  CUtensorMap md;
  if (int rc = make_map(&md, dop, g.n, g.tq, err, errlen)) return rc;
  const int64_t rows = g.n * g.tq;
  const int nkb = (g.tk + kTileRows - 1) / kTileRows;
  mark("tc_backward_prep", st, 0);
  backward_prep_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(dout, out, ssum, g.eps, rows, dbarp,
                                                                  (__nv_bfloat16*)dop, ghat, dq_main);
  mark("tc_backward_prep", st, 1);
  if (int rc = launch_status("tc backward_prep", err, errlen)) return rc;
  constexpr int smem_bwd = kBwdSmem;
  static_assert(smem_bwd <= 232448 && 2 * smem_bwd > 233472, "the backward main pass runs one CTA per SM");
  if (int rc = set_smem_attr((const void*)backward_main_kernel, smem_bwd, err, errlen)) return rc;
  mark("tc_backward_main", st, 0);
  backward_main_kernel<<<(unsigned)(g.n * nkb), 256, smem_bwd, st>>>(
      mq, mk, mv, md, g, rmax, rden, dbarp, carry, total, dq_main, dk_main, (__nv_bfloat16*)dv, ghat);
  mark("tc_backward_main", st, 1);
  if (int rc = launch_status("tc backward_main", err, errlen)) return rc;
  constexpr int smem = kCorrSmem > kTwoPerSm ? kCorrSmem : kTwoPerSm;
  if (int rc = set_smem_attr((const void*)backward_correction_kernel, smem, err, errlen)) return rc;
  mark("tc_backward_correction", st, 0);
  CUtensorMap mdq;
  if (int rc = make_map_f32(&mdq, dq_main, g.n, g.tq, err, errlen)) return rc;
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
