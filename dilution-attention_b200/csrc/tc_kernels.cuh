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
inline int make_map(CUtensorMap* map, const void* base, int64_t n, int64_t t, char* err, size_t errlen) {
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
  const cuuint32_t box[3] = {(cuuint32_t)kHeadDim, (cuuint32_t)kTileRows, 1};
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

// ---------------------------------------------------------------- pass 1: row statistics
// grid = n * ceil(tq/128), longest rows first.  S = Q K^T, lane = query.
// Shared: Q tile, two K stages.  TMEM: two 128-column S buffers, so the MMA of
// key tile jb+1 runs while the threads reduce tile jb.
constexpr int kRowstatsSmem = 3 * kTileBytes + 1024 + 256;

__global__ void __launch_bounds__(128) rowstats_kernel(const __grid_constant__ CUtensorMap map_q,
                                                       const __grid_constant__ CUtensorMap map_k,
                                                       Geom g, float* __restrict__ rmax,
                                                       float* __restrict__ rden) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sQ = smem_u32(smem), sK0 = sQ + kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t kfull = smem_u32(bars), sdone = smem_u32(bars + 2);   // [2] each

  const int tid = threadIdx.x, warp = tid >> 5;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int n = (int)(blockIdx.x % g.n);
  const int ib = nqb - 1 - (int)(blockIdx.x / g.n);
  const int q0 = g.q_off + ib * kTileRows;                   // absolute position of row 0
  const int njb = min(g.tk - 1, q0 + kTileRows - 1) / kTileRows + 1;

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 4; ++i) mbar_init(kfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 256);
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
    mbar_wait(kfull, 0, ctl, &g_status, kErrWaitTma);
    tc_fence_after();
    mma_scores(tmem, sQ, sK0, 128);
    mma_commit(sdone);
  }
  __syncwarp();

  float m = -INFINITY, s = 0.f;
  const int ia = q0 + tid;
  for (int jb = 0; jb < njb; ++jb) {
    const int b = jb & 1;
    if (tid == 0 && jb + 1 < njb) {     // MMA of the next tile into the other S buffer
      mbar_wait(kfull + 8 * (b ^ 1), ((jb + 1) >> 1) & 1, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      mma_scores(tmem + 128 * (b ^ 1), sQ, sK0 + kTileBytes * (b ^ 1), 128);
      mma_commit(sdone + 8 * (b ^ 1));
    }
    __syncwarp();
    mbar_wait(sdone + 8 * b, (jb >> 1) & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && jb + 2 < njb) {     // this K stage is free again
      mbar_expect_tx(kfull + 8 * b, kTileBytes);
      tma_load_tile(sK0 + kTileBytes * b, &map_k, (jb + 2) * kTileRows, n, kfull + 8 * b);
    }
    __syncwarp();
    const bool edge = (jb * kTileRows + kTileRows - 1 > q0) || ((jb + 1) * kTileRows > g.tk);
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + 128 * b;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float v[32];
      tmem_ld32(taddr + 32 * c, v);
      tmem_ld_wait();
      float cmax = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        float z = v[e] * g.zscale;
        if (edge) {
          const int ja = jb * kTileRows + c * 32 + e;
          if (ja > ia || ja >= g.tk) z = -INFINITY;
        }
        v[e] = z;
        cmax = fmaxf(cmax, z);
      }
      const float nm = fmaxf(m, cmax);
      if (nm > -INFINITY) {
        float ps = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) ps += fast_exp2(v[e] - nm);
        s = s * fast_exp2(m - nm) + ps;
        m = nm;
      }
    }
    tc_fence_before();
    __syncthreads();
  }
  const int i = ib * kTileRows + tid;
  if (i < g.tq) {
    rmax[(int64_t)n * g.tq + i] = m;
    rden[(int64_t)n * g.tq + i] = s;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// ---------------------------------------------------------------- pass 2: column sums + scan
// grid = n * ceil(tk/128), key blocks with the most query blocks first.
// S^T = K Q^T, lane = key.  The CTA keeps its K tile and walks the query blocks
// in causal order; each thread's running sum of p over the queries seen so far
// is the exclusive scan, stored as a checkpoint every 64 query rows.
constexpr int kColsumSmem = 3 * kTileBytes + 2 * 128 * 4 + 1024 + 256;

__device__ __forceinline__ void stage_lse(float* dst, const float* __restrict__ rmax,
                                          const float* __restrict__ rden, int64_t row_base, int i,
                                          int tq) {
  // log2-domain log-sum-exp of one query; +inf for rows past the end so their p is 0
  dst[threadIdx.x] = i < tq ? rmax[row_base + i] + log2f(rden[row_base + i]) : INFINITY;
}

__global__ void __launch_bounds__(128) colsum_scan_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, Geom g,
    const float* __restrict__ rmax, const float* __restrict__ rden,
    const float* __restrict__ carry_base, float* __restrict__ carry, float* __restrict__ total) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem), sQ0 = sK + kTileBytes;
  float* sL = reinterpret_cast<float*>(smem + 3 * kTileBytes);            // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes + 1024);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t qfull = smem_u32(bars), sdone = smem_u32(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5;
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
    for (int i = 0; i < 4; ++i) mbar_init(qfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 256);
  if (nib > 0) stage_lse(sL, rmax, rden, row_base, ib0 * kTileRows + tid, g.tq);
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
    mbar_wait(qfull, 0, ctl, &g_status, kErrWaitTma);
    tc_fence_after();
    mma_scores(tmem, sK, sQ0, 128);
    mma_commit(sdone);
  }
  __syncwarp();

  const int ja = k0 + tid;
  const float base = (carry_base != nullptr && ja < g.tk) ? carry_base[(int64_t)n * g.tk + ja] : 0.f;
  float local = 0.f;
  for (int it = 0; it < nib; ++it) {
    const int ib = ib0 + it, b = it & 1;
    if (tid == 0 && it + 1 < nib) {
      mbar_wait(qfull + 8 * (b ^ 1), ((it + 1) >> 1) & 1, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      mma_scores(tmem + 128 * (b ^ 1), sK, sQ0 + kTileBytes * (b ^ 1), 128);
      mma_commit(sdone + 8 * (b ^ 1));
    }
    __syncwarp();
    if (it + 1 < nib) stage_lse(sL + 128 * (b ^ 1), rmax, rden, row_base, (ib + 1) * kTileRows + tid, g.tq);
    mbar_wait(sdone + 8 * b, (it >> 1) & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && it + 2 < nib) {
      mbar_expect_tx(qfull + 8 * b, kTileBytes);
      tma_load_tile(sQ0 + kTileBytes * b, &map_q, (ib + 2) * kTileRows, n, qfull + 8 * b);
    }
    __syncwarp();
    const int i0 = g.q_off + ib * kTileRows;          // absolute position of the tile's first query
    const bool edge = i0 < k0 + kTileRows - 1;         // the diagonal tile
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + 128 * b;
    const float4* L4 = reinterpret_cast<const float4*>(sL + 128 * b);
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
      float colsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_ld32(taddr + 64 * h + 32 * c, v);
        tmem_ld_wait();
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l = L4[h * 16 + c * 8 + e4];
          const float ls[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float p = fast_exp2(fmaf(v[e4 * 4 + u], g.zscale, -ls[u]));
            if (edge && ja > i0 + h * 64 + c * 32 + e4 * 4 + u) p = 0.f;
            colsum += p;
          }
        }
      }
      const int rb = ib * 2 + h;
      if (rb < ncb && ja < g.tk) carry[((int64_t)n * ncb + rb) * g.tk + ja] = base + local;
      local += colsum;
    }
    tc_fence_before();
    __syncthreads();
  }
  if (ja < g.tk) total[(int64_t)n * g.tk + ja] = local;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// ---------------------------------------------------------------- pass 3: main pass
// grid = n * ceil(tq/128), longest rows first.  S^T = K Q^T, lane = key.
// Each thread walks the 128 queries of the tile in order with its key's demand
// in one register:  den += p;  share = p / den  (den = committed + p + eps),
// and writes the bf16 share tile to shared memory as an MN-major operand
// ([key][query], 128-byte swizzle, two 64-query sub-tiles).  Two MMAs consume it:
//   O   [query x d ] += share   * V      (A = share MN-major, B = V MN-major)
//   rs  [query x 16] += share   * ones   (row sums of the SAME bf16 shares)
// so the final divide out = O / (rs + eps) normalises exactly what was summed.
// TMEM: S^T 128 columns, O 64, rs 16 (256 allocated; two CTAs per SM).
constexpr int kMainTiles = 4;   // Q, K x2, V
constexpr int kMainSmem = kMainTiles * kTileBytes + 2 * kTileBytes + 2048 + 512 + 1024 + 256;

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Byte offset of the 16-byte chunk holding queries [q, q+8) of `key` in an
// MN-major [128 keys][128 queries] bf16 tile (q a multiple of 8).
__device__ __forceinline__ uint32_t share_chunk_offset(int key, int q) {
  return (uint32_t)((q >> 6) * (int)kTileBytes + key * 128 + ((((q & 63) >> 3) ^ (key & 7)) << 4));
}

__global__ void __launch_bounds__(128) forward_main_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, Geom g, const float* __restrict__ rmax,
    const float* __restrict__ rden, const float* __restrict__ carry,
    const float* __restrict__ carry_base, float* __restrict__ out, float* __restrict__ ssum) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sQ = smem_u32(smem), sK0 = sQ + kTileBytes, sV = sQ + 3 * kTileBytes;
  const uint32_t sSh = sQ + 4 * kTileBytes, sOnes = sQ + 6 * kTileBytes;
  uint8_t* ones_ptr = smem + 6 * kTileBytes;
  float* sL = reinterpret_cast<float*>(smem + 6 * kTileBytes + 2048);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes + 2048 + 512);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t kfull = smem_u32(bars), vfull = smem_u32(bars + 2), sdone = smem_u32(bars + 3);

  const int tid = threadIdx.x, warp = tid >> 5;
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
  stage_lse(sL, rmax, rden, (int64_t)n * g.tq, ib * kTileRows + tid, g.tq);
  reinterpret_cast<uint4*>(ones_ptr)[tid] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;
  const uint32_t tS = tmem, tO = tmem + 128, tR = tmem + 192;

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

  const float4* L4 = reinterpret_cast<const float4*>(sL);
  const int64_t carry_row = ((int64_t)n * ncb + 2 * ib) * g.tk;
  for (int jb = 0; jb < njb; ++jb) {
    const int b = jb & 1;
    const int ja = jb * kTileRows + tid;
    // demand committed before this tile's first query, plus eps once
    float den = g.eps;
    if (ja < g.tk) {
      den += carry[carry_row + ja];
      if (carry_base != nullptr) den += carry_base[(int64_t)n * g.tk + ja];
    }
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
    const bool diag = jb * kTileRows + kTileRows - 1 > q0;
    const bool dead = ja >= g.tk;
    const uint32_t taddr = tS + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float v[32];
      tmem_ld32(taddr + 32 * c, v);
      tmem_ld_wait();
#pragma unroll
      for (int e8 = 0; e8 < 4; ++e8) {
        uint32_t packed[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float4 l = L4[c * 8 + e8 * 2 + h];
          const float ls[4] = {l.x, l.y, l.z, l.w};
          float sh[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e8 * 8 + h * 4 + u;
            float p = fast_exp2(fmaf(v[e], g.zscale, -ls[u]));
            if (dead || (diag && ja > q0 + c * 32 + e)) p = 0.f;
            den += p;
            sh[u] = p * fast_rcp(den);
          }
          packed[h * 2 + 0] = pack_bf16(sh[0], sh[1]);
          packed[h * 2 + 1] = pack_bf16(sh[2], sh[3]);
        }
        const uint32_t dst = sSh + share_chunk_offset(tid, c * 32 + e8 * 8);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]),
                     "r"(packed[1]), "r"(packed[2]), "r"(packed[3])
                     : "memory");
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      mbar_wait(vfull, jb & 1, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      const uint32_t id_o = instr_desc(128, 64, 1, 1), id_r = instr_desc(128, 16, 1, 0);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t a = smem_desc(sSh + 2048 * kk, kTileBytes, 1024);
        mma_ss(tO, a, smem_desc(sV + 2048 * kk, kTileBytes, 1024), id_o, (jb > 0 || kk > 0));
        mma_ss(tR, a, smem_desc(sOnes + 32 * (kk & 3), 16, 1024), id_r, (jb > 0 || kk > 0));
      }
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
    // lane = query now: row tid of O and of the row sums
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float o[64], r[32];
    tmem_ld32(tO + lane_base, o);
    tmem_ld32(tO + lane_base + 32, o + 32);
    tmem_ld32(tR + lane_base, r);
    tmem_ld_wait();
    const int i = ib * kTileRows + tid;
    if (i < g.tq) {
      const float inv = 1.f / (r[0] + g.eps);
      float4* dst = reinterpret_cast<float4*>(out + ((int64_t)n * g.tq + i) * kHeadDim);
#pragma unroll
      for (int c = 0; c < 16; ++c)
        dst[c] = make_float4(o[4 * c] * inv, o[4 * c + 1] * inv, o[4 * c + 2] * inv, o[4 * c + 3] * inv);
      ssum[(int64_t)n * g.tq + i] = r[0];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// ---------------------------------------------------------------- host launchers
#define DILUTION_TC_HAS_MAIN 1
#define DILUTION_TC_HAS_BACKWARD 0

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

// Shared memory is padded so that at most two CTAs share an SM: each holds 256
// TMEM columns and an SM has 512.
constexpr int kTwoPerSm = 100 * 1024;

inline int rowstats(const void* q, const void* k, const Geom& g, float* rmax, float* rden,
                    cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  constexpr int smem = kRowstatsSmem > kTwoPerSm ? kRowstatsSmem : kTwoPerSm;
  if (int rc = set_smem_attr((const void*)rowstats_kernel, smem, err, errlen)) return rc;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  rowstats_kernel<<<(unsigned)(g.n * nqb), 128, smem, st>>>(mq, mk, g, rmax, rden);
  return launch_status("tc rowstats", err, errlen);
}

inline int colsum_scan(const void* q, const void* k, const Geom& g, const float* rmax,
                       const float* rden, const float* carry_base, float* carry, float* total,
                       cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  constexpr int smem = kColsumSmem > kTwoPerSm ? kColsumSmem : kTwoPerSm;
  if (int rc = set_smem_attr((const void*)colsum_scan_kernel, smem, err, errlen)) return rc;
  const int nkb = (g.tk + kTileRows - 1) / kTileRows;
  colsum_scan_kernel<<<(unsigned)(g.n * nkb), 128, smem, st>>>(mq, mk, g, rmax, rden, carry_base, carry,
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
  constexpr int smem = kMainSmem > kTwoPerSm ? kMainSmem : kTwoPerSm;
  static_assert(2 * (smem + 1024) <= 233472, "two CTAs of the main pass must fit one SM");
  if (int rc = set_smem_attr((const void*)forward_main_kernel, smem, err, errlen)) return rc;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  forward_main_kernel<<<(unsigned)(g.n * nqb), 128, smem, st>>>(mq, mk, mv, g, rmax, rden, carry, carry_base,
                                                              out, ssum);
  return launch_status("tc forward_main", err, errlen);
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
