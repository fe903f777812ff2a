// Key-stationary training forward on the tensor cores: passes 2 and 3 in one sweep
// (the reference's training forward, _dilution_key_forward + _dilution_normalize,
// kernels.py:200-248, does the same on its side of the fence).
//
// A CTA owns 256 keys (two 128-key halves, one per compute warpgroup; lane = key) and walks
// the query blocks that can see them in causal order.  The demand of a key is ONE register
// for the whole sweep, so no checkpoint is read; the checkpoints the backward needs
// (every 32 query rows) and the demand totals are stored on the way.  Per 128-query step:
//   S^T  = K Q^T            two 64-query halves per key half (so that the next step's scores run
//                           under this step's arithmetic): 16 MMAs of N = 64
//   p, den += p, share      exactly the arithmetic of forward_main_kernel
//   O | rs = share [V|1]    M = 128 queries, K = 256 keys, N = 80: 16 MMAs, a FRESH tile per step
// and the O | rs tile is added to `out` / `ssum` in global memory: a third warpgroup
// (lane = query) moves it from TMEM to a swizzled fp32 staging tile and issues two TMA
// tensor reductions, the row sums go by atomics.  `out` and `ssum` therefore start at zero and
// a small kernel divides at the end.  One exponential and one QK^T sweep per score less than
// column-sum pass + query-stationary main pass.
//
// 384 threads, one CTA per SM (TMEM: S^T 256 columns, two O | rs tiles of 80).  Thread 256
// issues every TMA copy and MMA.  Every wait is bounded.
#pragma once

#include "tc_kernels.cuh"

namespace dil {
namespace tc {

constexpr int kFusedThreads = 384;
constexpr int kFusedKeys = 2 * kTileRows;
// K[2] V[2] ones Q[2] shares[4] staging[2] + lse + barriers
constexpr int kFusedSmem = 13 * kTileBytes + 2048 + 256 + 1024;

__global__ void __launch_bounds__(kFusedThreads, 1) forward_fused_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_out, Geom g,
    const float* __restrict__ rmax, const float* __restrict__ rden, float* __restrict__ carry,
    float* __restrict__ total, float* __restrict__ ssum) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem);                       // [2] K-major
  const uint32_t sV = sK + 2 * kTileBytes;                  // [2], then the ones tile: [V | 1] MN-major
  const uint32_t sOnes = sK + 4 * kTileBytes;
  uint8_t* ones_ptr = smem + 4 * kTileBytes;
  const uint32_t sQ = sK + 5 * kTileBytes;                  // [2] stages
  const uint32_t sSh = sK + 7 * kTileBytes;                 // [2 key halves][2 query halves] MN-major shares
  const uint32_t sStage = sK + 11 * kTileBytes;             // 32 KB fp32 O tile for the reductions
  float* sL = reinterpret_cast<float*>(smem + 13 * kTileBytes);            // [2 warpgroups][2][128] lse of a step's queries
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 13 * kTileBytes + 2048);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 16);
  const uint32_t kfull = smem_u32(bars), qfull = smem_u32(bars + 1);       // qfull[2]
  const uint32_t sdone = smem_u32(bars + 3), sfree = smem_u32(bars + 5);   // [2] each: query halves
  const uint32_t shready = smem_u32(bars + 7), odone = smem_u32(bars + 8); // odone[2]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int ncb = (g.tq + 31) / 32;
  const int n = (int)(blockIdx.x % g.n);
  const int kb = (int)(blockIdx.x / g.n);
  const int k0 = kb * kFusedKeys;
  const int ib0 = 2 * kb;                       // first query block that sees these keys
  const int nsteps = nqb - ib0;                 // >= 1
  const int64_t row_base = (int64_t)n * g.tq;

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 5; ++i) mbar_init(kfull + 8 * i, 1);        // kfull, qfull[2], sdone[2]
    mbar_init(sfree, 8);
    mbar_init(sfree + 8, 8);
    mbar_init(shready, 8);
    mbar_init(odone, 1);
    mbar_init(odone + 8, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 512);
  if (wg == 1) {
#pragma unroll
    for (int c = 0; c < 8; ++c)
      reinterpret_cast<uint4*>(ones_ptr)[row * 8 + c] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // only now: the barriers these copies complete on were initialised by thread 0, and nothing but
  // the CTA-wide barrier above orders that against another warp's use of them
  if (tid == 256) {
    mbar_expect_tx(kfull, 4 * kTileBytes);
    tma_load_tile(sK, &map_k, k0, n, kfull);
    tma_load_tile(sK + kTileBytes, &map_k, k0 + kTileRows, n, kfull);
    tma_load_tile(sV, &map_v, k0, n, kfull);
    tma_load_tile(sV + kTileBytes, &map_v, k0 + kTileRows, n, kfull);
    for (int s = 0; s < 2 && s < nsteps; ++s) {
      mbar_expect_tx(qfull + 8 * s, kTileBytes);
      tma_load_tile(sQ + kTileBytes * s, &map_q, (ib0 + s) * kTileRows, n, qfull + 8 * s);
    }
  }
  __syncwarp();
  const uint32_t tmem = ctl->tmem;
  const uint32_t tS = tmem, tO = tmem + 256;              // O | rs tile b at tO + 128 b
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

  if (wg == 2) {
    // ------------------------------------------------------------ issue, and the O read-out
    constexpr uint32_t id_s = instr_desc(128, 64, 0, 0);     // scores: both operands K-major
    constexpr uint32_t id_o = instr_desc(128, 80, 1, 1);     // O | rs: A and B MN-major
    const Desc dK0 = make_desc(sK, 16, 1024), dK1 = make_desc(sK + kTileBytes, 16, 1024);
    const Desc dQ = make_desc(sQ, 16, 1024);
    const Desc dSh0 = make_desc(sSh, kTileBytes, 1024), dSh1 = make_desc(sSh + 2 * kTileBytes, kTileBytes, 1024);
    const Desc dV0 = make_desc(sV, sOnes - sV, 1024);
    const Desc dV1 = make_desc(sV + kTileBytes, sOnes - (sV + kTileBytes), 1024);
    // scores of query half `a` of the step whose Q tile sits in stage `st`, both key halves
    auto issue_scores = [&](int a, int st) {
      const uint32_t off = st * 1024 + a * 512;              // 16-byte units: a tile is 1024, 64 rows 512
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) mma_ss(tS + 64 * a, dK0, 2 * kk, dQ, off + 2 * kk, id_s, kk > 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) mma_ss(tS + 128 + 64 * a, dK1, 2 * kk, dQ, off + 2 * kk, id_s, kk > 0);
    };
    // O | rs of step s-1 from TMEM to global memory: lane = query
    auto read_out = [&](int s1) {
      const int b = s1 & 1;
      if (lane == 0) mbar_wait(odone + 8 * b, (s1 >> 1) & 1, ctl, &g_status, kErrWaitMma);
      __syncwarp();
      tc_fence_after();
      if (tid == 256) tma_wait_read_all();                   // the previous reductions have read the staging tile
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const uint32_t stage = sStage + row * 128;
      const uint32_t tOb = tO + 128 * b + lane_base;
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {                          // 16 columns at a time
        float o[16];
        tmem_ld16(tOb + 16 * j, o);
        tmem_ld_wait16(o);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage + kTileBytes * (j >> 1) + (((4 * (j & 1) + c) ^ (row & 7)) << 4)),
                       "f"(o[4 * c]), "f"(o[4 * c + 1]), "f"(o[4 * c + 2]), "f"(o[4 * c + 3])
                       : "memory");
      }
      float rs;
      tmem_ld1(tOb + 64, &rs);
      tmem_ld_wait();
      fence_async_smem();
      tc_fence_before();
      asm volatile("bar.sync 2, 128;" ::: "memory");         // every warp has read the tile: its buffer is free
      const int ibq = ib0 + s1;
      if (tid == 256) {
        tc_fence_after();
        tma_reduce_add_tile(&map_out, sStage, 0, ibq * kTileRows, n);
        tma_reduce_add_tile(&map_out, sStage + kTileBytes, 32, ibq * kTileRows, n);
      }
      const int i = ibq * kTileRows + row;
      if (i < g.tq) atomicAdd(ssum + row_base + i, rs);
    };
    if (tid == 256) {
      mbar_wait(kfull, 0, ctl, &g_status, kErrWaitTma);
      mbar_wait(qfull, 0, ctl, &g_status, kErrWaitTma);
      tc_fence_after();
      issue_scores(0, 0);
      mma_commit(sdone);
      issue_scores(1, 0);
      mma_commit(sdone + 8);
    }
    __syncwarp();
    for (int s = 0; s < nsteps; ++s) {
      if (s >= 1) read_out(s - 1);
      if (tid == 256) {
        const int b = s & 1;
        if (s + 1 < nsteps) {
          // scores of step s+1, each query half as soon as the compute warps have taken that
          // half of step s out of TMEM
          mbar_wait(qfull + 8 * (b ^ 1), ((s + 1) >> 1) & 1, ctl, &g_status, kErrWaitTma);
          mbar_wait(sfree, s & 1, ctl, &g_status, kErrWaitTile);
          tc_fence_after();
          issue_scores(0, b ^ 1);
          mma_commit(sdone);
          mbar_wait(sfree + 8, s & 1, ctl, &g_status, kErrWaitTile);
          tc_fence_after();
          issue_scores(1, b ^ 1);
          mma_commit(sdone + 8);
        }
        mbar_wait(shready, s & 1, ctl, &g_status, kErrWaitTile);
        tc_fence_after();
        const uint32_t tOb = tO + 128 * b;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss(tOb, dSh0, 128 * kk, dV0, 128 * kk, id_o, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_ss(tOb, dSh1, 128 * kk, dV1, 128 * kk, id_o, 1);
        mma_commit(odone + 8 * b);
        if (s + 2 < nsteps) {
          // the scores of step s are complete (its shares exist), so its Q stage takes step s+2
          mbar_expect_tx(qfull + 8 * b, kTileBytes);
          tma_load_tile(sQ + kTileBytes * b, &map_q, (ib0 + s + 2) * kTileRows, n, qfull + 8 * b);
        }
      }
      __syncwarp();
    }
    read_out(nsteps - 1);
    if (tid == 256) tma_wait_read_all();
  } else {
    // ------------------------------------------------------------ the compute warps: lane = key
    // Each warpgroup keeps its own copy of a step's lse values, so the two only meet through the
    // issuing thread's barriers.
    const int ja = k0 + wg * kTileRows + row;
    const bool dead = ja >= g.tk;
    const uint32_t tSw = tS + 128 * wg + lane_base;
    const uint32_t sShw = sSh + 2 * kTileBytes * wg;
    float* sLw = sL + 256 * wg;                              // [2][128]
    float den = g.eps;                                       // committed + eps, for the whole sweep
    sLw[row] = load_lse(rmax, rden, row_base, ib0 * kTileRows + row, g.tq);
    if (wg == 0) asm volatile("bar.sync 3, 128;" ::: "memory"); else asm volatile("bar.sync 4, 128;" ::: "memory");
    for (int s = 0; s < nsteps; ++s) {
      const int ib = ib0 + s, b = s & 1;
      float lse_next = INFINITY;
      if (s + 1 < nsteps) lse_next = load_lse(rmax, rden, row_base, (ib + 1) * kTileRows + row, g.tq);
      // The step's four 32-query chunks (query half a = IDX / 2).  The TMEM load of the next chunk
      // is issued before this chunk's arithmetic; the shares of the first two chunks wait in
      // registers until the O MMAs of the previous step have read the share tile.
      float v0[32], v1[32];
      uint32_t pk0[16], pk1[16];
      mbar_wait(sdone, s & 1, ctl, &g_status, kErrWaitMma);
      tc_fence_after();
      tmem_ld32(tSw, v0);
      auto arith = [&](const float* v, uint32_t* packed, int q0) {
        const int rb = q0 >> 5;                              // checkpoint in front of the chunk's first query
        if (!dead && rb < ncb) carry[((int64_t)n * ncb + rb) * g.tk + ja] = den - g.eps;
        const float4* L4 = reinterpret_cast<const float4*>(sLw + 128 * b + (q0 - ib * kTileRows));
        const bool masked = dead || (k0 + wg * kTileRows + kTileRows - 1 > q0);
        auto chunk = [&](auto mask_tag) {
          constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
          for (int e4 = 0; e4 < 8; ++e4) {
            const float4 l = L4[e4];
            const float ls[4] = {l.x, l.y, l.z, l.w};
            float sh[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              // two special-function ops per score on two warps per scheduler: every fourth
              // exponential is a degree-4 polynomial on the FMA pipe instead (7.30 -> 7.08 ms)
              const float z = fmaf(v[e4 * 4 + u], g.zscale, -ls[u]);
              float p = u == 3 ? poly_exp2<4>(z) : fast_exp2(z);
              if (MASK && (dead || ja > q0 + e4 * 4 + u)) p = 0.f;
              den += p;
              sh[u] = p * fast_rcp(den);
            }
            packed[e4 * 2] = pack_bf16(sh[0], sh[1]);
            packed[e4 * 2 + 1] = pack_bf16(sh[2], sh[3]);
          }
        };
        if (masked) chunk(std::true_type{}); else chunk(std::false_type{});
      };
      auto store = [&](const uint32_t* packed, int ql) {      // ql: first query of the chunk within the step
#pragma unroll
        for (int e8 = 0; e8 < 4; ++e8) {
          const uint32_t dst = sShw + share_chunk_offset(row, ql + e8 * 8);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[4 * e8]),
                       "r"(packed[4 * e8 + 1]), "r"(packed[4 * e8 + 2]), "r"(packed[4 * e8 + 3])
                       : "memory");
        }
      };
      auto release = [&](int a) {                            // this half of the scores is out of TMEM
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sfree + 8 * a);
      };
      const int qs = ib * kTileRows;
      // chunk 0
      tmem_ld_wait(v0);
      tmem_ld32(tSw + 32, v1);
      arith(v0, pk0, qs);
      // chunk 1
      tmem_ld_wait(v1);
      release(0);
      mbar_wait(sdone + 8, s & 1, ctl, &g_status, kErrWaitMma);
      tc_fence_after();
      tmem_ld32(tSw + 64, v0);
      arith(v1, pk1, qs + 32);
      if (s >= 1) mbar_wait(odone + 8 * (b ^ 1), ((s - 1) >> 1) & 1, ctl, &g_status, kErrWaitMma);
      store(pk0, 0);
      store(pk1, 32);
      // chunk 2
      tmem_ld_wait(v0);
      tmem_ld32(tSw + 96, v1);
      arith(v0, pk0, qs + 64);
      store(pk0, 64);
      // chunk 3
      tmem_ld_wait(v1);
      release(1);
      arith(v1, pk1, qs + 96);
      store(pk1, 96);
      if (s + 1 < nsteps) sLw[128 * (b ^ 1) + row] = lse_next;
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(shready);
      // the next step's lse is visible to the warpgroup
      if (wg == 0) asm volatile("bar.sync 3, 128;" ::: "memory"); else asm volatile("bar.sync 4, 128;" ::: "memory");
    }
    if (!dead) total[(int64_t)n * g.tk + ja] = den - g.eps;
  }
  drain_if_aborted(ctl);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 512);
}

// out = O / (rs + eps) in place, four columns per thread (grid over n*t*16 float4).
__global__ void normalize_out_kernel(float* __restrict__ out, const float* __restrict__ ssum, float eps,
                                     int64_t n4) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float inv = 1.f / (ssum[i >> 4] + eps);
  float4 x = reinterpret_cast<float4*>(out)[i];
  x.x *= inv; x.y *= inv; x.z *= inv; x.w *= inv;
  reinterpret_cast<float4*>(out)[i] = x;
}

// Passes 2 and 3 of a training forward (q_off = 0, tq = tk, checkpoints every 32 rows) in one
// key-stationary sweep.  carry: (n, ceil(t/32), t); total: (n, t); out: (n, t, 64) fp32; ssum: (n, t).
inline int forward_fused(const void* q, const void* k, const void* v, const Geom& g, const float* rmax,
                         const float* rden, float* carry, float* total, float* out, float* ssum,
                         cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk, mv, mo;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  if (int rc = make_map(&mv, v, g.n, g.tk, err, errlen)) return rc;
  if (int rc = make_map_f32(&mo, out, g.n, g.tq, err, errlen)) return rc;
  constexpr int smem = kFusedSmem;
  static_assert(smem <= 232448, "the fused forward pass fits one SM's shared memory");
  if (int rc = set_smem_attr((const void*)forward_fused_kernel, smem, err, errlen)) return rc;
  const int64_t rows = g.n * g.tq;
  cudaMemsetAsync(out, 0, sizeof(float) * (size_t)rows * kHeadDim, st);
  cudaMemsetAsync(ssum, 0, sizeof(float) * (size_t)rows, st);
  const int nsb = (g.tk + kFusedKeys - 1) / kFusedKeys;
  forward_fused_kernel<<<(unsigned)(g.n * nsb), kFusedThreads, smem, st>>>(mq, mk, mv, mo, g, rmax, rden, carry,
                                                                         total, ssum);
  return launch_status("tc forward_fused", err, errlen);
}

// The division that ends the fused forward: out = O / (rs + eps), in place.
inline int normalize_out(const Geom& g, float* out, const float* ssum, cudaStream_t st, char* err, size_t errlen) {
  const int64_t n4 = g.n * g.tq * kHeadDim / 4;
  normalize_out_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(out, ssum, g.eps, n4);
  return launch_status("tc normalize_out", err, errlen);
}

}  // namespace tc
}  // namespace dil
