// Row pass with a product: causal-softmax row statistics AND  O = P B  in one sweep,
// bf16 inputs, head_dim 64, on the same tcgen05 / TMEM / TMA building blocks as the other
// tensor-core kernels.
//
//   B = K : O / den * scale = pk = scale * softmax(q k^T) k, the query half of the
//           softmax-Jacobian correction that the reference's K1 saves for the backward
//           (kernels.py:161-188); with pk saved, the backward's correction pass only has the
//           key half left (kernels.py:777-826).
//   B = V : O / den = causal softmax attention, the reference's CausalSelfAttention layers
//           (model.py:96-117: F.scaled_dot_product_attention(q, k, v, is_causal=True)).
//
// grid = n * ceil(tq/128), longest rows first.  S = Q K^T, lane = query, 256 threads: the
// two warpgroups split a tile's 128 key columns and are independent of each other: each keeps,
// per query row, its own reference maximum, its own sum of 2^(z - reference) and its own
// accumulator O_wg [128 queries x 64] in TMEM, fed by P~ = 2^(z - reference) written as bf16
// pairs over the score columns the thread has just consumed (the A operand of O_wg += P~ B, with
// B the MN-major view of the K or V tile).  The two halves are merged once, at the end.
// The reference exponent follows the scores lazily: it is set from the first tile's maximum and
// moves again only when a tile's P~ sum to more than 2^40, and only then is the accumulator
// rescaled (one TMEM round trip per warp).  The common tile therefore takes no maximum and no
// rescaling; bf16 has fp32's exponent range, so P~ of any magnitude below that limit keeps its
// 8 bits, and sums run in fp32.  rmax therefore holds the reference, not the exact row maximum:
// the pair (rmax, rden) is exact only as the log-sum-exp rmax + log2(rden), which is all the
// other passes use.
// TMEM: S 128 columns + 2 x 64 accumulator columns = 256; two CTAs per SM.
#pragma once

#include "tc_kernels.cuh"

namespace dil {
namespace tc {

constexpr float kRefLimit = 1099511627776.f;         // 2^40: a tile whose P~ sum to more moves the reference
template <int MODE> struct RowpassSmem {
  // Q | K[stages] | (V[stages]) | stats [2][128] float4 | barriers + control.  Three stages when
  // K is the only streamed operand; two of K and two of V otherwise, so that two CTAs fit an SM.
  static constexpr int kStages = MODE == 2 ? 2 : 3;
  static constexpr int kTiles = 1 + kStages * (MODE == 2 ? 2 : 1);
  static constexpr int kBytes = kTiles * (int)kTileBytes + 4096 + 256 + 1024;
};

template <int MODE, typename TOut>
__global__ void __launch_bounds__(256, 2) rowpass_product_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, Geom g, float* __restrict__ rmax, float* __restrict__ rden,
    TOut* __restrict__ out) {
  static_assert(MODE == 1 || MODE == 2, "1: B = K (pk); 2: B = V (softmax attention)");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sQ = smem_u32(smem), sK0 = sQ + kTileBytes;
  constexpr int kRowpassStages = RowpassSmem<MODE>::kStages;
  const uint32_t sB0 = MODE == 2 ? sK0 + kRowpassStages * kTileBytes : sK0;
  constexpr int kTiles = RowpassSmem<MODE>::kTiles;
  float4* sStat = reinterpret_cast<float4*>(smem + kTiles * kTileBytes);            // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTiles * kTileBytes + 4096);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t kfull = smem_u32(bars), sdone = smem_u32(bars + 4);
  float* sX = reinterpret_cast<float*>(smem + kTileBytes);    // merge area over the K stages: [2][128][32]

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int n = (int)(blockIdx.x % g.n);
  const int ib = nqb - 1 - (int)(blockIdx.x / g.n);
  const int q0 = g.q_off + ib * kTileRows;
  const int njb = min(g.tk - 1, q0 + kTileRows - 1) / kTileRows + 1;
  constexpr uint32_t kStageTx = (MODE == 2 ? 2u : 1u) * kTileBytes;

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < kRowpassStages; ++i) mbar_init(kfull + 8 * i, 1);
    mbar_init(sdone, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t tS = tmem, tO = tmem + 128 + 64 * wg;      // this warpgroup's accumulator
  {
    uint32_t z[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) z[c] = 0u;
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_st16(tO + lane_base + 16 * c, z);
    tmem_st_wait();
  }
  auto load_stage = [&](int jb) {          // thread 0: K (and V) tile jb into its ring slot
    const int st = jb % kRowpassStages;
    mbar_expect_tx(kfull + 8 * st, kStageTx);
    tma_load_tile(sK0 + kTileBytes * st, &map_k, jb * kTileRows, n, kfull + 8 * st);
    if (MODE == 2) tma_load_tile(sB0 + kTileBytes * st, &map_v, jb * kTileRows, n, kfull + 8 * st);
  };
  if (tid == 0) {
    mbar_expect_tx(kfull, kStageTx + kTileBytes);
    tma_load_tile(sQ, &map_q, ib * kTileRows, n, kfull);
    tma_load_tile(sK0, &map_k, 0, n, kfull);
    if (MODE == 2) tma_load_tile(sB0, &map_v, 0, n, kfull);
    for (int jb = 1; jb < kRowpassStages && jb < njb; ++jb) load_stage(jb);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) {
    mbar_wait(kfull, 0, ctl, &g_status, kErrWaitTma);
    tc_fence_after();
    mma_scores(tS, sQ, sK0, 128);
    mma_commit(sdone);
  }
  __syncwarp();

  float m_ref = -INFINITY, s = 0.f;
  const int ia = q0 + row;
  const uint32_t taddr = tS + lane_base + 64 * wg;
  for (int jb = 0; jb < njb; ++jb) {
    const int st = jb % kRowpassStages;
    // scores of tile jb are ready, and the product of tile jb-1 has completed
    mbar_wait(sdone, jb & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && jb >= 1 && jb - 1 + kRowpassStages < njb)
      load_stage(jb - 1 + kRowpassStages);                          // the slot of tile jb-1 is free
    __syncwarp();
    float v[64];
    tmem_ld32(taddr, v);
    tmem_ld32(taddr + 32, v + 32);
    tmem_ld_wait(v);
    tmem_ld_wait(v + 32);
    uint32_t pw[32];
    float ps = 0.f;
    // P~ = 2^(z - reference) for the thread's 64 scores, two per instruction; their sum in ps
    auto exponentials = [&]() {
      const float mr = m_ref == -INFINITY ? 0.f : m_ref;
      const float2 zs = make_float2(g.zscale, g.zscale), off = make_float2(-mr, -mr);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
      for (int e = 0; e < 64; e += 4) {
        const float2 z0 = fma2(make_float2(v[e], v[e + 1]), zs, off);
        const float2 z1 = fma2(make_float2(v[e + 2], v[e + 3]), zs, off);
        const float2 p0 = make_float2(fast_exp2(z0.x), fast_exp2(z0.y));
        const float2 p1 = make_float2(fast_exp2(z1.x), fast_exp2(z1.y));
        acc0 = add2(acc0, p0);
        acc1 = add2(acc1, p1);
        pw[e >> 1] = pack_bf16(p0.x, p0.y);
        pw[(e >> 1) + 1] = pack_bf16(p1.x, p1.y);
      }
      const float2 acc = add2(acc0, acc1);
      ps = acc.x + acc.y;
    };
    // The common tile takes no maximum at all: the reference stays where it is as long as the
    // tile's sum of P~ stays below 2^40 (then every P~ does, and nothing overflowed).
    // Edge tiles (masking), rows that have not seen a score yet and tiles that outgrow the
    // reference take the slow path: mask, take the tile's maximum, move the reference there,
    // rescale what was accumulated under the old one, and form P~ again.
    const bool edge = (jb * kTileRows + kTileRows - 1 > q0) || ((jb + 1) * kTileRows > g.tk);
    bool slow = edge || __any_sync(0xffffffffu, m_ref == -INFINITY);
    if (!slow) {
      exponentials();
      slow = __any_sync(0xffffffffu, !(ps < kRefLimit));
      if (slow) {                      // rare: the scores are still in TMEM, fetch them again
        tmem_ld32(taddr, v);
        tmem_ld32(taddr + 32, v + 32);
        tmem_ld_wait(v);
        tmem_ld_wait(v + 32);
      }
    }
    if (slow) {
      float cmax = -INFINITY;
      if (edge) {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          const int ja = jb * kTileRows + wg * 64 + e;
          if (ja > ia || ja >= g.tk) v[e] = -INFINITY;
          cmax = fmaxf(cmax, v[e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 64; ++e) cmax = fmaxf(cmax, v[e]);
      }
      const float m_new = fmaxf(m_ref, cmax * g.zscale);
      if (__any_sync(0xffffffffu, m_new != m_ref)) {
        const bool fresh = __all_sync(0xffffffffu, m_ref == -INFINITY);   // nothing accumulated yet
        const float f = m_new == -INFINITY ? 1.f : fast_exp2(m_ref - m_new);
        if (!fresh) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float o[16];
            tmem_ld16(tO + lane_base + 16 * c, o);
            tmem_ld_wait16(o);
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) w[e] = __float_as_uint(o[e] * f);
            tmem_st16(tO + lane_base + 16 * c, w);
          }
        }
        s *= f;
        m_ref = m_new;
      }
      exponentials();
    }
    s += ps;
    // P~ goes over the first 32 of this thread's 64 consumed score columns: keys 2c, 2c+1 of the
    // warpgroup's half in column c
    tmem_st16(taddr, pw);
    tmem_st16(taddr + 16, pw + 16);
    tmem_st_wait();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t id_pv = instr_desc(128, 64, 0, 1);   // A from TMEM (M = queries), B MN-major
      const Desc dB = make_desc(sB0 + kTileBytes * st, kTileBytes, 1024);
#pragma unroll
      for (int w = 0; w < 2; ++w)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)      // 16 keys per instruction: 16 rows of 128 B = 128 units
          mma_ts(tmem + 128 + 64 * w, tS + 64 * w + 8 * kk, dB, 128 * (4 * w + kk), id_pv, 1);
      if (jb + 1 < njb) {
        const int sn = (jb + 1) % kRowpassStages;
        mbar_wait(kfull + 8 * sn, ((jb + 1) / kRowpassStages) & 1, ctl, &g_status, kErrWaitTma);
        tc_fence_after();
        mma_scores(tS, sQ, sK0 + kTileBytes * sn, 128);
      }
      mma_commit(sdone);
    }
    __syncwarp();
  }
  mbar_wait(sdone, njb & 1, ctl, &g_status, kErrWaitMma);
  tc_fence_after();
  // merge the two halves of every row.  Each warpgroup finishes 32 of the 64 output columns:
  // it hands the other 32 of its accumulator, with its statistics, to the other warpgroup.
  auto merge = [&](auto wg_c) {
    constexpr int WG = decltype(wg_c)::value;
    float o[64];
    tmem_ld32(tO + lane_base, o);
    tmem_ld32(tO + lane_base + 32, o + 32);
    tmem_ld_wait(o);
    tmem_ld_wait(o + 32);
    sStat[WG * 128 + row] = make_float4(m_ref, s, 0.f, 0.f);
    float* give = sX + ((1 - WG) * 128 + row) * 32;         // read by the other warpgroup
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      constexpr int base = 32 * (1 - WG);
      reinterpret_cast<float4*>(give)[c ^ (row & 7)] =
          make_float4(o[base + 4 * c], o[base + 4 * c + 1], o[base + 4 * c + 2], o[base + 4 * c + 3]);
    }
    __syncthreads();
    const float4 other = sStat[(1 - WG) * 128 + row];
    const float m = fmaxf(m_ref, other.x);                  // finite: warpgroup 0 always sees key 0
    const float f_own = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m);
    const float f_oth = other.x == -INFINITY ? 0.f : fast_exp2(other.x - m);
    const float den = s * f_own + other.y * f_oth;
    const float inv = (MODE == 1 ? g.scale : 1.f) / den;
    const float a_own = f_own * inv, a_oth = f_oth * inv;
    const float* take = sX + (WG * 128 + row) * 32;
    const int i = ib * kTileRows + row;
    if (i < g.tq) {
      float r[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 x = reinterpret_cast<const float4*>(take)[c ^ (row & 7)];
        r[4 * c] = o[32 * WG + 4 * c] * a_own + x.x * a_oth;
        r[4 * c + 1] = o[32 * WG + 4 * c + 1] * a_own + x.y * a_oth;
        r[4 * c + 2] = o[32 * WG + 4 * c + 2] * a_own + x.z * a_oth;
        r[4 * c + 3] = o[32 * WG + 4 * c + 3] * a_own + x.w * a_oth;
      }
      TOut* dst = out + ((int64_t)n * g.tq + i) * kHeadDim + 32 * WG;
      if (std::is_same<TOut, float>::value) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          reinterpret_cast<float4*>(dst)[c] = make_float4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          reinterpret_cast<uint4*>(dst)[c] =
              make_uint4(pack_bf16(r[8 * c], r[8 * c + 1]), pack_bf16(r[8 * c + 2], r[8 * c + 3]),
                         pack_bf16(r[8 * c + 4], r[8 * c + 5]), pack_bf16(r[8 * c + 6], r[8 * c + 7]));
      }
      if (WG == 0 && rmax != nullptr) {
        // the merged reference, not necessarily the row maximum (it lags behind it by design);
        // every consumer uses the pair only as the log-sum-exp rmax + log2(rden)
        rmax[(int64_t)n * g.tq + i] = m;
        rden[(int64_t)n * g.tq + i] = den;
      }
    }
  };
  if (wg == 0) merge(std::integral_constant<int, 0>{}); else merge(std::integral_constant<int, 1>{});
  drain_if_aborted(ctl);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// Key half of the softmax-Jacobian correction alone (the reference's BC, kernels.py:777-809),
// for a backward that has pk saved:  dk = dk_main - scale * P^T (ghat * Q).
// grid = n * ceil(t/128) key blocks; S^T = K Q^T, lane = key; W = p * ghat goes back into TMEM
// over the consumed score columns as the A operand (M = keys) of dKc += W Q.  Nothing passes
// through shared memory and nothing is reduced across CTAs.
// The pass runs in half-steps of 64 queries: S^T [128 keys x 64 queries] needs 64 TMEM columns, so
// a CTA allocates 128 (S^T 64 + dKc 64) and four CTAs share an SM (32 warps to hide each other's
// MMA round trips, as in the column-sum pass; a version with 128-query steps and two CTAs per SM
// measured 5% slower).  The two warpgroups split a half-step's 64 query columns.
constexpr int kCorrKey64Smem = 3 * kTileBytes + 2048 + 1024 + 256;
static_assert(5 * (kCorrKey64Smem + 1024) > 233472, "at most four CTAs of the half-step correction pass share an SM");

__global__ void __launch_bounds__(256, 4) backward_key_correction64_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, Geom g,
    const float* __restrict__ rmax, const float* __restrict__ rden, const float* __restrict__ ghat,
    const float* __restrict__ dk_main, __nv_bfloat16* __restrict__ dk) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  const uint32_t sK = smem_u32(smem), sQ0 = sK + kTileBytes;
  float2* sStat = reinterpret_cast<float2*>(smem + 3 * kTileBytes);           // [2][128] (lse, ghat)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes + 2048);
  Ctl* ctl = reinterpret_cast<Ctl*>(bars + 8);
  const uint32_t qfull = smem_u32(bars), sdone = smem_u32(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, row = tid & 127;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  const int n = (int)(blockIdx.x % g.n);
  const int jb = (int)(blockIdx.x / g.n);
  const int k0 = jb * kTileRows;
  const int nsteps = nqb - jb, nhalf = 2 * nsteps;
  const int64_t row_base = (int64_t)n * g.tq;

  if (tid == 0) {
    ctl->abort = 0;
    for (int i = 0; i < 3; ++i) mbar_init(qfull + 8 * i, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem), 128);
  if (wg == 1) {
    const int i = jb * kTileRows + row;
    float2 st = make_float2(INFINITY, 0.f);
    if (i < g.tq) st = make_float2(rmax[row_base + i] + log2f(rden[row_base + i]), ghat[row_base + i]);
    sStat[row] = st;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem;
  const uint32_t tS = tmem, tDK = tmem + 64;
  constexpr uint32_t id_s = instr_desc(128, 64, 0, 0), id_kd = instr_desc(128, 64, 0, 1);
  // scores of half-step (stage, odd): queries 64*odd.. of the Q tile in that stage (K-major: a
  // row is 128 B = 8 units)
  auto issue_scores = [&](int stage, int odd) {
    const Desc dKk = make_desc(sK, 16, 1024), dQk = make_desc(sQ0 + kTileBytes * stage, 16, 1024);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) mma_ss(tS, dKk, 2 * kk, dQk, 512 * odd + 2 * kk, id_s, kk > 0);
  };

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
    issue_scores(0, 0);
    mma_commit(sdone);
  }
  __syncwarp();

  const int ja = k0 + row;
  const bool dead = ja >= g.tk;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t tcol = tS + lane_base + 32 * wg;
  for (int h = 0; h < nhalf; ++h) {
    const int t = h >> 1, odd = h & 1, ib = jb + t, b = t & 1;
    float nx_max = INFINITY, nx_den = 1.f, nx_gh = 0.f;
    const bool fetch = odd == 0 && wg == 1 && t + 1 < nsteps;
    if (fetch && (ib + 1) * kTileRows + row < g.tq) {
      const int64_t i = row_base + (ib + 1) * kTileRows + row;
      nx_max = rmax[i];
      nx_den = rden[i];
      nx_gh = ghat[i];
    }
    // scores of this half-step are ready; every earlier dKc product has completed
    mbar_wait(sdone, h & 1, ctl, &g_status, kErrWaitMma);
    tc_fence_after();
    if (tid == 0 && odd == 0 && t >= 1 && t + 1 < nsteps) {      // the Q stage of step t-1 is free
      mbar_expect_tx(qfull + 8 * (b ^ 1), kTileBytes);
      tma_load_tile(sQ0 + kTileBytes * (b ^ 1), &map_q, (ib + 1) * kTileRows, n, qfull + 8 * (b ^ 1));
    }
    __syncwarp();
    const int i0 = ib * kTileRows + 64 * odd + 32 * wg;           // first query of this thread's 32
    const bool masked = dead || t == 0;
    const float4* St4 = reinterpret_cast<const float4*>(sStat + b * 128 + 64 * odd + 32 * wg);
    float vs[32];
    uint32_t wt[16];
    tmem_ld32(tcol, vs);
    tmem_ld_wait(vs);
    auto tile = [&](auto mask_tag) {
      constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
      for (int e2 = 0; e2 < 16; ++e2) {
        const float4 st = St4[e2];                                // (lse, ghat) of two queries
        float p0 = fast_exp2(fmaf(vs[2 * e2], g.zscale, -st.x));
        float p1 = fast_exp2(fmaf(vs[2 * e2 + 1], g.zscale, -st.z));
        if (MASK) {
          if (dead || ja > i0 + 2 * e2) p0 = 0.f;
          if (dead || ja > i0 + 2 * e2 + 1) p1 = 0.f;
        }
        wt[e2] = pack_bf16(p0 * st.y, p1 * st.w);
      }
    };
    if (masked) tile(std::true_type{}); else tile(std::false_type{});
    tmem_st16(tcol, wt);            // W over the first 16 of the 32 consumed columns
    if (fetch) sStat[(b ^ 1) * 128 + row] = make_float2(nx_max + log2f(nx_den), nx_gh);
    tmem_st_wait();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const Desc dQm = make_desc(sQ0 + kTileBytes * b, kTileBytes, 1024);
#pragma unroll
      for (int kq = 0; kq < 4; ++kq)        // 16 queries per instruction: 16 rows of 128 B = 128 units
        mma_ts(tDK, tS + 32 * (kq >> 1) + 8 * (kq & 1), dQm, 128 * (4 * odd + kq), id_kd, (h > 0 || kq > 0));
      if (h + 1 < nhalf) {
        if (odd) {                          // the next half-step opens step t+1
          mbar_wait(qfull + 8 * (b ^ 1), ((t + 1) >> 1) & 1, ctl, &g_status, kErrWaitTma);
          tc_fence_after();
          issue_scores(b ^ 1, 0);
        } else {
          issue_scores(b, 1);
        }
      }
      mma_commit(sdone);
    }
    __syncwarp();
  }
  mbar_wait(sdone, nhalf & 1, ctl, &g_status, kErrWaitMma);
  tc_fence_after();
  {
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
  if (warp == 0) tmem_free(tmem, 128);
}

// dq = bf16(dq_main - ghat * pk): the query half of the correction from the saved pk
// (the reference's dq epilogue, kernels.py:814-826; pk already carries the scale).
__global__ void dq_from_pk_kernel(const float* __restrict__ dq_main, const float* __restrict__ pk,
                                  const float* __restrict__ ghat, __nv_bfloat16* __restrict__ dq, int64_t n4) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 a = reinterpret_cast<const float4*>(dq_main)[i];
  const float4 b = reinterpret_cast<const float4*>(pk)[i];
  const float gh = ghat[i / (kHeadDim / 4)];
  reinterpret_cast<uint2*>(dq)[i] = make_uint2(pack_bf16(fmaf(-gh, b.x, a.x), fmaf(-gh, b.y, a.y)),
                                               pack_bf16(fmaf(-gh, b.z, a.z), fmaf(-gh, b.w, a.w)));
}

// ---------------------------------------------------------------- host launchers
// Pass 1 with the saved query correction: rmax, rden and pk = scale * softmax(q k^T) k.
inline int rowstats_pk(const void* q, const void* k, const Geom& g, float* rmax, float* rden, float* pk,
                       cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  auto kern = rowpass_product_kernel<1, float>;
  constexpr int smem = RowpassSmem<1>::kBytes > kTwoPerSm ? RowpassSmem<1>::kBytes : kTwoPerSm;
  if (int rc = set_smem_attr((const void*)kern, smem, err, errlen)) return rc;
  kern<<<(unsigned)(g.n * nqb), 256, smem, st>>>(mq, mk, mk, g, rmax, rden, pk);
  return launch_status("tc rowstats_pk", err, errlen);
}

// Causal softmax attention forward: out = softmax(q k^T * scale) v in bf16; rmax / rden
// (optional) as pass 1 writes them.
inline int softmax_forward(const void* q, const void* k, const void* v, const Geom& g, float* rmax,
                           float* rden, void* out, cudaStream_t st, char* err, size_t errlen) {
  CUtensorMap mq, mk, mv;
  if (int rc = make_map(&mq, q, g.n, g.tq, err, errlen)) return rc;
  if (int rc = make_map(&mk, k, g.n, g.tk, err, errlen)) return rc;
  if (int rc = make_map(&mv, v, g.n, g.tk, err, errlen)) return rc;
  auto kern = rowpass_product_kernel<2, __nv_bfloat16>;
  constexpr int smem = RowpassSmem<2>::kBytes;
  static_assert(2 * (smem + 1024) <= 233472 && 3 * (smem + 1024) > 233472, "two CTAs of the softmax pass fit one SM");
  if (int rc = set_smem_attr((const void*)kern, smem, err, errlen)) return rc;
  const int nqb = (g.tq + kTileRows - 1) / kTileRows;
  kern<<<(unsigned)(g.n * nqb), 256, smem, st>>>(mq, mk, mv, g, rmax, rden, (__nv_bfloat16*)out);
  return launch_status("tc softmax_forward", err, errlen);
}

// The tail of the backward when pk was saved by the forward: key correction + dq epilogue.
inline int backward_tail_with_pk(const CUtensorMap& mq, const CUtensorMap& mk, const Geom& g, const float* rmax,
                                 const float* rden, const float* ghat, const float* dk_main,
                                 const float* dq_main, const float* pk, void* dq, void* dk, cudaStream_t st,
                                 char* err, size_t errlen, void (*mark)(const char*, cudaStream_t, int)) {
  const int nkb = (g.tk + kTileRows - 1) / kTileRows;
  constexpr int smem = kCorrKey64Smem;
  if (int rc = set_smem_attr((const void*)backward_key_correction64_kernel, smem, err, errlen)) return rc;
  mark("tc_backward_key_correction", st, 0);
  backward_key_correction64_kernel<<<(unsigned)(g.n * nkb), 256, smem, st>>>(mq, mk, g, rmax, rden, ghat,
                                                                           dk_main, (__nv_bfloat16*)dk);
  mark("tc_backward_key_correction", st, 1);
  if (int rc = launch_status("tc backward_key_correction", err, errlen)) return rc;
  const int64_t n4 = g.n * g.tq * kHeadDim / 4;
  mark("tc_dq_from_pk", st, 0);
  dq_from_pk_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(dq_main, pk, ghat, (__nv_bfloat16*)dq, n4);
  mark("tc_dq_from_pk", st, 1);
  return launch_status("tc dq_from_pk", err, errlen);
}

}  // namespace tc
}  // namespace dil
