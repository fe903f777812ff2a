// extern "C" entry points of libdilution_b200.so: argument validation, kernel
// selection and launches.  Declarations and the reference interface each entry
// point replaces are in include/dilution_b200.h.

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/dilution_b200.h"
#include "decode_kernels.cuh"
#include "layer_kernels.cuh"
#include "simt_kernels.cuh"
#if __has_include("tc_kernels.cuh")
#include "tc_kernels.cuh"
#include "tc_rowpass_kernels.cuh"
#include "tc_fused_forward.cuh"
#define DILUTION_TENSOR_PATH 1
#endif

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(DILUTION_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return DILUTION_OK;
}

// Launch accounting: a global count of kernel launches and, when enabled, a pair
// of CUDA events around every launch on the launching stream.
struct ProfRecord {
  const char* name;
  cudaEvent_t a, b;
};
std::mutex g_prof_mu;
bool g_prof_on = false;
std::vector<ProfRecord> g_prof;
unsigned long long g_launches = 0;

struct Prof {
  cudaStream_t st;
  ProfRecord rec;
  bool on;
  Prof(const char* name, cudaStream_t s, bool timing = true) : st(s), on(false) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    ++g_launches;
    if (!g_prof_on || !timing) return;
    rec.name = name;
    if (cudaEventCreate(&rec.a) != cudaSuccess) return;
    if (cudaEventCreate(&rec.b) != cudaSuccess) { cudaEventDestroy(rec.a); return; }
    on = true;
    cudaEventRecord(rec.a, st);
  }
  ~Prof() {
    if (!on) return;
    cudaEventRecord(rec.b, st);
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof.push_back(rec);
  }
};

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return DILUTION_OK;
  const cudaError_t e =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess)
    return fail(DILUTION_ERR_CUDA, "cudaFuncSetAttribute(%zu): %s", bytes, cudaGetErrorString(e));
  return DILUTION_OK;
}

bool valid_d(int d) { return d == 16 || d == 32 || d == 64 || d == 128; }

int check_common(const char* fn, int dtype, int precision, int64_t n, int64_t tq, int64_t tk,
                 int64_t q_offset, int d) {
  if (dtype != DILUTION_F32 && dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "%s: dtype must be DILUTION_F32 or DILUTION_BF16", fn);
  if (precision < DILUTION_PREC_IEEE || precision > DILUTION_PREC_BF16)
    return fail(DILUTION_ERR_ARG, "%s: precision must be one of ieee, tf32, bf16", fn);
  if (!valid_d(d))
    return fail(DILUTION_ERR_UNSUPPORTED, "%s: head_dim %d not in {16, 32, 64, 128}", fn, d);
  if (n < 1 || tq < 1 || tk < 1 || q_offset < 0)
    return fail(DILUTION_ERR_ARG, "%s: sizes must be positive (n=%lld tq=%lld tk=%lld q_offset=%lld)",
                fn, (long long)n, (long long)tq, (long long)tk, (long long)q_offset);
  if (tq > (1 << 30) || tk > (1 << 30) || q_offset > (1 << 30))
    return fail(DILUTION_ERR_ARG, "%s: sequence length beyond 2^30", fn);
  const int64_t blocks = (tq > tk ? tq : tk) / 64 + 1;
  if (n * blocks >= (int64_t)1 << 31)
    return fail(DILUTION_ERR_ARG, "%s: n * blocks exceeds the grid limit", fn);
  return DILUTION_OK;
}

// Checkpoint spacings: the tensor-core kernels take 32 or 64 query rows; the fp32 kernels 32.
int check_carry_rows(const char* fn, int dtype, int precision, int d, int64_t q_offset, int carry_rows);

dil::Geom make_geom(int64_t n, int64_t tq, int64_t tk, int64_t q_offset, float scale, float eps,
                    int carry_rows = dil::kCarryRows, int bid = dil::kBidSoftmax,
                    int share = dil::kShareInclusive, float shift = 1.f) {
  dil::Geom g;
  g.carry_rows = carry_rows;
  g.bid = dil::bid_form(bid);
  g.share = share;
  g.normalised = bid == dil::kBidSoftmax || dil::row_sum_bid(bid);
  g.lshift = (bid == dil::kBidExpshift || bid == dil::kBidSigshift) ? log2f(shift) : 0.f;
  g.ghat_pass = 0;
  g.n = n;
  g.tq = (int)tq;
  g.tk = (int)tk;
  g.q_off = (int)q_offset;
  g.scale = scale;
  g.zscale = scale * dil::kLog2e;
  g.eps = eps;
  return g;
}

#define DIL_DISPATCH_D(d, ...)                         \
  switch (d) {                                         \
    case 16: { constexpr int D = 16; __VA_ARGS__; break; }   \
    case 32: { constexpr int D = 32; __VA_ARGS__; break; }   \
    case 64: { constexpr int D = 64; __VA_ARGS__; break; }   \
    default: { constexpr int D = 128; __VA_ARGS__; break; }  \
  }

#define DIL_DISPATCH(dtype, d, ...)                                        \
  if ((dtype) == DILUTION_F32) { using T = float; DIL_DISPATCH_D(d, __VA_ARGS__) } \
  else { using T = __nv_bfloat16; DIL_DISPATCH_D(d, __VA_ARGS__) }

// ---- fp32-tile launches ------------------------------------------------------
// MMA = false: fp32 FMAs (precision IEEE); MMA = true: tf32 tensor-core products with fp32
// accumulation (precision TF32 on fp32 tensors; every bf16-tensor case the tcgen05 kernels do
// not take).
#define DIL_DISPATCH_MMA(precision, ...)                          \
  if ((precision) == DILUTION_PREC_IEEE) { constexpr bool MMA = false; __VA_ARGS__; } \
  else { constexpr bool MMA = true; __VA_ARGS__; }

template <typename T, int D, bool MMA>
int launch_rowstats(const void* q, const void* k, const dil::Geom& g, float* rmax, float* rden,
                    cudaStream_t st) {
  using namespace dil::simt;
  auto kern = rowstats_kernel<T, D, MMA>;
  if (int rc = set_smem(kern, smem_rowstats<D>())) return rc;
  const int nqb = (g.tq + TS - 1) / TS;
  {
    Prof prof("simt_rowstats", st);
    kern<<<(unsigned)(g.n * nqb), NT, smem_rowstats<D>(), st>>>((const T*)q, (const T*)k, g, rmax, rden);
  }
  return check_launch("rowstats");
}

template <typename T, int D, bool MMA>
int launch_colsum(const void* q, const void* k, const dil::Geom& g, const float* rmax,
                  const float* rden, const float* base, float* carry, float* total,
                  cudaStream_t st) {
  using namespace dil::simt;
  auto kern = colsum_scan_kernel<T, D, MMA>;
  if (int rc = set_smem(kern, smem_colsum<D>())) return rc;
  const int nkb = (g.tk + TS - 1) / TS;
  {
    Prof prof("simt_colsum_scan", st);
    kern<<<(unsigned)(g.n * nkb), NT, smem_colsum<D>(), st>>>((const T*)q, (const T*)k, g, rmax, rden,
                                                               base, carry, total);
  }
  return check_launch("colsum_scan");
}

template <typename T, int D, bool MMA>
int launch_main(const void* q, const void* k, const void* v, const dil::Geom& g, const float* rmax,
                const float* rden, const float* carry, const float* base, float* out, float* ssum,
                float* pk, cudaStream_t st) {
  using namespace dil::simt;
  const int nqb = (g.tq + TS - 1) / TS;
  const unsigned grid = (unsigned)(g.n * nqb);
  Prof prof("simt_forward_main", st);
  if (pk) {
    auto kern = main_kernel<T, D, true, MMA>;
    if (int rc = set_smem(kern, smem_main<D>())) return rc;
    kern<<<grid, NT, smem_main<D>(), st>>>((const T*)q, (const T*)k, (const T*)v, g, rmax, rden,
                                            carry, base, out, ssum, pk);
  } else {
    auto kern = main_kernel<T, D, false, MMA>;
    if (int rc = set_smem(kern, smem_main<D>())) return rc;
    kern<<<grid, NT, smem_main<D>(), st>>>((const T*)q, (const T*)k, (const T*)v, g, rmax, rden,
                                            carry, base, out, ssum, nullptr);
  }
  return check_launch("forward_main");
}

struct BwdScratch {
  float *dq_main, *dk_main, *ghat, *dbar;
  void* dop;   // (n, t, d) bf16: dout pre-scaled by 1/(ssum+eps), tensor-core path only
};
BwdScratch carve_bwd(void* scratch, int64_t n, int64_t t, int d) {
  BwdScratch s;
  // dop is a TMA source (16-byte aligned start): it comes before the two (n, t) vectors,
  // whose length n * t may be odd
  s.dq_main = (float*)scratch;
  s.dk_main = s.dq_main + n * t * d;
  s.dop = s.dk_main + n * t * d;
  s.ghat = (float*)((char*)s.dop + 2 * (size_t)(n * t * d));
  s.dbar = s.ghat + n * t;
  return s;
}

// Start/stop a named timing scope from code that cannot see Prof.
thread_local Prof* g_mark = nullptr;
void mark_scope(const char* name, cudaStream_t st, int phase) {
  if (phase == 0) {
    g_mark = new Prof(name, st);
  } else if (g_mark != nullptr) {
    delete g_mark;
    g_mark = nullptr;
  }
}

template <typename T, int D, bool MMA>
int launch_backward(const void* q, const void* k, const void* v, const dil::Geom& g,
                    const float* dout, const float* out, const float* rmax, const float* rden,
                    const float* carry, const float* ssum, const float* pk, const BwdScratch& s,
                    void* dq, void* dk, void* dv, cudaStream_t st) {
  using namespace dil::simt;
  const int64_t rows = g.n * g.tq;
  {
    Prof prof("dbar", st);
    dbar_kernel<D><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(dout, out, rows, s.dbar, s.ghat, s.dq_main);
  }
  if (int rc = check_launch("dbar")) return rc;
  const int nkb = (g.tk + TS - 1) / TS;
  const unsigned grid = (unsigned)(g.n * nkb);
  // an f(a) / rowsum(f) bid under a share step: its Jacobian factor 1 / (row mass) is unbounded, so
  // ghat is found first and subtracted before the factor multiplies (two sweeps, as the reference's
  // B1-B2 then B4, kernels_bid.py:513-612, 659-728); everything else: one sweep, correction afterwards
  const bool two_sweeps = dil::row_sum_bid(g.bid) && g.share != dil::kShareNone;
  for (int sweep = two_sweeps ? 1 : 0; sweep <= (two_sweeps ? 2 : 0); ++sweep) {
    dil::Geom gs = g;
    gs.ghat_pass = sweep;
    auto kern = backward_main_kernel<T, D, MMA>;
    if (int rc = set_smem(kern, smem_bwd_main<D>())) return rc;
    {
      Prof prof(sweep == 1 ? "simt_backward_ghat" : "simt_backward_main", st);
      kern<<<grid, NT, smem_bwd_main<D>(), st>>>((const T*)q, (const T*)k, (const T*)v, gs, dout, s.dbar,
                                                  ssum, rmax, rden, carry, s.dq_main, s.dk_main,
                                                  (T*)dv, s.ghat);
    }
    if (int rc = check_launch("backward_main")) return rc;
  }
  const int64_t total = rows * D;
  // without a share step ghat is identically 0; with two sweeps it is already inside dk_main / dq_main
  const bool corrected = g.normalised && g.share != dil::kShareNone && !two_sweeps;
  if (corrected) {
    auto kern = backward_dk_correction_kernel<T, D, MMA>;
    if (int rc = set_smem(kern, smem_bwd_dk<D>())) return rc;
    {
      Prof prof("simt_backward_dk_correction", st);
      kern<<<grid, NT, smem_bwd_dk<D>(), st>>>((const T*)q, (const T*)k, g, rmax, rden, s.ghat,
                                                s.dk_main, (T*)dk);
    }
    if (int rc = check_launch("backward_dk_correction")) return rc;
  } else {
    // a bid without row normalisation has no Jacobian correction: dk is dk_main in the input dtype
    Prof prof("dk_store", st);
    dq_epilogue_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(s.dk_main, nullptr, nullptr, total, D,
                                                                          (T*)dk);
    if (int rc = check_launch("dk_store")) return rc;
  }
  {
    Prof prof("dq_epilogue", st);
    dq_epilogue_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        s.dq_main, s.ghat, corrected ? pk : nullptr, total, D, (T*)dq);
  }
  return check_launch("dq_epilogue");
}

// ---- decode ----------------------------------------------------------------
int decode_chunk(int64_t n, int64_t len) {
  int64_t chunk = 2048;
  while (chunk > dil::decode::ROUND && n * ((len + chunk - 1) / chunk) < 148 * 8) chunk /= 2;
  while ((len + chunk - 1) / chunk > dil::decode::MAX_CHUNKS) chunk *= 2;
  return (int)chunk;
}
int64_t decode_stride(int64_t len) { return (len + 31) / 32 * 32; }

dil::decode::Scratch carve_decode(void* scratch, int64_t n, int64_t len, int d) {
  dil::decode::Scratch s;
  char* p = (char*)scratch;
  s.aff = (float*)p;
  p += sizeof(float) * n * decode_stride(len);
  s.part = (float2*)p;
  p += sizeof(float2) * n * dil::decode::MAX_CHUNKS;
  s.pout = (float*)p;
  p += sizeof(float) * n * dil::decode::MAX_CHUNKS * d;
  s.psum = (float*)p;
  return s;
}

template <typename T, int D, int MODE = dil::decode::kSweepDilution>
int launch_decode(const void* q1, const void* kc, const void* vc, int64_t n, int64_t cap,
                  int64_t len, float scale, float eps, float* committed, void* out, void* scratch,
                  cudaStream_t st, bool timing = true, const void* knew = nullptr,
                  const void* vnew = nullptr, int bid = dil::kBidSoftmax, int share = dil::kShareInclusive,
                  float lshift = 0.f, const int* pos_dev = nullptr) {
  using namespace dil::decode;
  // with the length on the device (pos_dev) the launch geometry cannot follow it: the grid, the
  // chunking and the scratch layout are those of a full cache
  const int64_t geo = pos_dev != nullptr ? cap : len;
  const int chunk = decode_chunk(n, geo);
  const int nch = (int)((geo + chunk - 1) / chunk);
  const Scratch s = carve_decode(scratch, n, geo, D);
  const int64_t stride = decode_stride(geo);
  const dim3 grid((unsigned)nch, (unsigned)n);
  {
    Prof prof("decode_scores", st, timing);
    if (MODE == dil::decode::kSweepVariant && dil::row_sum_bid(bid))
      scores_kernel<T, D, true><<<grid, NT, 0, st>>>((const T*)q1, (const T*)kc, cap, (int)len, chunk,
                                                     scale * dil::kLog2e, stride, s.aff, s.part,
                                                     (const T*)knew, (T*)const_cast<void*>(kc), pos_dev, bid);
    else
      scores_kernel<T, D><<<grid, NT, 0, st>>>((const T*)q1, (const T*)kc, cap, (int)len, chunk,
                                               scale * dil::kLog2e, stride, s.aff, s.part,
                                               (const T*)knew, (T*)const_cast<void*>(kc), pos_dev);
  }
  if (int rc = check_launch("decode scores")) return rc;
  {
    Prof prof("decode_sweep", st, timing);
    sweep_kernel<T, D, MODE><<<grid, NT, 0, st>>>((const T*)vc, cap, (int)len, chunk, eps, stride, s.aff, s.part,
                                                  committed, s.pout, s.psum, (const T*)vnew,
                                                  (T*)const_cast<void*>(vc), bid, share, lshift, pos_dev);
  }
  if (int rc = check_launch("decode sweep")) return rc;
  {
    Prof prof("decode_finalize", st, timing);
    finalize_kernel<T, D><<<(unsigned)n, D, 0, st>>>(s.pout, s.psum, nch, eps, (T*)out);
  }
  return check_launch("decode finalize");
}

// ---- decode without caller-provided scratch ----------------------------------
// Scratch of dilution_decode_static: one array in device global memory, part of
// the library image, so every GPU that loads the library holds it until exit.
constexpr int64_t kStaticMaxRows = DILUTION_DECODE_STATIC_MAX_ROWS;
constexpr int64_t kStaticMaxKeys = DILUTION_DECODE_STATIC_MAX_KEYS;
constexpr size_t kStaticBytes =
    sizeof(float) * (size_t)kStaticMaxKeys +
    sizeof(float) * (size_t)kStaticMaxRows * dil::decode::MAX_CHUNKS * (2 + 128 + 1);
static_assert(kStaticBytes == DILUTION_DECODE_STATIC_BYTES, "header and library disagree on the array size");
static __device__ __align__(256) unsigned char g_decode_static[kStaticBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};

// Device address of g_decode_static on the CURRENT device.  In host code the
// array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device and cached.
int static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(DILUTION_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(DILUTION_ERR_UNSUPPORTED, "dilution_decode_static: device ordinal %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_static);
    if (e != cudaSuccess || p == nullptr)
      return fail(DILUTION_ERR_CUDA, "cudaGetSymbolAddress(static decode scratch): %s", cudaGetErrorString(e));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return DILUTION_OK;
}

}  // namespace

namespace {
int check_carry_rows(const char* fn, int dtype, int precision, int d, int64_t q_offset, int carry_rows) {
#ifdef DILUTION_TENSOR_PATH
  if (dil::tc::supported(dtype, precision, d, q_offset)) {
    if (carry_rows == 32 || carry_rows == 64) return DILUTION_OK;
    return fail(DILUTION_ERR_ARG, "%s: carry_rows must be 32 or 64 (got %d)", fn, carry_rows);
  }
#endif
  if (carry_rows == dil::kCarryRows) return DILUTION_OK;
  return fail(DILUTION_ERR_ARG, "%s: the fp32 kernels store a checkpoint every %d query rows (got %d)", fn,
              dil::kCarryRows, carry_rows);
}
}  // namespace

extern "C" {

int dilution_carry_rows(int dtype, int precision, int d, int training) {
#ifdef DILUTION_TENSOR_PATH
  if (dil::tc::supported(dtype, precision, d, 0)) return training ? 32 : 64;
#endif
  return dil::kCarryRows;
}

int dilution_version(void) { return DILUTION_ABI_VERSION; }

const char* dilution_last_error(void) { return g_err; }

int dilution_device_status(void) {
#ifdef DILUTION_TENSOR_PATH
  int v = 0;
  if (dil::tc::read_status(&v) != 0) return fail(DILUTION_ERR_CUDA, "dilution_device_status: could not read the status word");
  if (v != 0) return fail(DILUTION_ERR_DEVICE, "a kernel gave up a bounded wait (code %d)", v);
#endif
  return DILUTION_OK;
}

int dilution_selftest_bounded_wait(int* gave_up, void* stream) {
#ifdef DILUTION_TENSOR_PATH
  if (!gave_up) return fail(DILUTION_ERR_ARG, "dilution_selftest_bounded_wait: null pointer");
  return dil::tc::selftest_wait(gave_up, (cudaStream_t)stream, g_err, sizeof(g_err));
#else
  return fail(DILUTION_ERR_UNSUPPORTED, "built without the tensor-core path");
#endif
}

unsigned long long dilution_launch_count(void) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  return g_launches;
}

int dilution_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof_on = on != 0;
  return DILUTION_OK;
}

int dilution_profile_collect(char* buf, size_t cap) {
  std::vector<ProfRecord> recs;
  {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    recs.swap(g_prof);
  }
  struct Acc { std::string name; int count; double ms; };
  std::vector<Acc> accs;
  for (auto& r : recs) {
    float ms = 0.f;
    if (cudaEventSynchronize(r.b) == cudaSuccess) cudaEventElapsedTime(&ms, r.a, r.b);
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
    bool found = false;
    for (auto& a : accs)
      if (a.name == r.name) { a.count++; a.ms += ms; found = true; break; }
    if (!found) accs.push_back({r.name, 1, (double)ms});
  }
  std::string text;
  char line[160];
  for (auto& a : accs) {
    snprintf(line, sizeof(line), "%s %d %.6f\n", a.name.c_str(), a.count, a.ms);
    text += line;
  }
  if (!buf || cap == 0) return fail(DILUTION_ERR_ARG, "dilution_profile_collect: no buffer");
  if (text.size() + 1 > cap) return fail(DILUTION_ERR_ARG, "dilution_profile_collect: buffer too small");
  memcpy(buf, text.c_str(), text.size() + 1);
  return DILUTION_OK;
}

int dilution_rowstats(const void* q, const void* k, int dtype, int precision, int64_t n, int64_t tq,
                      int64_t tk, int64_t q_offset, int d, float scale, float* rmax, float* rden,
                      void* stream) {
  if (int rc = check_common("dilution_rowstats", dtype, precision, n, tq, tk, q_offset, d)) return rc;
  if (!q || !k || !rmax || !rden) return fail(DILUTION_ERR_ARG, "dilution_rowstats: null pointer");
  const dil::Geom g = make_geom(n, tq, tk, q_offset, scale, 0.f);
  cudaStream_t st = (cudaStream_t)stream;
#ifdef DILUTION_TENSOR_PATH
  if (dil::tc::supported(dtype, precision, d, q_offset)) {
    Prof prof("tc_rowstats", st);
    return dil::tc::rowstats(q, k, g, rmax, rden, st, g_err, sizeof(g_err));
  }
#endif
  DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, return (launch_rowstats<T, D, MMA>(q, k, g, rmax, rden, st))))
  return DILUTION_OK;
}

int dilution_rowstats_pk(const void* q, const void* k, int dtype, int precision, int64_t n, int64_t t,
                         int d, float scale, float* rmax, float* rden, float* pk, void* stream) {
  if (int rc = check_common("dilution_rowstats_pk", dtype, precision, n, t, t, 0, d)) return rc;
  if (!q || !k || !rmax || !rden || !pk) return fail(DILUTION_ERR_ARG, "dilution_rowstats_pk: null pointer");
#ifdef DILUTION_TENSOR_PATH
  if (dil::tc::supported(dtype, precision, d, 0)) {
    const dil::Geom g = make_geom(n, t, t, 0, scale, 0.f);
    cudaStream_t st = (cudaStream_t)stream;
    Prof prof("tc_rowstats_pk", st);
    return dil::tc::rowstats_pk(q, k, g, rmax, rden, pk, st, g_err, sizeof(g_err));
  }
#endif
  return fail(DILUTION_ERR_UNSUPPORTED, "dilution_rowstats_pk: bf16 inputs, BF16 precision and head_dim 64 only "
              "(other cases get pk from dilution_forward_main)");
}

int dilution_softmax_forward(const void* q, const void* k, const void* v, int dtype, int precision, int64_t n,
                             int64_t tq, int64_t tk, int64_t q_offset, int d, float scale, float* rmax,
                             float* rden, void* out, void* stream) {
  if (int rc = check_common("dilution_softmax_forward", dtype, precision, n, tq, tk, q_offset, d)) return rc;
  if (!q || !k || !v || !out) return fail(DILUTION_ERR_ARG, "dilution_softmax_forward: null pointer");
  if ((rmax == nullptr) != (rden == nullptr))
    return fail(DILUTION_ERR_ARG, "dilution_softmax_forward: rmax and rden go together");
#ifdef DILUTION_TENSOR_PATH
  if (dil::tc::supported(dtype, precision, d, q_offset)) {
    const dil::Geom g = make_geom(n, tq, tk, q_offset, scale, 0.f);
    cudaStream_t st = (cudaStream_t)stream;
    Prof prof("tc_softmax_forward", st);
    return dil::tc::softmax_forward(q, k, v, g, rmax, rden, out, st, g_err, sizeof(g_err));
  }
#endif
  return fail(DILUTION_ERR_UNSUPPORTED, "dilution_softmax_forward: bf16 inputs, BF16 precision, head_dim 64 and "
              "q_offset a multiple of 128 only");
}

int dilution_colsum_scan(const void* q, const void* k, int dtype, int precision, int64_t n,
                         int64_t tq, int64_t tk, int64_t q_offset, int d, float scale,
                         const float* rmax, const float* rden, const float* carry_base,
                         int carry_rows, float* carry, float* total, void* stream) {
  if (int rc = check_common("dilution_colsum_scan", dtype, precision, n, tq, tk, q_offset, d)) return rc;
  if (!q || !k || !rmax || !rden || !carry || !total)
    return fail(DILUTION_ERR_ARG, "dilution_colsum_scan: null pointer");
  if (int rc = check_carry_rows("dilution_colsum_scan", dtype, precision, d, q_offset, carry_rows)) return rc;
  const dil::Geom g = make_geom(n, tq, tk, q_offset, scale, 0.f, carry_rows);
  cudaStream_t st = (cudaStream_t)stream;
#ifdef DILUTION_TENSOR_PATH
  if (dil::tc::supported(dtype, precision, d, q_offset)) {
    Prof prof("tc_colsum_scan", st);
    return dil::tc::colsum_scan(q, k, g, rmax, rden, carry_base, carry, total, st, g_err, sizeof(g_err));
  }
#endif
  DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, return (launch_colsum<T, D, MMA>(q, k, g, rmax, rden, carry_base, carry, total, st))))
  return DILUTION_OK;
}

int dilution_forward_main(const void* q, const void* k, const void* v, int dtype, int precision,
                          int64_t n, int64_t tq, int64_t tk, int64_t q_offset, int d, float scale,
                          float eps, const float* rmax, const float* rden, const float* carry,
                          int carry_rows, const float* carry_base, float* out, float* ssum, float* pk,
                          void* stream) {
  if (int rc = check_common("dilution_forward_main", dtype, precision, n, tq, tk, q_offset, d)) return rc;
  if (!q || !k || !v || !rmax || !rden || !carry || !out || !ssum)
    return fail(DILUTION_ERR_ARG, "dilution_forward_main: null pointer");
  if (int rc = check_carry_rows("dilution_forward_main", dtype, precision, d, q_offset, carry_rows)) return rc;
  const dil::Geom g = make_geom(n, tq, tk, q_offset, scale, eps, carry_rows);
  cudaStream_t st = (cudaStream_t)stream;
#ifdef DILUTION_TENSOR_PATH
#if DILUTION_TC_HAS_MAIN
  // pk is produced by the fp32 kernel only: the tensor-core backward does not need it
  if (pk == nullptr && dil::tc::supported(dtype, precision, d, q_offset)) {
    Prof prof("tc_forward_main", st);
    return dil::tc::forward_main(q, k, v, g, rmax, rden, carry, carry_base, out, ssum, st, g_err,
                                 sizeof(g_err));
  }
#endif
#endif
  DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, return (launch_main<T, D, MMA>(q, k, v, g, rmax, rden, carry, carry_base, out, ssum, pk, st))))
  return DILUTION_OK;
}

int dilution_forward_fused(const void* q, const void* k, const void* v, int dtype, int precision, int64_t n,
                           int64_t t, int d, float scale, float eps, const float* rmax, const float* rden,
                           float* carry, float* total, float* out, float* ssum, void* stream) {
  if (int rc = check_common("dilution_forward_fused", dtype, precision, n, t, t, 0, d)) return rc;
  if (!q || !k || !v || !rmax || !rden || !carry || !total || !out || !ssum)
    return fail(DILUTION_ERR_ARG, "dilution_forward_fused: null pointer");
#if defined(DILUTION_TENSOR_PATH) && DILUTION_TC_HAS_MAIN
  if (dil::tc::supported(dtype, precision, d, 0)) {
    const dil::Geom g = make_geom(n, t, t, 0, scale, eps, 32);
    cudaStream_t st = (cudaStream_t)stream;
    {
      Prof prof("tc_forward_fused", st);
      if (int rc = dil::tc::forward_fused(q, k, v, g, rmax, rden, carry, total, out, ssum, st, g_err, sizeof(g_err)))
        return rc;
    }
    Prof prof("tc_normalize_out", st);
    return dil::tc::normalize_out(g, out, ssum, st, g_err, sizeof(g_err));
  }
#endif
  return fail(DILUTION_ERR_UNSUPPORTED, "dilution_forward_fused: bf16 inputs, BF16 precision and head_dim 64 only "
              "(other cases run dilution_colsum_scan and dilution_forward_main)");
}

size_t dilution_backward_scratch_bytes(int64_t n, int64_t t, int d) {
  if (n < 1 || t < 1 || d < 1) return 0;
  return sizeof(float) * (size_t)(2 * n * t * d + 2 * n * t) + 2 * (size_t)(n * t * d);
}

int dilution_backward(const void* q, const void* k, const void* v, int dtype, int precision,
                      int64_t n, int64_t t, int d, float scale, float eps, const void* dout,
                      int dout_dtype, const float* out, const float* rmax, const float* rden, const float* carry,
                      int carry_rows, const float* total, const float* ssum, const float* pk, void* scratch,
                      void* dq, void* dk, void* dv, void* stream) {
  if (int rc = check_common("dilution_backward", dtype, precision, n, t, t, 0, d)) return rc;
  if (!q || !k || !v || !dout || !out || !rmax || !rden || !carry || !total || !ssum || !scratch ||
      !dq || !dk || !dv)
    return fail(DILUTION_ERR_ARG, "dilution_backward: null pointer");
  if (dout_dtype != DILUTION_F32 && dout_dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "dilution_backward: dout_dtype must be DILUTION_F32 or DILUTION_BF16");
  if (int rc = check_carry_rows("dilution_backward", dtype, precision, d, 0, carry_rows)) return rc;
  if (carry_rows == 64) return fail(DILUTION_ERR_ARG, "dilution_backward: checkpoints every 64 rows serve forward-only calls");
  const dil::Geom g = make_geom(n, t, t, 0, scale, eps, carry_rows);
  const BwdScratch s = carve_bwd(scratch, n, t, d);
  cudaStream_t st = (cudaStream_t)stream;
#ifdef DILUTION_TENSOR_PATH
#if DILUTION_TC_HAS_BACKWARD
  if (dil::tc::supported(dtype, precision, d, 0))
    return dil::tc::backward(q, k, v, g, dout, dout_dtype, out, rmax, rden, carry, total, ssum, pk, s.dq_main, s.dk_main,
                             s.ghat, s.dbar, s.dop, dq, dk, dv, st, g_err, sizeof(g_err), mark_scope);
#endif
  if (!pk) return fail(DILUTION_ERR_ARG, "dilution_backward: the fp32 path needs pk from dilution_forward_main");
#endif
  if (dout_dtype != DILUTION_F32)
    return fail(DILUTION_ERR_UNSUPPORTED, "dilution_backward: the fp32 path takes an fp32 dout");
  DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, return (launch_backward<T, D, MMA>(
      q, k, v, g, (const float*)dout, out, rmax, rden, carry, ssum, pk, s, dq, dk, dv, st))))
  return DILUTION_OK;
}

size_t dilution_decode_scratch_bytes(int64_t n, int64_t length, int d) {
  if (n < 1 || length < 1 || d < 1) return 0;
  return sizeof(float) * (size_t)(n * decode_stride(length)) +
         sizeof(float) * (size_t)(n * dil::decode::MAX_CHUNKS) * (size_t)(2 + d + 1);
}

int dilution_decode(const void* q1, const void* k_cache, const void* v_cache, int dtype, int64_t n,
                    int64_t capacity, int64_t length, int d, float scale, float eps,
                    float* committed, void* out, void* scratch, void* stream) {
  if (dtype != DILUTION_F32 && dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "dilution_decode: dtype must be DILUTION_F32 or DILUTION_BF16");
  if (!valid_d(d)) return fail(DILUTION_ERR_UNSUPPORTED, "dilution_decode: head_dim %d not in {16, 32, 64, 128}", d);
  if (n < 1 || n > 65535) return fail(DILUTION_ERR_ARG, "dilution_decode: n must be in [1, 65535] rows per call");
  if (capacity < 1 || length < 1 || length > capacity || capacity > (1 << 30))
    return fail(DILUTION_ERR_ARG, "dilution_decode: length %lld outside cache capacity %lld",
                (long long)length, (long long)capacity);
  if (!q1 || !k_cache || !v_cache || !committed || !out || !scratch)
    return fail(DILUTION_ERR_ARG, "dilution_decode: null pointer");
  if (((uintptr_t)q1 | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
    return fail(DILUTION_ERR_ARG, "dilution_decode: q1 / caches must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  DIL_DISPATCH(dtype, d, return (launch_decode<T, D>(q1, k_cache, v_cache, n, capacity, length, scale, eps,
                                                     committed, out, scratch, st)))
  return DILUTION_OK;
}

int dilution_decode_append(const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                           int dtype, int64_t n, int64_t capacity, int64_t length, int d, float scale,
                           float eps, float* committed, void* out, void* scratch, void* stream) {
  if (dtype != DILUTION_F32 && dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "dilution_decode_append: dtype must be DILUTION_F32 or DILUTION_BF16");
  if (!valid_d(d))
    return fail(DILUTION_ERR_UNSUPPORTED, "dilution_decode_append: head_dim %d not in {16, 32, 64, 128}", d);
  if (n < 1 || n > 65535)
    return fail(DILUTION_ERR_ARG, "dilution_decode_append: n must be in [1, 65535] rows per call");
  if (capacity < 1 || length < 1 || length > capacity || capacity > (1 << 30))
    return fail(DILUTION_ERR_ARG, "dilution_decode_append: decode step past the cache capacity "
                "(length %lld, capacity %lld)", (long long)length, (long long)capacity);
  if (!q1 || !k1 || !v1 || !k_cache || !v_cache || !committed || !out || !scratch)
    return fail(DILUTION_ERR_ARG, "dilution_decode_append: null pointer");
  if (((uintptr_t)q1 | (uintptr_t)k1 | (uintptr_t)v1 | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
    return fail(DILUTION_ERR_ARG, "dilution_decode_append: q1 / k1 / v1 / caches must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  DIL_DISPATCH(dtype, d, return (launch_decode<T, D>(q1, k_cache, v_cache, n, capacity, length, scale, eps,
                                                     committed, out, scratch, st, true, k1, v1)))
  return DILUTION_OK;
}

static int split_heads_rope_impl(void* qkv, void* q, void* k, void* v, const void* cos_table,
                                 const void* sin_table, int64_t batch, int64_t seq, int heads, int d,
                                 int inverse, const int* pos_dev, int64_t table_rows, void* stream) {
  if (!qkv || !q || !k || !v) return fail(DILUTION_ERR_ARG, "dilution_split_heads_rope: null pointer");
  if ((cos_table == nullptr) != (sin_table == nullptr))
    return fail(DILUTION_ERR_ARG, "dilution_split_heads_rope: cos and sin tables go together");
  if (d != 64 && d != 128 && d != 32)
    return fail(DILUTION_ERR_UNSUPPORTED, "dilution_split_heads_rope: head_dim %d not in {32, 64, 128}", d);
  if (batch < 1 || seq < 1 || heads < 1 || batch * seq * heads * (d / 8) >= ((int64_t)1 << 39))
    return fail(DILUTION_ERR_ARG, "dilution_split_heads_rope: sizes out of range");
  if (((uintptr_t)qkv | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15 ||
      ((uintptr_t)cos_table | (uintptr_t)sin_table) & 7)
    return fail(DILUTION_ERR_ARG, "dilution_split_heads_rope: tensors must be 16-byte aligned (tables 8)");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = batch * seq * heads * (d / 8);
  const unsigned grid = (unsigned)((total + 255) / 256);
  using bf = __nv_bfloat16;
  Prof prof(inverse ? "merge_heads_rope_grad" : "split_heads_rope", st);
#define DIL_ROPE(DD)                                                                                           \
  if (inverse)                                                                                                 \
    dil::layer::split_heads_rope_kernel<false, DD><<<grid, 256, 0, st>>>(                                      \
        (bf*)qkv, (bf*)q, (bf*)k, (bf*)v, (const bf*)cos_table, (const bf*)sin_table, batch, seq, heads,      \
        pos_dev, table_rows);                                                                                  \
  else                                                                                                         \
    dil::layer::split_heads_rope_kernel<true, DD><<<grid, 256, 0, st>>>(                                       \
        (bf*)qkv, (bf*)q, (bf*)k, (bf*)v, (const bf*)cos_table, (const bf*)sin_table, batch, seq, heads,      \
        pos_dev, table_rows);
  if (d == 32) { DIL_ROPE(32) } else if (d == 64) { DIL_ROPE(64) } else { DIL_ROPE(128) }
#undef DIL_ROPE
  return check_launch("split_heads_rope");
}

int dilution_split_heads_rope(void* qkv, void* q, void* k, void* v, const void* cos_table,
                              const void* sin_table, int64_t batch, int64_t seq, int heads, int d,
                              int inverse, void* stream) {
  return split_heads_rope_impl(qkv, q, k, v, cos_table, sin_table, batch, seq, heads, d, inverse, nullptr, 0, stream);
}

int dilution_split_heads_rope_at(void* qkv, void* q, void* k, void* v, const void* cos_table,
                                 const void* sin_table, int64_t table_rows, int64_t batch, int heads, int d,
                                 const int* position_dev, void* stream) {
  if (!position_dev) return fail(DILUTION_ERR_ARG, "dilution_split_heads_rope_at: null position");
  if (cos_table != nullptr && table_rows < 1)
    return fail(DILUTION_ERR_ARG, "dilution_split_heads_rope_at: table_rows must be the tables' row count");
  return split_heads_rope_impl(qkv, q, k, v, cos_table, sin_table, batch, 1, heads, d, 0, position_dev,
                               table_rows, stream);
}

int dilution_softmax_decode_append(const void* q1, const void* k1, const void* v1, void* k_cache,
                                   void* v_cache, int dtype, int64_t n, int64_t capacity, int64_t length,
                                   int d, float scale, void* out, void* scratch, void* stream) {
  if (dtype != DILUTION_F32 && dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "dilution_softmax_decode_append: dtype must be DILUTION_F32 or DILUTION_BF16");
  if (!valid_d(d))
    return fail(DILUTION_ERR_UNSUPPORTED, "dilution_softmax_decode_append: head_dim %d not in {16, 32, 64, 128}", d);
  if (n < 1 || n > 65535)
    return fail(DILUTION_ERR_ARG, "dilution_softmax_decode_append: n must be in [1, 65535] rows per call");
  if (capacity < 1 || length < 1 || length > capacity || capacity > (1 << 30))
    return fail(DILUTION_ERR_ARG, "dilution_softmax_decode_append: decode step past the cache capacity "
                "(length %lld, capacity %lld)", (long long)length, (long long)capacity);
  if (!q1 || !k_cache || !v_cache || !out || !scratch || ((k1 == nullptr) != (v1 == nullptr)))
    return fail(DILUTION_ERR_ARG, "dilution_softmax_decode_append: null pointer");
  if (((uintptr_t)q1 | (uintptr_t)k1 | (uintptr_t)v1 | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
    return fail(DILUTION_ERR_ARG, "dilution_softmax_decode_append: q1 / k1 / v1 / caches must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  DIL_DISPATCH(dtype, d, return (launch_decode<T, D, dil::decode::kSweepSoftmax>(q1, k_cache, v_cache, n, capacity, length, scale,
                                                            0.f, nullptr, out, scratch, st, true, k1, v1)))
  return DILUTION_OK;
}

// ---- share / bid variants (the tile kernels; kernels_bid.py of the reference) -------------
static int check_variant(const char* fn, int bid, int share, float shift) {
  if (bid < 0 || bid > 7)
    return fail(DILUTION_ERR_ARG, "%s: bid %d is not one of softmax 0, relu 1, relu2 2, softplus 3, minshift 4, "
                "sigmoid 5, expshift 6, sigshift 7", fn, bid);
  if ((bid == dil::kBidExpshift || bid == dil::kBidSigshift) && !(shift > 0.f))
    return fail(DILUTION_ERR_ARG, "%s: shift must be positive", fn);
  if (share != dil::kShareNone && share != dil::kShareInclusive && share != dil::kShareExclusive)
    return fail(DILUTION_ERR_ARG, "%s: share must be 0 (none), 1 (inclusive) or 2 (exclusive)", fn);
  return DILUTION_OK;
}

int dilution_variant_forward(const void* q, const void* k, const void* v, int dtype, int precision, int64_t n,
                             int64_t t, int d, float scale, float eps, int bid, int share, float shift, float* rmax,
                             float* rden, float* carry, float* total, float* out, float* ssum, float* pk,
                             void* stream) {
  if (int rc = check_common("dilution_variant_forward", dtype, precision, n, t, t, 0, d)) return rc;
  if (int rc = check_variant("dilution_variant_forward", bid, share, shift)) return rc;
  const bool stats = bid == dil::kBidSoftmax || dil::row_sum_bid(bid);   // bids with row statistics
  // without a share step nothing downstream reads the checkpoints: carry and total may both be
  // NULL, and the column-sum pass is skipped
  const bool scan = !(share == dil::kShareNone && carry == nullptr && total == nullptr);
  if (!q || !k || !v || (scan && (!carry || !total)) || !out || !ssum || (stats && (!rmax || !rden)))
    return fail(DILUTION_ERR_ARG, "dilution_variant_forward: null pointer");
  if (!stats) rmax = rden = nullptr;
  if (bid != dil::kBidSoftmax) pk = nullptr;       // only the softmax bid's backward reads pk
  const dil::Geom g = make_geom(n, t, t, 0, scale, eps, dil::kCarryRows, bid, share, shift);
  cudaStream_t st = (cudaStream_t)stream;
#if defined(DILUTION_TENSOR_PATH) && DILUTION_TC_HAS_MAIN
  if (dil::tc::supported(dtype, precision, d, 0) && !dil::row_sum_bid(bid)) {
    // bf16 tensors, head_dim 64: the tcgen05 kernels, instantiated for the bid and share step
    if (stats && pk) {
      Prof prof("tc_rowstats_pk", st);
      if (int rc = dil::tc::rowstats_pk(q, k, g, rmax, rden, pk, st, g_err, sizeof(g_err))) return rc;
    } else if (stats) {
      Prof prof("tc_rowstats", st);
      if (int rc = dil::tc::rowstats(q, k, g, rmax, rden, st, g_err, sizeof(g_err))) return rc;
    }
    if (scan) {
      Prof prof("tc_colsum_scan", st);
      if (int rc = dil::tc::colsum_scan(q, k, g, rmax, rden, nullptr, carry, total, st, g_err, sizeof(g_err))) return rc;
    }
    Prof prof("tc_forward_main", st);
    return dil::tc::forward_main(q, k, v, g, rmax, rden, carry, nullptr, out, ssum, st, g_err, sizeof(g_err));
  }
#endif
  if (stats) {
    DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, {
      if (int rc = launch_rowstats<T, D, MMA>(q, k, g, rmax, rden, st)) return rc;
    }))
  }
  if (scan) {
    DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, {
      if (int rc = launch_colsum<T, D, MMA>(q, k, g, rmax, rden, nullptr, carry, total, st)) return rc;
    }))
  }
  DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, return (launch_main<T, D, MMA>(q, k, v, g, rmax, rden, carry, nullptr, out, ssum, pk, st))))
  return DILUTION_OK;
}

int dilution_variant_backward(const void* q, const void* k, const void* v, int dtype, int precision, int64_t n,
                              int64_t t, int d, float scale, float eps, int bid, int share, float shift, const float* dout,
                              const float* out, const float* rmax, const float* rden, const float* carry,
                              const float* total, const float* ssum, const float* pk, void* scratch, void* dq,
                              void* dk, void* dv, void* stream) {
  if (int rc = check_common("dilution_variant_backward", dtype, precision, n, t, t, 0, d)) return rc;
  if (int rc = check_variant("dilution_variant_backward", bid, share, shift)) return rc;
  const bool stats = bid == dil::kBidSoftmax || dil::row_sum_bid(bid);
  if (!q || !k || !v || !dout || !out || !ssum || !scratch || !dq || !dk || !dv ||
      (share != dil::kShareNone && (!carry || !total)) || (stats && (!rmax || !rden)) ||
      (bid == dil::kBidSoftmax && share != dil::kShareNone && !pk))
    return fail(DILUTION_ERR_ARG, "dilution_variant_backward: null pointer");
  if (!stats) rmax = rden = nullptr;
  if (bid != dil::kBidSoftmax || share == dil::kShareNone) pk = nullptr;
  const dil::Geom g = make_geom(n, t, t, 0, scale, eps, dil::kCarryRows, bid, share, shift);
  const BwdScratch s = carve_bwd(scratch, n, t, d);
  cudaStream_t st = (cudaStream_t)stream;
#if defined(DILUTION_TENSOR_PATH) && DILUTION_TC_HAS_BACKWARD
  if (dil::tc::supported(dtype, precision, d, 0) && !dil::row_sum_bid(bid))
    return dil::tc::backward(q, k, v, g, dout, DILUTION_F32, out, rmax, rden, carry, total, ssum, pk, s.dq_main,
                             s.dk_main, s.ghat, s.dbar, s.dop, dq, dk, dv, st, g_err, sizeof(g_err), mark_scope);
#endif
  DIL_DISPATCH(dtype, d, DIL_DISPATCH_MMA(precision, return (launch_backward<T, D, MMA>(
      q, k, v, g, dout, out, rmax, rden, carry, ssum, pk, s, dq, dk, dv, st))))
  return DILUTION_OK;
}

int dilution_variant_decode(const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                            int dtype, int64_t n, int64_t capacity, int64_t length, int d, float scale,
                            float eps, int bid, int share, float shift, float* committed, void* out, void* scratch,
                            void* stream) {
  if (dtype != DILUTION_F32 && dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "dilution_variant_decode: dtype must be DILUTION_F32 or DILUTION_BF16");
  if (int rc = check_variant("dilution_variant_decode", bid, share, shift)) return rc;
  if (!valid_d(d))
    return fail(DILUTION_ERR_UNSUPPORTED, "dilution_variant_decode: head_dim %d not in {16, 32, 64, 128}", d);
  if (n < 1 || n > 65535)
    return fail(DILUTION_ERR_ARG, "dilution_variant_decode: n must be in [1, 65535] rows per call");
  if (capacity < 1 || length < 1 || length > capacity || capacity > (1 << 30))
    return fail(DILUTION_ERR_ARG, "dilution_variant_decode: length %lld outside cache capacity %lld",
                (long long)length, (long long)capacity);
  if (!q1 || !k_cache || !v_cache || !committed || !out || !scratch || ((k1 == nullptr) != (v1 == nullptr)))
    return fail(DILUTION_ERR_ARG, "dilution_variant_decode: null pointer");
  if (((uintptr_t)q1 | (uintptr_t)k1 | (uintptr_t)v1 | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
    return fail(DILUTION_ERR_ARG, "dilution_variant_decode: q1 / k1 / v1 / caches must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  DIL_DISPATCH(dtype, d, return (launch_decode<T, D, dil::decode::kSweepVariant>(
      q1, k_cache, v_cache, n, capacity, length, scale, eps, committed, out, scratch, st, true, k1, v1, bid, share,
      (bid == dil::kBidExpshift || bid == dil::kBidSigshift) ? log2f(shift) * 1.f : 0.f)))
  return DILUTION_OK;
}

// ---- cached steps whose length lives on the device (for a captured graph) ------------------
static int check_decode_at(const char* fn, int dtype, int64_t n, int64_t capacity, int d, const void* q1,
                           const void* k1, const void* v1, const void* kc, const void* vc, const void* pos,
                           const void* out, const void* scratch) {
  if (dtype != DILUTION_F32 && dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "%s: dtype must be DILUTION_F32 or DILUTION_BF16", fn);
  if (!valid_d(d)) return fail(DILUTION_ERR_UNSUPPORTED, "%s: head_dim %d not in {16, 32, 64, 128}", fn, d);
  if (n < 1 || n > 65535) return fail(DILUTION_ERR_ARG, "%s: n must be in [1, 65535] rows per call", fn);
  if (capacity < 1 || capacity > (1 << 30)) return fail(DILUTION_ERR_ARG, "%s: capacity out of range", fn);
  if (!q1 || !k1 || !v1 || !kc || !vc || !pos || !out || !scratch) return fail(DILUTION_ERR_ARG, "%s: null pointer", fn);
  if (((uintptr_t)q1 | (uintptr_t)k1 | (uintptr_t)v1 | (uintptr_t)kc | (uintptr_t)vc) & 15)
    return fail(DILUTION_ERR_ARG, "%s: q1 / k1 / v1 / caches must be 16-byte aligned", fn);
  return DILUTION_OK;
}

int dilution_decode_append_at(const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                              int dtype, int64_t n, int64_t capacity, const int* position_dev, int d,
                              float scale, float eps, float* committed, void* out, void* scratch,
                              void* stream) {
  if (int rc = check_decode_at("dilution_decode_append_at", dtype, n, capacity, d, q1, k1, v1, k_cache, v_cache,
                               position_dev, out, scratch)) return rc;
  if (!committed) return fail(DILUTION_ERR_ARG, "dilution_decode_append_at: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  DIL_DISPATCH(dtype, d, return (launch_decode<T, D>(q1, k_cache, v_cache, n, capacity, 0, scale, eps, committed, out,
                                                     scratch, st, true, k1, v1, dil::kBidSoftmax,
                                                     dil::kShareInclusive, 0.f, position_dev)))
  return DILUTION_OK;
}

int dilution_softmax_decode_append_at(const void* q1, const void* k1, const void* v1, void* k_cache,
                                      void* v_cache, int dtype, int64_t n, int64_t capacity,
                                      const int* position_dev, int d, float scale, void* out, void* scratch,
                                      void* stream) {
  if (int rc = check_decode_at("dilution_softmax_decode_append_at", dtype, n, capacity, d, q1, k1, v1, k_cache,
                               v_cache, position_dev, out, scratch)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  DIL_DISPATCH(dtype, d, return (launch_decode<T, D, dil::decode::kSweepSoftmax>(
      q1, k_cache, v_cache, n, capacity, 0, scale, 0.f, nullptr, out, scratch, st, true, k1, v1, dil::kBidSoftmax,
      dil::kShareInclusive, 0.f, position_dev)))
  return DILUTION_OK;
}

int dilution_decode_static(const void* q1, const void* k_cache, const void* v_cache, int dtype,
                           int64_t n, int64_t capacity, int64_t length, int d, float scale, float eps,
                           float* committed, void* out, void* stream) {
  if (dtype != DILUTION_F32 && dtype != DILUTION_BF16)
    return fail(DILUTION_ERR_ARG, "dilution_decode_static: dtype must be DILUTION_F32 or DILUTION_BF16");
  if (!valid_d(d))
    return fail(DILUTION_ERR_UNSUPPORTED, "dilution_decode_static: head_dim %d not in {16, 32, 64, 128}", d);
  if (n < 1 || capacity < 1 || length < 1 || length > capacity || capacity > (1 << 30))
    return fail(DILUTION_ERR_ARG, "dilution_decode_static: length %lld outside cache capacity %lld",
                (long long)length, (long long)capacity);
  if (n > kStaticMaxRows || n * decode_stride(length) > kStaticMaxKeys)
    return fail(DILUTION_ERR_ARG,
                "dilution_decode_static: %lld rows x %lld keys exceeds the built-in scratch "
                "(at most %lld rows and rows * round_up(length, 32) <= %lld); use dilution_decode "
                "with caller-provided scratch",
                (long long)n, (long long)length, (long long)kStaticMaxRows, (long long)kStaticMaxKeys);
  if (!q1 || !k_cache || !v_cache || !committed || !out)
    return fail(DILUTION_ERR_ARG, "dilution_decode_static: null pointer");
  if (((uintptr_t)q1 | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
    return fail(DILUTION_ERR_ARG, "dilution_decode_static: q1 / caches must be 16-byte aligned");
  void* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  DIL_DISPATCH(dtype, d, return (launch_decode<T, D>(q1, k_cache, v_cache, n, capacity, length, scale, eps,
                                                     committed, out, scratch, st, /*timing=*/false)))
  return DILUTION_OK;
}

}  // extern "C"
