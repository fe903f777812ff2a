/*
 * dilution_b200.h — C ABI of libdilution_b200.so (sm_100a).
 *
 * Drop-in boundary for ONE path of Royer-Research-Labs/Dilution-Attention: the
 * entry points of its `dilution.kernels` module (src/dilution/kernels.py).  The
 * reference launches Triton kernels from Python; a host that wants this library
 * instead binds the functions below (ctypes from Python) and keeps the
 * Python-level signatures unchanged.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer owned by the caller; nothing here
 *    allocates, frees or synchronises; every launch goes to `stream`
 *    (a cudaStream_t passed as void*);
 *  - q/k/v/… are contiguous (n, t, d) row-major, n = batch*heads, exactly what
 *    the reference builds with reshape(n, seq, d).contiguous() (kernels.py:362-364);
 *  - `dtype` is the element type of q/k/v (and of the decode caches);
 *  - `precision` mirrors the reference's dot_precision (kernels.py:318-325):
 *    IEEE keeps fp32 products (fp32 FMAs); TF32 rounds the operands of every
 *    product to tf32 and accumulates in fp32 on the tensor cores, as tl.dot does
 *    with input_precision="tf32" (kernels.py:81-92); BF16 uses bf16 tensor-core
 *    operands with fp32 accumulation (tcgen05 for bf16 tensors of head_dim 64;
 *    the tf32 tile kernels, which hold bf16 values without loss, otherwise);
 *  - row statistics are in the log2 domain as in kernels.py:159-184:
 *    rmax = max_j z_ij, rden = sum_j 2^(z_ij - rmax), z = q.k * scale * log2(e);
 *  - `q_offset`: absolute position of local query row 0 (0 for a whole sequence;
 *    a multiple of 128 for a sequence-parallel rank that owns a query chunk).
 *    Query i (local) sees keys j <= i + q_offset, j < tk;
 *  - carry rows are checkpoints of per-key cumulative demand every `carry_rows`
 *    query rows (aux["bwd_block_m"] of the reference, kernels.py:374-377):
 *    carry[n][rb][j] = (carry_base[n][j]) + sum over local rows i < rb*carry_rows
 *    of p_ij.  Entries for keys a row block cannot see are left unwritten (as
 *    kernels.py:353-354).  The spacing is the caller's choice among what the kernels
 *    for its case take — dilution_carry_rows() names the preferred one — and must be
 *    the same in every call that shares a carry buffer;
 *  - return value 0 = ok; otherwise an error code, with a message available
 *    from dilution_last_error() (thread-local).
 */
#ifndef DILUTION_B200_H
#define DILUTION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DILUTION_ABI_VERSION 5
#define DILUTION_CARRY_ROWS 32      /* query rows per carry checkpoint of the fp32 kernels */

enum { DILUTION_F32 = 0, DILUTION_BF16 = 1 };                       /* dtype */
enum { DILUTION_PREC_IEEE = 0, DILUTION_PREC_TF32 = 1, DILUTION_PREC_BF16 = 2 }; /* precision */
enum { DILUTION_BID_SOFTMAX = 0, DILUTION_BID_RELU = 1, DILUTION_BID_RELU2 = 2, DILUTION_BID_SOFTPLUS = 3,
       DILUTION_BID_MINSHIFT = 4, DILUTION_BID_SIGMOID = 5, DILUTION_BID_EXPSHIFT = 6,
       DILUTION_BID_SIGSHIFT = 7 };                                 /* bid codes of kernels_bid.py:84 */
enum { DILUTION_SHARE_NONE = 0, DILUTION_SHARE_INCLUSIVE = 1, DILUTION_SHARE_EXCLUSIVE = 2 }; /* kernels_bid.py:123-127 */
enum {
  DILUTION_OK = 0,
  DILUTION_ERR_ARG = 1,        /* bad size / dtype / null pointer / alignment */
  DILUTION_ERR_UNSUPPORTED = 2,/* head_dim or dtype combination not built */
  DILUTION_ERR_CUDA = 3,       /* a CUDA runtime call or launch failed */
  DILUTION_ERR_DEVICE = 4      /* a kernel reported a bounded wait that ran out */
};

/* ABI version of the loaded library. No reference counterpart (the reference's
 * availability flag is HAS_TRITON, kernels.py:31-37). */
int dilution_version(void);

/* Message of the last failing call on this host thread ("" if none). */
const char* dilution_last_error(void);

/* Every wait inside a kernel (on a TMA copy or a tensor-core batch) is bounded; a
 * wait that runs out records a code in a device status word and the kernel
 * drains and returns instead of hanging.  This call SYNCHRONISES the device
 * (cudaDeviceSynchronize, so kernels on non-blocking streams are included),
 * returns DILUTION_ERR_DEVICE if a code was recorded since the last call (and
 * clears it), else DILUTION_OK.  No reference counterpart. */
int dilution_device_status(void);

/* Exercises the bounded wait without faulting anything: launches one tiny kernel
 * that waits (about a millisecond) on a barrier nothing will complete.  The wait
 * gives up, the kernel writes 1 to *gave_up (device int) and returns normally, and
 * the next dilution_device_status() reports DILUTION_ERR_DEVICE once.  The context
 * stays usable.  No reference counterpart. */
int dilution_selftest_bounded_wait(int* gave_up, void* stream);

/* Kernel launches issued by this library so far in this process.
 * No reference counterpart. */
unsigned long long dilution_launch_count(void);

/* Per-kernel timing with CUDA events on the launching stream (off by default).
 * The reference profiles the same way from Python, with torch.profiler and CUDA
 * events (scripts/step_profile.py:29-47, scripts/profile_kernels.py:115-124).
 * dilution_profile_collect waits for the recorded events, writes one line
 * "<kernel> <launches> <total_ms>" per kernel into buf and clears the records. */
int dilution_profile_enable(int on);
int dilution_profile_collect(char* buf, size_t cap);

/* Preferred checkpoint spacing for this case: 32 query rows when a backward will follow (the
 * reference's bwd_block_m; the reverse pass gives every thread 32 queries) and on the fp32
 * kernels; 64 for forward-only calls of the tensor-core kernels (bf16, BF16 precision,
 * d == 64): half the scratch.  The tensor-core forward kernels accept 32 and 64, everything
 * else 32 only. */
int dilution_carry_rows(int dtype, int precision, int d, int training);

/* Pass 1 — causal-softmax row statistics for every query.
 * Replaces _dilution_k1's sweep 1 (kernels.py:158-185).
 * rmax, rden: (n, tq) fp32 out. */
int dilution_rowstats(const void* q, const void* k, int dtype, int precision,
                      int64_t n, int64_t tq, int64_t tk, int64_t q_offset, int d, float scale,
                      float* rmax, float* rden, void* stream);

/* Pass 1 with the saved query correction: rmax, rden as dilution_rowstats writes them, and
 * pk = scale * softmax(q k^T) k, (n, t, d) fp32, from the same sweep — what the reference's K1
 * computes with PK set (kernels.py:161-188).  Whole sequences only (tq == tk == t, offset 0);
 * bf16 inputs, BF16 precision, d == 64 (DILUTION_ERR_UNSUPPORTED otherwise: the fp32 kernels
 * produce pk in dilution_forward_main).  dilution_backward given this pk skips the query
 * half of its correction pass. */
int dilution_rowstats_pk(const void* q, const void* k, int dtype, int precision,
                         int64_t n, int64_t t, int d, float scale,
                         float* rmax, float* rden, float* pk, void* stream);

/* Causal softmax attention forward, out = softmax(q k^T * scale) v: the reference's
 * CausalSelfAttention layers (model.py:96-117, F.scaled_dot_product_attention with
 * is_causal=True) on the same pipeline — pass 1 plus a plain P V product.
 * bf16 inputs, BF16 precision, d == 64, q_offset a multiple of 128.
 * out: (n, tq, d) bf16.  rmax, rden: optional (n, tq) fp32 row statistics (both or neither). */
int dilution_softmax_forward(const void* q, const void* k, const void* v, int dtype, int precision,
                             int64_t n, int64_t tq, int64_t tk, int64_t q_offset, int d, float scale,
                             float* rmax, float* rden, void* out, void* stream);

/* Pass 2 — per-(query-block, key-block) column sums of p and their exclusive
 * scan over query blocks, in one key-stationary sweep.
 * Replaces _dilution_k1's sweep 2 (kernels.py:190-198) + _dilution_scan (:250-264).
 * carry_base: optional (n, tk) fp32 demand already committed by earlier query
 *   chunks (sequence-parallel ranks), or NULL.
 * carry: (n, ceil(tq/carry_rows), tk) fp32 out.
 * total: (n, tk) fp32 out, column sums of p over the LOCAL rows (the decode
 *   accumulator `committed_total`, kernels.py:451-453, when tq covers the sequence). */
int dilution_colsum_scan(const void* q, const void* k, int dtype, int precision,
                         int64_t n, int64_t tq, int64_t tk, int64_t q_offset, int d, float scale,
                         const float* rmax, const float* rden, const float* carry_base,
                         int carry_rows, float* carry, float* total, void* stream);

/* Pass 3 — main forward pass: rebuild p, committed = carry + in-tile exclusive
 * column cumsum, share = p/(committed+p+eps), out = (share@v)/(rowsum(share)+eps).
 * Replaces _dilution_k2 (kernels.py:266-315); with pk != NULL it also emits
 * pk = scale * p@k (n, tq, d) fp32, which the reference's K1 saves for the
 * backward (kernels.py:161-188).
 * carry_base: optional (n, tk) fp32 added to every carry row on the fly (demand
 *   committed by earlier query chunks, known only after pass 2 ran), or NULL.
 * out: (n, tq, d) fp32.  ssum: (n, tq) fp32 row sums of share. */
int dilution_forward_main(const void* q, const void* k, const void* v, int dtype, int precision,
                          int64_t n, int64_t tq, int64_t tk, int64_t q_offset, int d,
                          float scale, float eps,
                          const float* rmax, const float* rden, const float* carry, int carry_rows,
                          const float* carry_base,
                          float* out, float* ssum, float* pk, void* stream);

/* Bytes of scratch dilution_backward needs (fp32 dq_main, dk_main, ghat, dbar and a
 * bf16 copy of dout). */
/* Passes 2 and 3 of a TRAINING forward in one key-stationary sweep (the reference's training
 * forward does the same: _dilution_key_forward + _dilution_normalize, kernels.py:200-248):
 * after dilution_rowstats[_pk], writes the checkpoints every 32 query rows (carry:
 * (n, ceil(t/32), t)), the demand totals, out (n, t, d) fp32 and ssum (n, t) that
 * dilution_colsum_scan + dilution_forward_main would write, with one QK^T sweep and one
 * exponential per score less.  The per-key demand is a register for the whole sweep; the
 * output tiles of the key blocks are added to `out` by tensor reductions (out and ssum are
 * zeroed first, on the stream), so the summation order of `out` across key blocks is not
 * fixed.  bf16 tensors, DILUTION_PREC_BF16, head_dim 64, whole sequences (tq = tk, no offset)
 * only: DILUTION_ERR_UNSUPPORTED otherwise. */
int dilution_forward_fused(const void* q, const void* k, const void* v, int dtype, int precision, int64_t n,
                           int64_t t, int d, float scale, float eps, const float* rmax, const float* rden,
                           float* carry, float* total, float* out, float* ssum, void* stream);

size_t dilution_backward_scratch_bytes(int64_t n, int64_t t, int d);

/* Pass 4 — backward of the whole operator.
 * Replaces torch dbar (kernels.py:866), _dilution_ba (:677-775), _dilution_bc
 * (:777-809) and _dilution_dq_epilogue (:814-826).
 * out: (n, t, d) fp32.  dout: (n, t, d) in `dout_dtype` — fp32 as autograd hands it
 * over (kernels.py:860-866), or bf16 when the upstream gradient already is (tensor-core
 * path only; halves what a host-resident caller has to copy in).  rmax, rden, ssum: (n, t).  carry and total as written
 * by dilution_colsum_scan with tq == tk == t, q_offset == 0, carry_base == NULL.
 * pk as written by dilution_forward_main or dilution_rowstats_pk; it may be NULL for bf16
 * inputs with BF16 precision and d == 64 (the tensor-core backward then recomputes the dq correction
 * itself).  scratch: dilution_backward_scratch_bytes.
 * dq, dk, dv: (n, t, d) in `dtype` (the input dtype, as kernels.py:873-875). */
int dilution_backward(const void* q, const void* k, const void* v, int dtype, int precision,
                      int64_t n, int64_t t, int d, float scale, float eps,
                      const void* dout, int dout_dtype, const float* out,
                      const float* rmax, const float* rden, const float* carry, int carry_rows,
                      const float* total, const float* ssum, const float* pk,
                      void* scratch, void* dq, void* dk, void* dv, void* stream);

/* Bytes of scratch dilution_decode needs for n rows at this `length`. */
size_t dilution_decode_scratch_bytes(int64_t n, int64_t length, int d);

/* Pass 5 — one cached decode step for every (batch, head) row.
 * Replaces dilution_decode_step / _dilution_decode (kernels.py:936-1038).
 * q1: (n, d).  k_cache, v_cache: contiguous (n, capacity, d) in `dtype` with the
 * new token already at length-1.  committed: (n, capacity) fp32, advanced IN
 * PLACE on [0, length) (+= p); rows >= length of every buffer are never touched.
 * out: (n, d) in `dtype`. */
int dilution_decode(const void* q1, const void* k_cache, const void* v_cache, int dtype,
                    int64_t n, int64_t capacity, int64_t length, int d, float scale, float eps,
                    float* committed, void* out, void* scratch, void* stream);

/* The same step with the token append fused in: replaces the model's _append_kv
 * (model.py:85-93) followed by dilution_decode_step (kernels.py:994-1038), so a token
 * costs three launches and no separate copy.  k1, v1: (n, d) rows of the new token in
 * `dtype`; the kernels write them to position length-1 of k_cache / v_cache (which they
 * therefore take as writable) and use them from registers; the demand at length-1 is
 * taken as zero whatever the buffer holds (a new key has none) and set to this step's p.
 * `length` counts the new token, as in dilution_decode.  Everything else as there. */
int dilution_decode_append(const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                           int dtype, int64_t n, int64_t capacity, int64_t length, int d, float scale,
                           float eps, float* committed, void* out, void* scratch, void* stream);

/* The cached step of a softmax layer on the same streaming kernels: attention of one new
 * token per row over `length` cached keys, the token's k1, v1 rows written to position
 * length-1 on the way.  Replaces CausalSelfAttention.step_cache's _append_kv +
 * F.scaled_dot_product_attention over the cache (model.py:112-117).  k1 and v1 may both be
 * NULL when the token is already in the caches.  scratch: dilution_decode_scratch_bytes.
 * out: (n, d) in `dtype`. */
int dilution_softmax_decode_append(const void* q1, const void* k1, const void* v1, void* k_cache,
                                   void* v_cache, int dtype, int64_t n, int64_t capacity, int64_t length,
                                   int d, float scale, void* out, void* scratch, void* stream);

/* Head split of the fused q/k/v projection with rotary position embedding applied on the way
 * (model.py:59-67 + rope.py:26-44), and its transpose for the backward.
 * qkv: (batch, seq, 3, heads, d) bf16.  q, k, v: contiguous (batch, heads, seq, d) bf16.
 * cos_table, sin_table: (seq, d/2) bf16 for the positions of the rows, built as the reference
 * builds them (fp32 angles cast to bf16), or both NULL for no rotation; q and k are rotated,
 * v is moved.  inverse == 0: qkv -> q, k, v.  inverse != 0: (dq, dk, dv) -> dqkv with the
 * inverse rotation.  d in {32, 64, 128}. */
int dilution_split_heads_rope(void* qkv, void* q, void* k, void* v, const void* cos_table,
                              const void* sin_table, int64_t batch, int64_t seq, int heads, int d,
                              int inverse, void* stream);

/* The same decode step for callers that cannot hand over scratch memory.
 * No counterpart in the reference (its decode allocates out and scratch with
 * torch on every call, kernels.py:1029-1030).
 *
 * Who needs this: a serving process that gave the whole device heap to its own
 * KV-cache pool at start-up, so a later cudaMalloc fails or fragments the pool;
 * a token loop in which an allocation would stall the device; a host that binds
 * this C ABI from a language without a device allocator at hand.  For them the
 * step's scratch (the per-key scores and the per-chunk partial results) lives
 * in one array inside the library image, DILUTION_DECODE_STATIC_BYTES (~17 MB)
 * of device memory on every GPU that loads the library, held until exit.  The
 * call allocates nothing: no cudaMalloc/cudaFree, no library allocator.
 *
 * Limits: n <= DILUTION_DECODE_STATIC_MAX_ROWS and
 * n * round_up(length, 32) <= DILUTION_DECODE_STATIC_MAX_KEYS (e.g. 128 rows at
 * 16K keys, or 16 rows at 128K keys); anything larger is refused with
 * DILUTION_ERR_ARG and a message.  Arguments are those of dilution_decode
 * without `scratch`; results are identical to it.
 *
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and caches it; make that
 * first call before starting any stream capture.  All calls on a device share
 * the one array: it keeps the previous call's contents (nothing in it needs to
 * start at zero — every entry read in a step was written earlier in that step),
 * and two calls that overlap on the GPU (different streams, no ordering) race
 * on it.  Serialise them, or use dilution_decode with separate scratch. */
#define DILUTION_DECODE_STATIC_MAX_ROWS 128
#define DILUTION_DECODE_STATIC_MAX_KEYS (1 << 21)
#define DILUTION_DECODE_STATIC_BYTES \
  (4u * DILUTION_DECODE_STATIC_MAX_KEYS + 4u * DILUTION_DECODE_STATIC_MAX_ROWS * 128u * (2u + 128u + 1u))
int dilution_decode_static(const void* q1, const void* k_cache, const void* v_cache, int dtype,
                           int64_t n, int64_t capacity, int64_t length, int d, float scale, float eps,
                           float* committed, void* out, void* stream);

/* ---- cached steps for a captured graph -------------------------------------------------
 * A CUDA graph freezes the arguments of the launches it records, and a decode step's launches
 * take the cache length (grid, chunking) and the token's position (RoPE table row) as host
 * scalars.  These three entries read both from ONE int in device memory instead —
 * *position_dev = the new token's position = the number of keys already cached — so the
 * per-token layer loop of the model (model.py:464-470) can be captured once and replayed per
 * token, with a one-element increment of that int recorded at the end of the step.  The launch
 * geometry is that of a full cache: the scratch is dilution_decode_scratch_bytes(n, capacity, d),
 * chunks behind the last key write neutral statistics and return.  The caller guarantees
 * 0 <= *position_dev < capacity; a value outside is held at the nearest row (the step then
 * rewrites that row: a wrong result, never an access outside the cache or the tables).
 *   dilution_decode_append_at          dilution_decode_append with length = *position_dev + 1
 *   dilution_softmax_decode_append_at  dilution_softmax_decode_append likewise (k1, v1 required)
 *   dilution_split_heads_rope_at       the head split of ONE token per batch row (seq = 1) whose
 *                                      rotation uses row *position_dev of cos / sin tables of
 *                                      table_rows rows (every position up to the capacity) */
int dilution_decode_append_at(const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                              int dtype, int64_t n, int64_t capacity, const int* position_dev, int d,
                              float scale, float eps, float* committed, void* out, void* scratch,
                              void* stream);
int dilution_softmax_decode_append_at(const void* q1, const void* k1, const void* v1, void* k_cache,
                                      void* v_cache, int dtype, int64_t n, int64_t capacity,
                                      const int* position_dev, int d, float scale, void* out, void* scratch,
                                      void* stream);
int dilution_split_heads_rope_at(void* qkv, void* q, void* k, void* v, const void* cos_table,
                                 const void* sin_table, int64_t table_rows, int64_t batch, int heads,
                                 int d, const int* position_dev, void* stream);

/* ---- share / bid variants ------------------------------------------------------------
 * The ablations a model configuration can select besides the operator itself
 * (config.py:68-72; kernels_bid.py of the reference, generated from kernels.py with
 * three more arguments):
 *   bid    DILUTION_BID_SOFTMAX  p = causal softmax of the scaled scores (the operator);
 *          DILUTION_BID_RELU, _RELU2, _SOFTPLUS, _MINSHIFT
 *                                p = f(a) / rowsum(f) with f = relu(a), relu(a)^2, softplus(a),
 *                                a - rowmin(a) (the minimum is a constant in the backward); a row
 *                                without mass bids uniformly over its causal window, with a zero
 *                                Jacobian (kernels_bid.py:5-10, 27-33, 206-225);
 *          DILUTION_BID_SIGMOID  p = sigmoid of the scaled score, element-wise, no row
 *                                statistics and no Jacobian correction (kernels_bid.py:196-198);
 *          DILUTION_BID_EXPSHIFT p = exp(a) / shift, softmax's exponential without the row sum
 *                                (kernels_bid.py:199-201);
 *          DILUTION_BID_SIGSHIFT p = exp(a) / (exp(a) + shift) = sigmoid(a - log shift)
 *                                (kernels_bid.py:202-204); `shift` > 0 is read by these two only
 *                                (the model passes its context length, model.py:152-156);
 *   share  INCLUSIVE  share = p / (committed + p + eps)   (the operator);
 *          EXCLUSIVE  share = p / (committed + eps)       (earlier queries' demand only);
 *          NONE       share = p                           (no share step: out = p v / rowsum p).
 * bf16 tensors of head_dim 64 under DILUTION_PREC_BF16 run on the tcgen05 kernels, instantiated
 * for the bid and share step (softmax and the three element-wise bids); every other dtype,
 * precision and head_dim, and the four f(a) / rowsum(f) bids always, on the fp32 tile kernels
 * (IEEE: fp32 FMAs; otherwise tf32 tensor-core products).  Checkpoints every
 * DILUTION_CARRY_ROWS query rows.
 *
 * dilution_variant_forward: all forward passes of one call (kernels_bid.py:424-489):
 * rmax, rden (n, t) — row statistics of the bids that divide by a row sum (softmax: exponent and
 * sum; f(a) / rowsum(f): the row minimum for minshift, else 0, and the row's mass), may be NULL
 * for the element-wise bids; carry
 * (n, ceil(t/32), t); total (n, t) = column totals of p (the decode accumulator after this
 * prefix) — with DILUTION_SHARE_NONE carry and total may both be NULL and the column-sum
 * pass is skipped; out (n, t, d) fp32; ssum (n, t); pk (n, t, d) fp32 or NULL — sum_j p_ij k_j * scale,
 * which dilution_variant_backward needs for the softmax bid with a share step (without one
 * the Jacobian correction vanishes identically and pk is not read; the f(a) / rowsum(f) bids,
 * whose Jacobian factor 1 / mass is unbounded, find ghat in a sweep of its own and subtract it
 * before the factor multiplies, kernels_bid.py:718, so they read no pk either).
 * dilution_variant_backward: dq, dk, dv in the input dtype from an fp32 dout
 * (kernels_bid.py:731-815), given what the forward wrote; scratch of
 * dilution_backward_scratch_bytes(n, t, d).
 * dilution_variant_decode: one cached token (kernels_bid.py:853-1012); k1 / v1 (n, d) are
 * the new token's rows to append at position length-1, or both NULL when the caller has
 * written them; committed advances by p in place for every variant; scratch of
 * dilution_decode_scratch_bytes(n, length, d). */
int dilution_variant_forward(const void* q, const void* k, const void* v, int dtype, int precision, int64_t n,
                             int64_t t, int d, float scale, float eps, int bid, int share, float shift, float* rmax,
                             float* rden, float* carry, float* total, float* out, float* ssum, float* pk,
                             void* stream);
int dilution_variant_backward(const void* q, const void* k, const void* v, int dtype, int precision, int64_t n,
                              int64_t t, int d, float scale, float eps, int bid, int share, float shift, const float* dout,
                              const float* out, const float* rmax, const float* rden, const float* carry,
                              const float* total, const float* ssum, const float* pk, void* scratch, void* dq,
                              void* dk, void* dv, void* stream);
int dilution_variant_decode(const void* q1, const void* k1, const void* v1, void* k_cache, void* v_cache,
                            int dtype, int64_t n, int64_t capacity, int64_t length, int d, float scale,
                            float eps, int bid, int share, float shift, float* committed, void* out, void* scratch,
                            void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DILUTION_B200_H */
