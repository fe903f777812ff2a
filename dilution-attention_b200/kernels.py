"""Dilution attention on B200: the `dilution.kernels` entry points, unchanged.

Same names, arguments, return values and errors as the reference module
(src/dilution/kernels.py), backed by hand-written sm_100a CUDA kernels in
libdilution_b200.so instead of Triton:

    dilution_attention_reference(q, k, v)                      kernels.py:40-68
    dilution_attention_forward(q, k, v, dot_precision=...,     kernels.py:328-455
                               return_aux=..., _save_pk=...)
    dilution_attention(q, k, v, dot_precision=...)             kernels.py:906-930
    dilution_decode_step(q1, k_cache, v_cache, committed, t)   kernels.py:994-1038
    dilution_decode_append_step(q1, k1, v1, cache)             model.py:85-93 + :236-239
    softmax_attention_forward(q, k, v)                         model.py:96-117 (forward)

The operator (docs/operator.md of the reference):

    p         = causal_softmax(q k^T / sqrt(D))
    committed = exclusive cumsum of p down the query axis, per key
    share     = p / (committed + p + 1e-9)
    out       = (share / (rowsum(share) + 1e-9)) @ v            fp32

Forward = three passes (row statistics; per-key column sums with their
exclusive scan over query blocks; main pass), backward = a reverse key-stationary
pass plus the softmax-Jacobian corrections, decode = a bandwidth-bound streaming
kernel.  All tensors must live on a CUDA device; there is no CPU, Triton or
eager fallback — a missing library raises RuntimeError.

Triton tuning keywords of the reference (block_m, block_n, num_warps, num_stages,
bwd_*, b3_*, b4_*) are accepted and ignored.
"""

from __future__ import annotations

import math
import os

import torch

from . import _lib

EPS = 1e-9                      # kernels.py:66-67 of the reference, twice
CARRY_ROWS = _lib.CARRY_ROWS    # query rows per demand checkpoint of the fp32 kernels
KEY_FORWARD_MIN_SEQ = 256       # read by the reference's scripts; no meaning here
HAS_TRITON = False              # this backend never uses Triton
HAS_CUDA_LIB = _lib.available()
# Training forward on the tensor-core path: pass 1 also saves pk = scale * softmax(q k^T) k (as the
# reference's K1 does, kernels.py:161-188), and the backward's correction pass then has only its
# key half left.  False (or DILUTION_SAVE_PK=0 in the environment): nothing is saved and the
# correction pass recomputes the query half.
TC_SAVE_PK = os.environ.get("DILUTION_SAVE_PK", "1") != "0"
# Training forward on the tensor-core path: one key-stationary sweep for passes 2 and 3
# (dilution_forward_fused) instead of the column-sum pass plus the query-stationary main pass.
TC_FUSED_FORWARD = os.environ.get("DILUTION_FUSED_FORWARD", "1") != "0"


def _resolve_precision(dot_precision: str) -> tuple[int, str]:
    """"ieee": fp32 products; "tf32": tf32 tensor-core products of fp32 operands; "bf16": bf16 tensor-core operands
    (kernels.py:318-325, same return values and error)."""
    if dot_precision == "bf16":
        return 1, "tf32"
    if dot_precision in ("ieee", "tf32"):
        return 0, dot_precision
    raise ValueError("dot_precision must be one of ieee, tf32, bf16")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _prepare(q, k, v, dot_precision):
    """Contiguous (n, t, d) operands in the dtype the kernels take
    (kernels.py:362-364), the dtype code and the precision code."""
    lowp, _ = _resolve_precision(dot_precision)
    if not q.is_cuda:
        raise RuntimeError("dilution attention needs CUDA tensors (no CPU fallback in this backend)")
    batch, heads, seq, head_dim = q.shape
    n = batch * heads
    want = torch.bfloat16 if (lowp or q.dtype == torch.bfloat16) else torch.float32
    ops = []
    for x in (q, k, v):
        if x is None:
            ops.append(None)
            continue
        x = x.reshape(n, x.shape[2], head_dim)
        if x.dtype != want:
            x = x.to(want)
        ops.append(x.contiguous())
    code = _lib.BF16 if want == torch.bfloat16 else _lib.F32
    return ops, code, _lib.PREC[dot_precision], n


def _forward_rows(lib, qf, kf, vf, code, prec, scale, out, ssum, rmax, rden, carry, total, pk,
                  carry_rows, q_offset=0, carry_base=None):
    """Passes 1-3 on a slab of (batch*head) rows.  On the tensor-core path a requested pk comes
    out of pass 1; otherwise out of pass 3 (the fp32 kernel)."""
    n, tq, d = qf.shape
    tk = kf.shape[1]
    st = _stream(qf.device)
    if pk is not None and _lib.tensor_core_path(code, prec, d) and q_offset == 0 and tq == tk:
        _lib.check(lib.dilution_rowstats_pk(qf.data_ptr(), kf.data_ptr(), code, prec, n, tq, d, scale,
                                            rmax.data_ptr(), rden.data_ptr(), pk.data_ptr(), st),
                   "dilution_rowstats_pk")
        pk = None
    else:
        _lib.check(lib.dilution_rowstats(qf.data_ptr(), kf.data_ptr(), code, prec, n, tq, tk, q_offset,
                                         d, scale, rmax.data_ptr(), rden.data_ptr(), st), "dilution_rowstats")
    if (TC_FUSED_FORWARD and carry_rows == 32 and carry_base is None and q_offset == 0 and tq == tk
            and _lib.tensor_core_path(code, prec, d)):
        _lib.check(lib.dilution_forward_fused(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), code, prec, n, tq, d,
                                              scale, EPS, rmax.data_ptr(), rden.data_ptr(), carry.data_ptr(),
                                              total.data_ptr(), out.data_ptr(), ssum.data_ptr(), st),
                   "dilution_forward_fused")
        return
    _lib.check(lib.dilution_colsum_scan(qf.data_ptr(), kf.data_ptr(), code, prec, n, tq, tk, q_offset,
                                        d, scale, rmax.data_ptr(), rden.data_ptr(), None, carry_rows,
                                        carry.data_ptr(), total.data_ptr(), st), "dilution_colsum_scan")
    _lib.check(lib.dilution_forward_main(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), code, prec,
                                         n, tq, tk, q_offset, d, scale, EPS,
                                         rmax.data_ptr(), rden.data_ptr(), carry.data_ptr(), carry_rows,
                                         _ptr(carry_base), out.data_ptr(), ssum.data_ptr(), _ptr(pk), st),
               "dilution_forward_main")


def dilution_attention_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dot_precision: str = "ieee",
    block_m: int = 64,
    block_n: int = 64,
    return_aux: bool = False,
    num_warps: int = 4,
    num_stages: int = 2,
    _save_pk: bool = False,
    scratch_budget_gib: float = 16.0,
    _training: bool | None = None,
):
    """Fused forward; returns fp32 (B, H, T, D)  (kernels.py:328-455).

    With return_aux=True also returns the aux dict of the reference: pk (or
    None), rmax, rden, carry, ssum, bwd_block_m, block_m, block_n,
    dot_precision, num_warps and committed_total (B, H, T) fp32 — the inclusive
    column totals of p, i.e. the decode accumulator after this prefix.
    `carry` holds one per-key demand checkpoint every aux["bwd_block_m"] query
    rows; entries for keys a row block cannot see are unwritten.  The spacing
    follows the kernels that will read it: 32 rows when a backward will follow and
    on the fp32 kernels, 64 for forward-only calls of the tensor-core kernels (the
    reference stores every 32 or 64 in the same way, kernels.py:374-377).

    Without return_aux the (batch*head) rows are processed in slabs so that the
    quadratic carry scratch stays under scratch_budget_gib; rows are independent,
    so this changes nothing numerically.
    """
    lib = _lib.load()
    (qf, kf, vf), code, prec, n = _prepare(q, k, v, dot_precision)
    batch, heads, seq, head_dim = q.shape
    dev = q.device
    scale = 1.0 / math.sqrt(head_dim)
    training = _save_pk if _training is None else _training
    carry_rows = _lib.carry_rows(code, prec, head_dim, training)
    ncb = (seq + carry_rows - 1) // carry_rows

    f32 = dict(device=dev, dtype=torch.float32)
    out = torch.empty(n, seq, head_dim, **f32)
    pk = torch.empty(n, seq, head_dim, **f32) if _save_pk else None
    rmax = torch.empty(n, seq, **f32)
    rden = torch.empty(n, seq, **f32)
    ssum = torch.empty(n, seq, **f32)
    total = torch.empty(n, seq, **f32)

    rows = n
    if not return_aux:
        per_row = ncb * seq * 4
        rows = max(1, min(n, int(scratch_budget_gib * 2**30) // max(per_row, 1)))
    carry = torch.empty(rows, ncb, seq, **f32)
    for a in range(0, n, rows):
        b = min(a + rows, n)
        _forward_rows(lib, qf[a:b], kf[a:b], vf[a:b], code, prec, scale, out[a:b], ssum[a:b],
                      rmax[a:b], rden[a:b], carry[: b - a], total[a:b],
                      None if pk is None else pk[a:b], carry_rows)

    result = out.reshape(batch, heads, seq, head_dim)
    if return_aux:
        aux = dict(pk=pk, rmax=rmax, rden=rden, carry=carry, ssum=ssum, bwd_block_m=carry_rows,
                   block_m=block_m, block_n=block_n, dot_precision=dot_precision,
                   num_warps=num_warps,
                   committed_total=total.reshape(batch, heads, seq))
        return result, aux
    return result


class _DilutionAttentionFn(torch.autograd.Function):
    """Autograd op (kernels.py:829-903): fp32 output; dq, dk, dv in the input dtypes."""

    @staticmethod
    def forward(ctx, q, k, v, dot_precision):
        # the tensor-core backward can apply the dq correction itself, without a saved pk
        lowp, _ = _resolve_precision(dot_precision)
        on_tc = _lib.tensor_core_path(_lib.BF16 if (lowp or q.dtype == torch.bfloat16) else _lib.F32,
                                      _lib.PREC[dot_precision], q.shape[-1])
        out, aux = dilution_attention_forward(
            q, k, v, dot_precision=dot_precision, return_aux=True,
            _save_pk=any(ctx.needs_input_grad[:3]) and (TC_SAVE_PK or not on_tc),
            _training=any(ctx.needs_input_grad[:3]))
        ctx.carry_rows = aux["bwd_block_m"]
        ctx.save_for_backward(q, k, v, out, aux["rmax"], aux["rden"], aux["carry"], aux["ssum"], aux["pk"],
                              aux["committed_total"])
        ctx.dot_precision = dot_precision
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, rmax, rden, carry, ssum, pk, total = ctx.saved_tensors
        lib = _lib.load()
        batch, heads, seq, head_dim = q.shape
        (qf, kf, vf), code, prec, n = _prepare(q, k, v, ctx.dot_precision)
        dev = q.device
        # the tensor-core path reads a bf16 upstream gradient as it is (its first kernel makes a
        # scaled bf16 copy anyway); everything else is widened to fp32 as the reference does
        on_tc = _lib.tensor_core_path(code, prec, head_dim)
        dof = dout.reshape(n, seq, head_dim)
        if not (on_tc and dof.dtype == torch.bfloat16):
            dof = dof.float()
        dof = dof.contiguous()
        do_code = _lib.BF16 if dof.dtype == torch.bfloat16 else _lib.F32
        of = out.reshape(n, seq, head_dim)
        gdt = qf.dtype
        dq = torch.empty(n, seq, head_dim, device=dev, dtype=gdt)
        dk = torch.empty_like(dq)
        dv = torch.empty_like(dq)
        nbytes = lib.dilution_backward_scratch_bytes(n, seq, head_dim)
        scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
        _lib.check(lib.dilution_backward(
            qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), code, prec, n, seq, head_dim,
            1.0 / math.sqrt(head_dim), EPS, dof.data_ptr(), do_code, of.data_ptr(),
            rmax.data_ptr(), rden.data_ptr(), carry.data_ptr(), ctx.carry_rows, total.data_ptr(), ssum.data_ptr(),
            _ptr(pk), scratch.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _stream(dev)),
            "dilution_backward")
        shape4 = (batch, heads, seq, head_dim)
        return (dq.reshape(shape4).to(q.dtype), dk.reshape(shape4).to(k.dtype),
                dv.reshape(shape4).to(v.dtype), None)


def dilution_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dot_precision: str = "bf16",
    block_m: int = 64,
    block_n: int = 64,
    num_warps: int = 4,
    bwd_num_warps: int = 4,
    bwd_num_stages: int = 1,
    b3_block_n: int | None = None,
    b3_num_warps: int | None = None,
    b4_num_warps: int | None = 4,
) -> torch.Tensor:
    """Differentiable fused dilution attention (kernels.py:906-930).

    "bf16" (default): bf16 tensor-core operands, fp32 accumulation and fp32
    cumsum/share maths; "tf32": tf32 tensor-core products of fp32 operands; "ieee": fp32 products.
    """
    _resolve_precision(dot_precision)
    return _DilutionAttentionFn.apply(q, k, v, dot_precision)


def dilution_attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """The operator in fp32 with the reference's signature (kernels.py:40-68):
    q/k/v (B, H, T, D) -> (B, H, T, D) fp32, differentiable.

    Inputs are cast to fp32 and every product is an fp32 FMA on the GPU; unlike
    the reference's dense PyTorch version nothing (T x T)-shaped is materialised.
    """
    return _DilutionAttentionFn.apply(q.float(), k.float(), v.float(), "ieee")


def softmax_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, return_lse: bool = False):
    """Causal softmax attention on the same tcgen05 pipeline: what the reference's
    CausalSelfAttention layers compute with F.scaled_dot_product_attention(q, k, v,
    is_causal=True) (model.py:96-117).  Forward only (inference / prefill).

    q, k, v: (B, H, T, 64) bfloat16 on a CUDA device.  Returns (B, H, T, 64) bfloat16 and, with
    return_lse, the natural-log row log-sum-exp of the scaled scores (B, H, T) fp32.
    Pass 1 of dilution attention plus a plain P V product is exactly this operator
    (tests/test_kernels.py:349-357 of the reference shows it for share_cumsum=False).
    """
    lib = _lib.load()
    if not q.is_cuda:
        raise RuntimeError("softmax attention needs CUDA tensors (no CPU fallback in this backend)")
    batch, heads, seq, head_dim = q.shape
    if q.dtype != torch.bfloat16 or head_dim != 64:
        raise ValueError("softmax_attention_forward takes bfloat16 tensors with head_dim 64")
    (qf, kf, vf), code, prec, n = _prepare(q, k, v, "bf16")
    out = torch.empty(n, seq, head_dim, device=q.device, dtype=torch.bfloat16)
    rmax = rden = None
    if return_lse:
        rmax = torch.empty(n, seq, device=q.device, dtype=torch.float32)
        rden = torch.empty_like(rmax)
    _lib.check(lib.dilution_softmax_forward(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), code, prec, n, seq,
                                            kf.shape[1], 0, head_dim, 1.0 / math.sqrt(head_dim), _ptr(rmax),
                                            _ptr(rden), out.data_ptr(), _stream(q.device)),
               "dilution_softmax_forward")
    result = out.reshape(batch, heads, seq, head_dim)
    if return_lse:
        lse = (rmax + torch.log2(rden)) * math.log(2.0)
        return result, lse.reshape(batch, heads, seq)
    return result


def decode_scratch(n: int, capacity: int, head_dim: int, device) -> torch.Tensor:
    """Scratch buffer for dilution_decode_step, big enough for any length up to
    `capacity`.  Reuse it across steps to keep allocation out of the token loop."""
    nbytes = _lib.load().dilution_decode_scratch_bytes(n, capacity, head_dim)
    return torch.empty(nbytes, device=device, dtype=torch.uint8)


def _decode_args(q1, k_cache, v_cache, committed, length):
    """Validation shared by the decode entry points (kernels.py:1012-1021)."""
    batch, heads, one, head_dim = q1.shape
    if one != 1:
        raise ValueError("decode step takes exactly one query row per (batch, head)")
    if head_dim & (head_dim - 1):
        raise ValueError("head_dim must be a power of two")
    capacity = k_cache.shape[2]
    if not 1 <= length <= capacity:
        raise ValueError(f"length {length} outside cache capacity {capacity}")
    if not q1.is_cuda:
        raise RuntimeError("dilution decode needs CUDA tensors (no CPU fallback in this backend)")
    if q1.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("decode supports float32 and bfloat16 caches")
    if k_cache.dtype != q1.dtype or v_cache.dtype != q1.dtype or committed.dtype != torch.float32:
        raise ValueError("caches must have q1's dtype and committed must be float32")
    return batch, heads, head_dim, capacity


def _rows(x, n, head_dim):
    x = x.reshape(n, head_dim)
    return x if x.is_contiguous() else x.contiguous()


def dilution_decode_step(
    q1: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    committed: torch.Tensor,
    length: int,
    block_n: int = 512,
    num_warps: int = 8,
    scratch: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Fused decode step (kernels.py:994-1038).  Returns (B, H, 1, D) in q1.dtype.

    q1: (B, H, 1, D).  k_cache / v_cache: contiguous (B, H, capacity, D) buffers
    whose first `length` positions are valid, the new token already written at
    length-1.  committed: contiguous (B, H, capacity) fp32 accumulator, advanced
    IN PLACE to include this row; positions >= length are never touched.
    `scratch` (from decode_scratch) and `out` ((B*H, D) in q1.dtype) are optional
    caller buffers that keep allocation out of the token loop.
    """
    lib = _lib.load()
    batch, heads, head_dim, capacity = _decode_args(q1, k_cache, v_cache, committed, length)
    n = batch * heads
    qf = _rows(q1, n, head_dim)
    kf = k_cache.view(n, capacity, head_dim)      # .view: the caches must be contiguous
    vf = v_cache.view(n, capacity, head_dim)
    cf = committed.view(n, capacity)
    if out is None:
        out = torch.empty(n, head_dim, device=q1.device, dtype=q1.dtype)
    need = lib.dilution_decode_scratch_bytes(n, length, head_dim)
    if scratch is None or scratch.numel() * scratch.element_size() < need:
        scratch = torch.empty(need, device=q1.device, dtype=torch.uint8)
    code = _lib.BF16 if q1.dtype == torch.bfloat16 else _lib.F32
    _lib.check(lib.dilution_decode(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), code, n, capacity,
                                   length, head_dim, 1.0 / math.sqrt(head_dim), EPS,
                                   cf.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                   _stream(q1.device)), "dilution_decode")
    return out.view(batch, heads, 1, head_dim)


def dilution_decode_append_step(
    q1: torch.Tensor,
    k1: torch.Tensor,
    v1: torch.Tensor,
    cache: dict,
    scratch: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """One cached token with the append fused in: what the model does as
    `_append_kv(cache, k1, v1)` (model.py:85-93) followed by
    `dilution_decode_step(q1, cache["k"], cache["v"], cache["committed"], t)`
    (model.py:236-239), as three kernel launches and no separate copy.

    q1, k1, v1: (B, H, 1, D) of the new token.  cache: the model's dict
    {"k", "v", "len", "committed"} (model.py:76-83, 224-228); its k / v rows at
    position len are written by the kernels, committed is advanced in place and
    cache["len"] grows by one.  Raises ValueError past the capacity, as
    _append_kv does.  Returns (B, H, 1, D) in q1.dtype.

    A cache that carries "pos_dev" (a one-element int32 device tensor holding the new token's
    position, see layers.GraphedDecode) takes the length from there: the launches then have
    the geometry of a full cache and can be recorded into a CUDA graph.
    """
    lib = _lib.load()
    t = cache["len"]
    if t >= cache["k"].shape[2]:
        raise ValueError("decode step past the cache capacity (context_length)")
    k_cache, v_cache, committed = cache["k"], cache["v"], cache["committed"]
    batch, heads, head_dim, capacity = _decode_args(q1, k_cache, v_cache, committed, t + 1)
    if k1.dtype != q1.dtype or v1.dtype != q1.dtype:
        raise ValueError("k1 and v1 must have q1's dtype")
    n = batch * heads
    qf, kn, vn = (_rows(x, n, head_dim) for x in (q1, k1, v1))
    kf = k_cache.view(n, capacity, head_dim)
    vf = v_cache.view(n, capacity, head_dim)
    cf = committed.view(n, capacity)
    pos_dev = cache.get("pos_dev")
    if out is None:
        out = torch.empty(n, head_dim, device=q1.device, dtype=q1.dtype)
    need = lib.dilution_decode_scratch_bytes(n, capacity if pos_dev is not None else t + 1, head_dim)
    if scratch is None or scratch.numel() * scratch.element_size() < need:
        scratch = torch.empty(need, device=q1.device, dtype=torch.uint8)
    code = _lib.BF16 if q1.dtype == torch.bfloat16 else _lib.F32
    if pos_dev is not None:
        _lib.check(lib.dilution_decode_append_at(qf.data_ptr(), kn.data_ptr(), vn.data_ptr(), kf.data_ptr(),
                                                 vf.data_ptr(), code, n, capacity, pos_dev.data_ptr(), head_dim,
                                                 1.0 / math.sqrt(head_dim), EPS, cf.data_ptr(), out.data_ptr(),
                                                 scratch.data_ptr(), _stream(q1.device)), "dilution_decode_append_at")
    else:
        _lib.check(lib.dilution_decode_append(qf.data_ptr(), kn.data_ptr(), vn.data_ptr(), kf.data_ptr(),
                                              vf.data_ptr(), code, n, capacity, t + 1, head_dim,
                                              1.0 / math.sqrt(head_dim), EPS, cf.data_ptr(), out.data_ptr(),
                                              scratch.data_ptr(), _stream(q1.device)), "dilution_decode_append")
    cache["len"] = t + 1
    return out.view(batch, heads, 1, head_dim)


_COPY_STREAMS: dict = {}


def _copy_streams(device):
    """The copy-in and copy-out streams of a device, created once: the caching allocator keeps
    a pool per stream, so fresh streams on every call would never find a cached block."""
    key = (device.type, device.index)
    if key not in _COPY_STREAMS:
        _COPY_STREAMS[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
    return _COPY_STREAMS[key]


def dilution_attention_host(q, k, v, dout=None, dot_precision: str = "bf16", device=None, slabs: int = 8,
                            out=None, grads=None, wait: bool = True):
    """The operator for tensors that live in HOST memory (ideally pinned).

    q, k, v: (B, H, T, D) CPU tensors; dout: optional (B, H, T, D) upstream gradient.
    Returns out (fp32, CPU) and, when dout is given, (out, dq, dk, dv) with the
    gradients in the input dtypes.  `out` / `grads` may be preallocated (pinned)
    result buffers.

    The (batch*head) rows are independent, so the call is cut into `slabs` row
    slabs that flow through three CUDA streams: host->device copy of slab i+1,
    forward+backward of slab i and device->host copy of slab i-1 run at the same
    time.  End-to-end time approaches max(compute, one copy direction) instead of
    their sum.  The maths and kernels are those of `dilution_attention`.  dout
    may be bf16 (a bf16 model's upstream gradient): it is then copied and used as
    it is, which halves that part of the host->device traffic.

    With wait=True (default) the call returns once the results are in the host
    buffers.  wait=False returns as soon as everything is queued; the caller must
    then synchronise the device (or the current stream) before reading them.
    """
    lib_device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    batch, heads, seq, head_dim = q.shape
    n = batch * heads
    slabs = max(1, min(slabs, n))
    bounds = [n * i // slabs for i in range(slabs + 1)]
    qh, kh, vh = (x.reshape(n, 1, seq, head_dim) for x in (q, k, v))
    doh = None if dout is None else dout.reshape(n, 1, seq, head_dim)
    if out is None:
        out = torch.empty(batch, heads, seq, head_dim, dtype=torch.float32, pin_memory=True)
    oh = out.reshape(n, 1, seq, head_dim)
    if dout is not None and grads is None:
        grads = tuple(torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in (q, k, v))
    gh = None if dout is None else tuple(x.reshape(n, 1, seq, head_dim) for x in grads)

    main = torch.cuda.current_stream(lib_device)
    s_in, s_out = _copy_streams(lib_device)
    s_in.wait_stream(main)
    staged, done = [], []

    def stage(i):
        a, b = bounds[i], bounds[i + 1]
        with torch.cuda.stream(s_in):
            bufs = [x[a:b].to(lib_device, non_blocking=True) for x in (qh, kh, vh)]
            bufs.append(None if doh is None else doh[a:b].to(lib_device, non_blocking=True))
            ev = torch.cuda.Event()
            ev.record(s_in)
        return bufs, ev

    staged.append(stage(0))
    for i in range(slabs):
        a, b = bounds[i], bounds[i + 1]
        if i + 1 < slabs:
            staged.append(stage(i + 1))
        (qd, kd, vd, dd), ev = staged[i]
        main.wait_event(ev)
        if dd is None:
            od = dilution_attention_forward(qd, kd, vd, dot_precision=dot_precision)
            res = (od,)
        else:
            qd, kd, vd = (x.requires_grad_(True) for x in (qd, kd, vd))
            od = dilution_attention(qd, kd, vd, dot_precision=dot_precision)
            od.backward(dd)
            res = (od.detach(), qd.grad, kd.grad, vd.grad)
        for x in (qd, kd, vd, dd) + res:
            if x is not None:
                x.record_stream(main)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ready)
            oh[a:b].copy_(res[0], non_blocking=True)
            if dd is not None:
                for dst, src in zip(gh, res[1:]):
                    dst[a:b].copy_(src, non_blocking=True)
            for x in res:
                x.record_stream(s_out)
        staged[i] = None
    main.wait_stream(s_out)
    if wait:
        s_out.synchronize()       # the device->host copies are asynchronous: the host waits for them here
    return out if dout is None else (out, *grads)


def _fused_step_cache(self, x1, cache):
    """DilutionAttention.step_cache (model.py:231-240) with the append fused into
    the decode launch; falls back to the model's own method whenever that one
    would not take the kernel path."""
    if not self._kernel_ok(x1) or not self._standard():
        return self._unfused_step_cache(x1, cache)
    batch = x1.shape[0]
    if cache.get("pos_dev") is not None:       # the position lives on the device (a captured step)
        from . import layers
        q1, k1, v1 = layers.split_heads_at(self, x1, cache)
    else:
        q1, k1, v1 = self._split_heads(x1, offset=cache["len"])
    y = dilution_decode_append_step(q1, k1, v1, cache).to(q1.dtype)
    return self._merge_heads(y, batch, 1)


def install(target=None, fused_decode: bool = False):
    """Plug this backend into the reference package: assign the fused entry
    points onto `dilution.kernels` (or `target`), the same way the reference's
    scripts/train_kernel_variant.py:39 swaps implementations.  The model looks
    the functions up at call time (model.py:145-150), so DilutionLM then runs on
    these kernels after enable_dilution_kernel().

    fused_decode=True also replaces `DilutionAttention.step_cache` of the
    imported `dilution.model` with a version that hands the new token's k and v
    to the decode kernels instead of writing them into the caches first
    (model.py:85-93): one torch copy pair less per layer and token.  The original
    method stays reachable and is used whenever the kernel path does not apply.
    `uninstall()` undoes both.
    """
    if target is None:
        import dilution.kernels as target  # the reference package, if importable
    saved = getattr(target, "_b200_saved", None)
    if saved is None:
        saved = {name: getattr(target, name, None)
                 for name in ("dilution_attention_forward", "dilution_attention", "dilution_decode_step",
                              "HAS_TRITON")}
        target._b200_saved = saved
    for name in ("dilution_attention_forward", "dilution_attention", "dilution_decode_step"):
        setattr(target, name, globals()[name])
    target.HAS_TRITON = True   # the reference gates its kernel path on this flag
    if getattr(target, "__name__", "") == "dilution.kernels":
        from . import kernels_bid      # the module the model binds for the bid / share ablations
        kernels_bid.install()
    if fused_decode:
        import dilution.model as model
        cls = model.DilutionAttention
        if not hasattr(cls, "_unfused_step_cache"):
            cls._unfused_step_cache = cls.step_cache
            cls.step_cache = _fused_step_cache
    return target


def uninstall(target=None):
    """Put back what install() replaced."""
    if target is None:
        import dilution.kernels as target
    saved = getattr(target, "_b200_saved", None)
    if saved is not None:
        for name, value in saved.items():
            if value is not None:
                setattr(target, name, value)
        del target._b200_saved
    import sys
    if getattr(target, "__name__", "") == "dilution.kernels":
        from . import kernels_bid
        kernels_bid.uninstall()
    model = sys.modules.get("dilution.model")
    if model is not None and hasattr(model.DilutionAttention, "_unfused_step_cache"):
        model.DilutionAttention.step_cache = model.DilutionAttention._unfused_step_cache
        del model.DilutionAttention._unfused_step_cache
    return target
