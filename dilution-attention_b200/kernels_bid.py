"""Host-side mirror of the reference's `dilution.kernels_bid`: dilution attention with a
selectable bid function and share step (kernels_bid.py:1-43), the module the reference's
model binds instead of `dilution.kernels` whenever its configuration selects an ablation
(model.py:142-156).

    bid           "softmax"   p = causal softmax of the scaled scores       (the operator)
                  "relu", "relu2", "softplus", "minshift"
                              p = f(a) / rowsum(f) with f = relu(a), relu(a)^2, softplus(a),
                              a - rowmin(a); a row without mass bids uniformly
                  "sigmoid"   p = sigmoid of the scaled score, element-wise, no row sum
                  "expshift"  p = exp(a) / shift: softmax's exponential without the row sum
                  "sigshift"  p = exp(a) / (exp(a) + shift) = sigmoid(a - log shift)
    share_cumsum  True         share = p / (committed + p + eps)           (the operator)
                  "exclusive"  share = p / (committed + eps): earlier queries' demand only
                  False        no share step: out = p v / rowsum(p)

Same entry points and keyword arguments as the reference module (`bid`, `share_cumsum`,
`shift` after the arguments of `dilution.kernels`); `shift` is read by the two shifted bids only
(the model passes its context length, model.py:152-156).  The operator itself (softmax, True) is handed to
`kernels.py`; every other combination goes through the C ABI's dilution_variant_* calls: the
tcgen05 kernels instantiated for the bid and share step for bf16 tensors of head_dim 64 under
"bf16" (softmax and the three element-wise bids), the fp32 tile kernels otherwise (fp32 FMAs for
"ieee", tf32 tensor-core products else; the four f(a) / rowsum(f) bids always).
"""

from __future__ import annotations

import math

import torch

from . import _lib
from . import kernels as K

EPS = K.EPS
HAS_TRITON = False
BID_TYPES = ("softmax", "relu", "relu2", "softplus", "minshift", "sigmoid", "expshift", "sigshift")
BUILT_BIDS = BID_TYPES

_resolve_precision = K._resolve_precision


def _bid_code(bid: str) -> int:
    """Code of a bid function (kernels_bid.py:88-91); ValueError for names the reference does not
    know."""
    if bid not in BID_TYPES:
        raise ValueError(f"bid must be one of {BID_TYPES}")
    if bid not in BUILT_BIDS:
        raise ValueError(f"bid {bid!r} is not built in this backend (built: {BUILT_BIDS})")
    return _lib.BID[bid]


def _share_code(share_cumsum) -> int:
    """True/1 -> inclusive dilution, "exclusive" -> earlier queries only, False/0 -> none
    (kernels_bid.py:123-127)."""
    if share_cumsum == "exclusive":
        return 2
    return int(bool(share_cumsum))


def _is_operator(bid: str, share_cumsum) -> bool:
    return bid == "softmax" and _share_code(share_cumsum) == 1


def _variant_forward(q, k, v, dot_precision, bid, share, shift, save_pk, scratch_budget_gib=16.0,
                     keep_carry=False, need_total=True):
    """All forward passes of one call, (batch*head) rows in slabs under the scratch budget unless
    the checkpoints are kept for a backward.  Without a share step nothing reads the checkpoints:
    unless the demand totals are asked for, the column-sum pass is skipped altogether."""
    lib = _lib.load()
    (qf, kf, vf), code, prec, n = K._prepare(q, k, v, dot_precision)
    batch, heads, seq, head_dim = q.shape
    f32 = dict(device=q.device, dtype=torch.float32)
    stats = bid in _lib.ROW_SUM_BIDS       # bids that divide by a row sum have row statistics
    out = torch.empty(n, seq, head_dim, **f32)
    ssum = torch.empty(n, seq, **f32)
    scan = share != 0 or need_total
    total = torch.empty(n, seq, **f32) if scan else None
    rmax = torch.empty(n, seq, **f32) if stats else None
    rden = torch.empty(n, seq, **f32) if stats else None
    pk = torch.empty(n, seq, head_dim, **f32) if (save_pk and bid == _lib.BID["softmax"]) else None
    ncb = (seq + _lib.CARRY_ROWS - 1) // _lib.CARRY_ROWS
    rows = n
    if not keep_carry:
        rows = max(1, min(n, int(scratch_budget_gib * 2**30) // max(ncb * seq * 4, 1)))
    carry = torch.empty(rows, ncb, seq, **f32) if scan else None
    scale = 1.0 / math.sqrt(head_dim)
    st = K._stream(q.device)
    part = lambda x, a, b: None if x is None else x[a:b].data_ptr()
    for a in range(0, n, rows):
        b = min(a + rows, n)
        _lib.check(lib.dilution_variant_forward(
            qf[a:b].data_ptr(), kf[a:b].data_ptr(), vf[a:b].data_ptr(), code, prec, b - a, seq, head_dim,
            scale, EPS, bid, share, float(shift), part(rmax, a, b), part(rden, a, b), K._ptr(carry), part(total, a, b),
            out[a:b].data_ptr(), ssum[a:b].data_ptr(), part(pk, a, b), st), "dilution_variant_forward")
    return out, dict(rmax=rmax, rden=rden, carry=carry, ssum=ssum, pk=pk, total=total)


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
    bid: str = "softmax",
    share_cumsum=True,
    shift: float = 1.0,
):
    """Fused forward, fp32 (B, H, T, D) (kernels_bid.py:424-489).  With return_aux also the
    aux dict of the reference: rmax, rden (None for the sigmoid bid), carry, ssum, the tuning
    arguments, bid, share_cumsum, shift and committed_total (B, H, T) fp32: the column totals of
    p, the cached-decode accumulator after this prefix."""
    code_b, code_s = _bid_code(bid), _share_code(share_cumsum)
    _resolve_precision(dot_precision)
    if _is_operator(bid, share_cumsum):
        res = K.dilution_attention_forward(q, k, v, dot_precision=dot_precision, block_m=block_m, block_n=block_n,
                                           return_aux=return_aux, num_warps=num_warps, num_stages=num_stages)
        if return_aux:
            res[1].update(bid=bid, share_cumsum=share_cumsum, shift=shift)
        return res
    batch, heads, seq, head_dim = q.shape
    out, aux = _variant_forward(q, k, v, dot_precision, code_b, code_s, shift, save_pk=False,
                                keep_carry=return_aux, need_total=return_aux)
    result = out.reshape(batch, heads, seq, head_dim)
    if return_aux:
        return result, dict(rmax=aux["rmax"], rden=aux["rden"], carry=aux["carry"], ssum=aux["ssum"],
                            block_m=block_m, block_n=block_n, dot_precision=dot_precision, num_warps=num_warps,
                            bwd_block_m=_lib.CARRY_ROWS, bid=bid, share_cumsum=share_cumsum, shift=shift,
                            committed_total=aux["total"].reshape(batch, heads, seq))
    return result


class _VariantFn(torch.autograd.Function):
    """Autograd op of the variants (kernels_bid.py:731-815): fp32 output; dq, dk, dv in the
    input dtypes."""

    @staticmethod
    def forward(ctx, q, k, v, dot_precision, bid, share, shift):
        training = any(ctx.needs_input_grad[:3])
        # without a share step the softmax bid's Jacobian correction is identically zero: no pk
        out, aux = _variant_forward(q, k, v, dot_precision, bid, share, shift, save_pk=training and share != 0,
                                    keep_carry=True, need_total=False)
        ctx.args = (dot_precision, bid, share, shift)
        stats = [x for x in (aux["rmax"], aux["rden"]) if x is not None]
        ctx.n_stats = len(stats)
        ctx.has_pk = aux["pk"] is not None
        if ctx.has_pk:
            stats.append(aux["pk"])
        scan = [x for x in (aux["carry"], aux["total"]) if x is not None]
        ctx.n_scan = len(scan)
        ctx.save_for_backward(q, k, v, out, aux["ssum"], *scan, *stats)
        return out.reshape(q.shape)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, ssum, *rest = ctx.saved_tensors
        carry, total = rest[:2] if ctx.n_scan == 2 else (None, None)
        stats = rest[ctx.n_scan:]
        rmax, rden = stats[:2] if ctx.n_stats == 2 else (None, None)
        pk = stats[-1] if ctx.has_pk else None
        dot_precision, bid, share, shift = ctx.args
        lib = _lib.load()
        batch, heads, seq, head_dim = q.shape
        (qf, kf, vf), code, prec, n = K._prepare(q, k, v, dot_precision)
        dof = dout.reshape(n, seq, head_dim).float().contiguous()
        dq = torch.empty(n, seq, head_dim, device=q.device, dtype=qf.dtype)
        dk, dv = torch.empty_like(dq), torch.empty_like(dq)
        scratch = torch.empty(lib.dilution_backward_scratch_bytes(n, seq, head_dim), device=q.device,
                              dtype=torch.uint8)
        _lib.check(lib.dilution_variant_backward(
            qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), code, prec, n, seq, head_dim, 1.0 / math.sqrt(head_dim),
            EPS, bid, share, float(shift), dof.data_ptr(), out.data_ptr(), K._ptr(rmax), K._ptr(rden), K._ptr(carry),
            K._ptr(total), ssum.data_ptr(), K._ptr(pk), scratch.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            K._stream(q.device)), "dilution_variant_backward")
        shape4 = (batch, heads, seq, head_dim)
        return (dq.reshape(shape4).to(q.dtype), dk.reshape(shape4).to(k.dtype), dv.reshape(shape4).to(v.dtype),
                None, None, None, None)


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
    bid: str = "softmax",
    share_cumsum=True,
    shift: float = 1.0,
) -> torch.Tensor:
    """Differentiable fused attention under the selected bid and share step
    (kernels_bid.py:818-849)."""
    code_b, code_s = _bid_code(bid), _share_code(share_cumsum)
    _resolve_precision(dot_precision)
    if _is_operator(bid, share_cumsum):
        return K.dilution_attention(q, k, v, dot_precision=dot_precision)
    return _VariantFn.apply(q, k, v, dot_precision, code_b, code_s, shift)


def dilution_attention_reference(q, k, v, bid: str = "softmax", share_cumsum=True, shift: float = 1.0):
    """The fp32 spec's signature (kernels_bid.py:130-166) on the GPU: inputs cast to fp32, fp32
    FMA products, nothing (T x T)-shaped materialised; differentiable."""
    code_b, code_s = _bid_code(bid), _share_code(share_cumsum)
    if _is_operator(bid, share_cumsum):
        return K.dilution_attention_reference(q, k, v)
    return _VariantFn.apply(q.float(), k.float(), v.float(), "ieee", code_b, code_s, shift)


def dilution_decode_step(
    q1: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    committed: torch.Tensor,
    length: int,
    block_n: int = 512,
    num_warps: int = 8,
    bid: str = "softmax",
    share_cumsum=True,
    shift: float = 1.0,
    scratch: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Fused decode step under the selected bid and share step (kernels_bid.py:962-1012): same
    contract as kernels.dilution_decode_step; `committed` advances by p in place whatever the
    share step."""
    code_b, code_s = _bid_code(bid), _share_code(share_cumsum)
    if _is_operator(bid, share_cumsum):
        return K.dilution_decode_step(q1, k_cache, v_cache, committed, length, scratch=scratch, out=out)
    lib = _lib.load()
    batch, heads, head_dim, capacity = K._decode_args(q1, k_cache, v_cache, committed, length)
    n = batch * heads
    qf = K._rows(q1, n, head_dim)
    if out is None:
        out = torch.empty(n, head_dim, device=q1.device, dtype=q1.dtype)
    need = lib.dilution_decode_scratch_bytes(n, length, head_dim)
    if scratch is None or scratch.numel() * scratch.element_size() < need:
        scratch = torch.empty(need, device=q1.device, dtype=torch.uint8)
    code = _lib.BF16 if q1.dtype == torch.bfloat16 else _lib.F32
    _lib.check(lib.dilution_variant_decode(
        qf.data_ptr(), None, None, k_cache.view(n, capacity, head_dim).data_ptr(),
        v_cache.view(n, capacity, head_dim).data_ptr(), code, n, capacity, length, head_dim,
        1.0 / math.sqrt(head_dim), EPS, code_b, code_s, float(shift), committed.view(n, capacity).data_ptr(),
        out.data_ptr(),
        scratch.data_ptr(), K._stream(q1.device)), "dilution_variant_decode")
    return out.view(batch, heads, 1, head_dim)


_PATCHED = ("dilution_attention_forward", "dilution_attention", "dilution_decode_step")


def install(target=None):
    """Assign the entry points above onto `dilution.kernels_bid` (or `target`): the module the
    reference's DilutionAttention binds when its configuration selects a bid or share step other
    than the operator's (model.py:145-150).  `uninstall()` puts the originals back."""
    if target is None:
        import dilution.kernels_bid as target
    if getattr(target, "_b200_saved", None) is None:
        target._b200_saved = {name: getattr(target, name, None) for name in _PATCHED + ("HAS_TRITON",)}
    for name in _PATCHED:
        setattr(target, name, globals()[name])
    target.HAS_TRITON = True
    return target


def uninstall(target=None):
    if target is None:
        import sys
        target = sys.modules.get("dilution.kernels_bid")
        if target is None:
            return None
    saved = getattr(target, "_b200_saved", None)
    if saved is not None:
        for name, value in saved.items():
            if value is not None:
                setattr(target, name, value)
        del target._b200_saved
    return target
