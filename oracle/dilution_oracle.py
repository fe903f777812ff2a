"""CPU oracle for dilution attention.  TEST INFRASTRUCTURE ONLY.

This module is a plain restatement, on the CPU, of the reference operator in
`src/dilution/kernels.py:40-68` (the fp32 spec `dilution_attention_reference`),
of its bid / share variants in `src/dilution/kernels_bid.py:94-166` (softmax,
sigmoid, expshift and sigshift bids; inclusive, exclusive and absent share step) and of the eager
cached-decode step in `src/dilution/model.py:242-257`.  Only
the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import it; the product path never does, and it raises when the CUDA library is
missing rather than falling back to anything here.

Pinning: `tests/golden/make_golden.py` imports the unmodified reference and
stores its outputs and autograd gradients for seeded inputs;
`tests/test_oracle.py` checks every function below against those fixtures, so
parity of this oracle is pinned to the reference itself.

All functions take and return torch CPU tensors.  Arithmetic is fp32 unless the
caller passes fp64 tensors to `dilution_dense`, which is used to measure the
fp32 reference's own rounding error.
"""

from __future__ import annotations

import math

import torch

EPS = 1e-9  # hard-coded twice in the reference: kernels.py:66 and :67


def dilution_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """The operator, densely, line for line as kernels.py:59-68.

    q/k/v: (..., T, D).  Returns (..., T, D) in fp32 (fp64 if the inputs are
    fp64).  Differentiable by autograd.
    """
    wide = torch.float64 if q.dtype == torch.float64 else torch.float32
    seq, head_dim = q.shape[-2], q.shape[-1]
    aff = (q.to(wide) @ k.to(wide).transpose(-2, -1)) / math.sqrt(head_dim)   # :60
    mask = torch.tril(torch.ones(seq, seq, dtype=torch.bool))                 # :61
    aff = aff.masked_fill(~mask, torch.finfo(torch.float32).min)              # :62
    p = aff.softmax(dim=-1)                                                   # :64
    committed = p.cumsum(dim=-2) - p                                          # :65
    share = p / (committed + p + EPS)                                         # :66
    attn = share / (share.sum(dim=-1, keepdim=True) + EPS)                    # :67
    return attn @ v.to(wide)                                                  # :68


def bids(q: torch.Tensor, k: torch.Tensor, q_offset: int = 0) -> torch.Tensor:
    """Causal-softmax bids p (kernels.py:60-64) for queries at absolute
    positions q_offset.. against keys 0..Tk-1; (..., Tq, Tk) fp32."""
    tq, tk, head_dim = q.shape[-2], k.shape[-2], q.shape[-1]
    aff = (q.float() @ k.float().transpose(-2, -1)) / math.sqrt(head_dim)
    rows = torch.arange(tq)[:, None] + q_offset
    cols = torch.arange(tk)[None, :]
    aff = aff.masked_fill(cols > rows, torch.finfo(torch.float32).min)
    return aff.softmax(dim=-1)


def dilution_chunked(q, k, v, chunk: int = 1024, return_demand: bool = False):
    """Same four lines as kernels.py:64-68, evaluated in query-row chunks with a
    running per-key column sum, so memory is O(chunk * T) instead of O(T^2).

    Returns out (..., T, D) fp32 and, with return_demand, the inclusive column
    totals of p (..., T) — the decode accumulator after this prefix
    (kernels.py:451-453).
    """
    seq = q.shape[-2]
    lead = q.shape[:-2]
    out = torch.empty(*lead, seq, v.shape[-1], dtype=torch.float32)
    demand = torch.zeros(*lead, seq, dtype=torch.float32)
    for a in range(0, seq, chunk):
        b = min(a + chunk, seq)
        p = bids(q[..., a:b, :], k[..., :b, :], q_offset=a)          # (..., b-a, b)
        committed = demand[..., None, :b] + p.cumsum(dim=-2) - p      # :65 with carry
        share = p / (committed + p + EPS)                             # :66
        attn = share / (share.sum(dim=-1, keepdim=True) + EPS)        # :67
        out[..., a:b, :] = attn @ v[..., :b, :].float()               # :68
        demand[..., :b] += p.sum(dim=-2)
    return (out, demand) if return_demand else out


def demand_totals(q, k) -> torch.Tensor:
    """Inclusive column totals of p over all rows, `p.sum(-2)`: what the
    reference's tests compare `aux["committed_total"]` with
    (tests/test_kernels.py:142)."""
    return bids(q, k).sum(dim=-2)


def block_carry(q, k, block: int) -> torch.Tensor:
    """Exclusive demand at the start of every `block`-row query block:
    carry[..., rb, j] = sum_{i < rb*block} p_ij  (tests/test_kernels.py:145-149)."""
    p = bids(q, k)
    seq = p.shape[-1]
    nb = (seq + block - 1) // block
    inclusive = p.cumsum(dim=-2)
    rows = [torch.zeros_like(inclusive[..., 0, :])]
    for rb in range(1, nb):
        rows.append(inclusive[..., rb * block - 1, :])
    return torch.stack(rows, dim=-2)


def row_stats(q, k):
    """(rmax, rden) of the causal softmax in the log2 domain, as K1 stores them
    (kernels.py:159-184): rmax = max_j aff*log2(e), rden = sum_j 2^(aff*log2e - rmax)."""
    seq, head_dim = q.shape[-2], q.shape[-1]
    z = (q.float() @ k.float().transpose(-2, -1)) * (1.4426950408889634 / math.sqrt(head_dim))
    mask = torch.tril(torch.ones(seq, seq, dtype=torch.bool))
    z = z.masked_fill(~mask, float("-inf"))
    rmax = z.max(dim=-1).values
    rden = torch.exp2(z - rmax[..., None]).sum(dim=-1)
    return rmax, rden


def query_correction(q, k) -> torch.Tensor:
    """pk = (p @ k) / sqrt(D), the saved softmax-Jacobian term for dq
    (tests/test_kernels.py:55-59)."""
    return (bids(q, k) @ k.float()) / math.sqrt(q.shape[-1])


def dilution_backward(q, k, v, dout):
    """out, dq, dk, dv by autograd through `dilution_dense`, exactly how the
    reference's gradient tests obtain them (tests/test_kernels.py:116-120)."""
    qs, ks, vs = (t.detach().clone().float().requires_grad_(True) for t in (q, k, v))
    out = dilution_dense(qs, ks, vs)
    out.backward(dout.float())
    return out.detach(), qs.grad, ks.grad, vs.grad


def dilution_backward_analytic(q, k, v, dout):
    """The closed-form gradient the fused backward evaluates (the maths of
    kernels.py:460-465, 677-826 written densely): used to pin the formulas the
    CUDA kernels implement against autograd, independently of any kernel.

    Returns dq, dk, dv and the intermediates (ghat, pk, dbar) the kernels store.
    """
    q, k, v, dout = (t.float() for t in (q, k, v, dout))
    scale = 1.0 / math.sqrt(q.shape[-1])
    p = bids(q, k)
    c = p.cumsum(dim=-2) - p
    inv = 1.0 / (c + p + EPS)
    share = p * inv
    ssum = share.sum(dim=-1, keepdim=True)
    sinv = 1.0 / (ssum + EPS)
    attn = share * sinv
    out = attn @ v
    dbar = (dout * out).sum(dim=-1, keepdim=True)
    ds = (dout @ v.transpose(-2, -1) - dbar) * sinv            # kernels.py:463-464
    ds = ds * (p > 0)                                          # causal mask (:465)
    g = -ds * p * inv * inv                                    # dk_share (:761)
    suffix = g.flip(-2).cumsum(dim=-2).flip(-2) - g            # later queries only (:763)
    pdp = p * (ds * (c + EPS) * inv * inv + suffix)            # (:765)
    ghat = pdp.sum(dim=-1, keepdim=True)                       # (:766)
    dz = pdp - p * ghat
    dq = scale * (dz @ k)
    dk = scale * (dz.transpose(-2, -1) @ q)
    dv = attn.transpose(-2, -1) @ dout                         # (:758)
    pk = scale * (p @ k)
    return dq, dk, dv, dict(ghat=ghat.squeeze(-1), pk=pk, dbar=dbar.squeeze(-1), out=out)


def dilution_backward_chunked(q, k, v, dout, chunk: int = 1024):
    """out, dq, dk, dv with O(chunk * T) memory: the closed-form gradient of
    `dilution_backward_analytic` (kernels.py:460-465, 677-826) evaluated in
    query-row chunks.  A forward sweep (first chunk to last) records the demand
    in front of every chunk and the outputs; a reverse sweep (last chunk to
    first) carries the per-key suffix of dk_share (kernels.py:763-764).  Every
    row sees all of its keys inside one chunk, so ghat is complete per chunk.
    For lengths where autograd through the dense T x T version does not fit.
    """
    q, k, v, dout = (t.float() for t in (q, k, v, dout))
    seq, head_dim = q.shape[-2], q.shape[-1]
    lead = q.shape[:-2]
    scale = 1.0 / math.sqrt(head_dim)
    starts = list(range(0, seq, chunk))
    demand = torch.zeros(*lead, seq)
    before = []                                   # demand in front of each chunk, keys [0, b)
    out = torch.empty(*lead, seq, v.shape[-1])
    for a in starts:
        b = min(a + chunk, seq)
        p = bids(q[..., a:b, :], k[..., :b, :], q_offset=a)
        before.append(demand[..., :b].clone())
        c = before[-1][..., None, :] + p.cumsum(dim=-2) - p
        share = p / (c + p + EPS)
        attn = share / (share.sum(dim=-1, keepdim=True) + EPS)
        out[..., a:b, :] = attn @ v[..., :b, :]
        demand[..., :b] += p.sum(dim=-2)
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    suffix_carry = torch.zeros(*lead, seq)        # sum of dk_share over the chunks already visited
    for idx in range(len(starts) - 1, -1, -1):
        a = starts[idx]
        b = min(a + chunk, seq)
        p = bids(q[..., a:b, :], k[..., :b, :], q_offset=a)
        c = before[idx][..., None, :] + p.cumsum(dim=-2) - p
        inv = 1.0 / (c + p + EPS)
        share = p * inv
        sinv = 1.0 / (share.sum(dim=-1, keepdim=True) + EPS)
        attn = share * sinv
        do = dout[..., a:b, :]
        dbar = (do * out[..., a:b, :]).sum(dim=-1, keepdim=True)
        ds = (do @ v[..., :b, :].transpose(-2, -1) - dbar) * sinv * (p > 0)
        g = -ds * p * inv * inv
        suffix = g.flip(-2).cumsum(dim=-2).flip(-2) - g + suffix_carry[..., None, :b]
        pdp = p * (ds * (c + EPS) * inv * inv + suffix)
        dz = pdp - p * pdp.sum(dim=-1, keepdim=True)
        dq[..., a:b, :] = scale * (dz @ k[..., :b, :])
        dk[..., :b, :] += scale * (dz.transpose(-2, -1) @ q[..., a:b, :])
        dv[..., :b, :] += attn.transpose(-2, -1) @ do
        suffix_carry[..., :b] += g.sum(dim=-2)
    return out, dq, dk, dv


def demand_before(q, k, upto: int, chunk: int = 2048) -> torch.Tensor:
    """Per-key demand committed by query rows [0, upto): column sums of p over
    those rows (kernels.py:65 evaluated at row `upto`), (..., upto) fp32, in
    query-row chunks."""
    demand = torch.zeros(*q.shape[:-2], upto)
    for a in range(0, upto, chunk):
        b = min(a + chunk, upto)
        demand[..., :b] += bids(q[..., a:b, :], k[..., :b, :], q_offset=a).sum(dim=-2)
    return demand


def dilution_rows(q, k, v, row_a: int, row_b: int, chunk: int = 2048) -> torch.Tensor:
    """Output rows [row_a, row_b) of the operator without the rows behind them:
    the demand in front of row_a by `demand_before`, then kernels.py:64-68 on
    the block.  (..., row_b - row_a, D) fp32."""
    front = demand_before(q, k, row_a, chunk)
    p = bids(q[..., row_a:row_b, :], k[..., :row_b, :], q_offset=row_a)
    committed = p.cumsum(dim=-2) - p
    committed[..., :row_a] += front[..., None, :]
    share = p / (committed + p + EPS)
    attn = share / (share.sum(dim=-1, keepdim=True) + EPS)
    return attn @ v[..., :row_b, :].float()


def decode_step(q1, k_cache, v_cache, committed, length: int) -> torch.Tensor:
    """One cached decode step, the eager maths of model.py:242-257 with the
    softmax bid (kernels_bid.py bids_from_affinity, 'softmax' branch).

    q1 (B,H,1,D); caches (B,H,cap,D) with the new token already at length-1;
    committed (B,H,cap) fp32, advanced IN PLACE on [..., :length].  Returns
    (B,H,1,D) fp32.
    """
    head_dim = q1.shape[-1]
    k = k_cache[:, :, :length].float()
    v = v_cache[:, :, :length].float()
    c = committed[:, :, :length]
    aff = (q1.float() @ k.transpose(-2, -1)).squeeze(2) / math.sqrt(head_dim)   # :246
    p = aff.softmax(dim=-1)
    share = p / (c + p + EPS)                                                   # :250-251
    attn = share / (share.sum(dim=-1, keepdim=True) + EPS)                      # :252
    y = attn.unsqueeze(2) @ v                                                   # :255
    c += p                                                                      # :256
    return y


def variant_bids(q, k, bid: str = "softmax", shift: float = 1.0) -> torch.Tensor:
    """Bids under a selectable bid function, the branches of bids_from_affinity
    (kernels_bid.py:94-120): "softmax" as kernels.py:60-64; "sigmoid", "expshift"
    (exp(a) / shift) and "sigshift" (sigmoid(a - log shift)) element-wise with zeros outside the
    causal window; "relu", "relu2", "softplus", "minshift" as f(a) / rowsum(f) with the row
    minimum held constant and a uniform row where there is no mass.  (..., T, T) fp32."""
    seq, head_dim = q.shape[-2], q.shape[-1]
    aff = (q.float() @ k.float().transpose(-2, -1)) / math.sqrt(head_dim)        # kernels_bid.py:153
    causal = torch.tril(torch.ones(seq, seq, dtype=torch.bool))                  # :154
    if bid == "softmax":
        return aff.masked_fill(~causal, torch.finfo(torch.float32).min).softmax(dim=-1)   # :97-98
    if bid == "sigmoid":
        return torch.sigmoid(aff).masked_fill(~causal, 0.0)                      # :99-100
    if bid == "expshift":
        return (torch.exp(aff) / float(shift)).masked_fill(~causal, 0.0)         # :101-102
    if bid == "sigshift":
        return torch.sigmoid(aff - math.log(float(shift))).masked_fill(~causal, 0.0)   # :103-104
    if bid == "relu":
        f = aff.clamp_min(0.0)                                                   # :105-106
    elif bid == "relu2":
        f = aff.clamp_min(0.0) ** 2                                              # :107-108
    elif bid == "softplus":
        f = torch.nn.functional.softplus(aff)                                    # :109-110
    elif bid == "minshift":
        rmin = aff.masked_fill(~causal, float("inf")).amin(dim=-1, keepdim=True).detach()   # :111-113
        f = aff - rmin
    else:
        raise ValueError(f"unknown bid {bid!r}")
    f = f.masked_fill(~causal, 0.0)                                              # :116
    rsum = f.sum(dim=-1, keepdim=True)                                           # :117
    uniform = causal.to(f.dtype) / causal.sum(dim=-1, keepdim=True).to(f.dtype)  # :118-119
    return torch.where(rsum > 0, f / rsum.clamp_min(1e-30), uniform)             # :120


def variant_dense(q, k, v, bid: str = "softmax", share_cumsum=True, shift: float = 1.0) -> torch.Tensor:
    """The operator with a selectable bid and share step, as the dense spec of
    kernels_bid.py:152-166: share_cumsum True (inclusive, the operator), "exclusive"
    (earlier queries' demand only) or False (no share step).  Differentiable by autograd."""
    p = variant_bids(q, k, bid, shift)                                           # :155
    if not share_cumsum:
        return (p / p.sum(dim=-1, keepdim=True)) @ v.float()                     # :156-157
    committed = p.cumsum(dim=-2) - p                                             # :158
    if share_cumsum == "exclusive":
        share = p / (committed + EPS)                                            # :159-160
    else:
        share = p / (committed + p + EPS)                                        # :161-162
    attn = share / (share.sum(dim=-1, keepdim=True) + EPS)                       # :163
    return attn @ v.float()                                                      # :164


def variant_backward(q, k, v, dout, bid: str = "softmax", share_cumsum=True, shift: float = 1.0):
    """out, dq, dk, dv by autograd through `variant_dense`."""
    qs, ks, vs = (t.detach().clone().float().requires_grad_(True) for t in (q, k, v))
    out = variant_dense(qs, ks, vs, bid, share_cumsum, shift)
    out.backward(dout.float())
    return out.detach(), qs.grad, ks.grad, vs.grad


def variant_decode_step(q1, k_cache, v_cache, committed, length: int, bid: str = "softmax", share_cumsum=True,
                        shift: float = 1.0):
    """One cached decode step under a bid / share variant: the maths of the reference's decode
    kernel (kernels_bid.py:905-950), which is the eager step of model.py:242-257 except that
    with no share step the kernel still divides by the row sum of the bids (:948) where the
    eager model returns p v as it is (model.py:254).  Same contract as decode_step;
    `committed` advances by p in place whatever the share step (:947)."""
    head_dim = q1.shape[-1]
    k = k_cache[:, :, :length].float()
    v = v_cache[:, :, :length].float()
    c = committed[:, :, :length]
    aff = (q1.float() @ k.transpose(-2, -1)).squeeze(2) / math.sqrt(head_dim)   # :873, :887
    if bid == "softmax":                                                         # :913-920
        p = aff.softmax(dim=-1)
    elif bid == "expshift":
        p = torch.exp(aff) / float(shift)
    elif bid in ("sigmoid", "sigshift"):
        p = torch.sigmoid(aff - (math.log(float(shift)) if bid == "sigshift" else 0.0))
    else:                                                                        # :880-911, :929-945
        if bid == "minshift":
            f = aff - aff.amin(dim=-1, keepdim=True)
        elif bid == "softplus":
            f = torch.nn.functional.softplus(aff)
        else:
            f = aff.clamp_min(0.0) ** (2 if bid == "relu2" else 1)
        mass = f.sum(dim=-1, keepdim=True)
        p = torch.where(mass > 0, f / mass.clamp_min(1e-30), torch.full_like(f, 1.0 / length))
    if share_cumsum == "exclusive":
        share = p / (c + EPS)                                                   # :937-938
    elif share_cumsum:
        share = p / (c + p + EPS)                                               # :939-940
    else:
        share = p                                                               # :941-942
    y = (share / (share.sum(dim=-1, keepdim=True) + EPS)).unsqueeze(2) @ v      # :943-948
    c += p                                                                      # :947
    return y


def equal_area_bounds(seq: int, ranks: int, tile: int = 128) -> list[int]:
    """Contiguous query-chunk boundaries with (nearly) equal causal area per
    rank: a_r = seq*sqrt(r/R) rounded to the tile size.  Mirrors the host-side
    partition used by the sequence-parallel prefill so tests can cross-check it."""
    bounds = [0]
    for r in range(1, ranks):
        a = int(round(seq * math.sqrt(r / ranks) / tile)) * tile
        bounds.append(min(max(a, bounds[-1]), seq))
    bounds.append(seq)
    return bounds


def softmax_attention(q, k, v, q_offset: int = 0) -> torch.Tensor:
    """Causal softmax attention in fp32: what the reference's softmax layers compute with
    F.scaled_dot_product_attention(q, k, v, is_causal=True) (model.py:96-117).  The same bids as
    kernels.py:60-64 followed by a plain product with v."""
    return bids(q, k, q_offset) @ v.float()


def rope(x: torch.Tensor, offset: int = 0, theta: float = 10000.0) -> torch.Tensor:
    """Rotary position embedding of (..., T, D) as rope.py:26-44: adjacent pairs (2i, 2i+1),
    fp32 angles pos * theta^(-2i/D) cast to x's dtype, out = x*cos + rotate(x)*sin in x's dtype."""
    seq, dim = x.shape[-2], x.shape[-1]
    positions = torch.arange(offset, offset + seq, dtype=torch.float32)
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))      # :34-36
    freqs = torch.outer(positions, inv_freq)
    cos = freqs.cos().to(x.dtype).repeat_interleave(2, dim=-1)                            # :38-41
    sin = freqs.sin().to(x.dtype).repeat_interleave(2, dim=-1)
    pairs = x.reshape(*x.shape[:-1], dim // 2, 2)
    rotated = torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).flatten(-2)            # :43
    return x * cos + rotated * sin


def split_heads(qkv: torch.Tensor, heads: int, offset: int = 0, theta: float | None = 10000.0):
    """q, k, v (B, H, T, D) from the fused projection (B, T, 3*H*D) as model.py:59-67; q and k
    rotated unless theta is None."""
    batch, seq, width = qkv.shape
    d = width // (3 * heads)
    q, k, v = (t.view(batch, seq, heads, d).transpose(1, 2) for t in qkv.split(heads * d, dim=2))
    if theta is not None:
        q, k = rope(q, offset, theta), rope(k, offset, theta)
    return q, k, v
