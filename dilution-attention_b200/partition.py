"""Partitioning of dilution attention over the GPUs of one box.

Two ways, both one process per GPU (`torch.distributed`, NCCL on GPUs, gloo in
the CPU tests):

* batch x head rows are independent (every kernel indexes by the row n = b*H+h
  only), so training and decode shard the rows with no collective at all:
  `row_shard`.

* long-context prefill is sequence-parallel: rank r owns the contiguous query
  rows [a_r, a_{r+1}) — boundaries chosen for equal causal AREA, since with equal
  lengths the last rank would own (2R-1)/R^2 of the work — all-gathers K/V into
  its own memory, runs the three forward passes on its chunk, and needs exactly
  one exchange: the exclusive prefix over ranks of the per-key column sums of p
  (`exclusive_demand_prefix`).  NCCL has no scan collective, so the prefix is an
  all-gather of the (rows, T) sums followed by a local masked sum.

Nothing here touches device memory of a peer directly: remote data always lands
in local memory through the collective first.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

from . import _lib
from . import kernels as K

TILE = 128  # chunk boundaries are multiples of the largest kernel tile


def row_shard(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous [begin, end) slice of the batch*head rows owned by `rank`."""
    base, extra = divmod(n_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def equal_area_bounds(seq: int, world: int, tile: int = TILE) -> list[int]:
    """Query-chunk boundaries a_0=0 <= ... <= a_R=seq with near-equal causal
    area a_{r+1}^2 - a_r^2, rounded to `tile`."""
    bounds = [0]
    for r in range(1, world):
        a = int(round(seq * math.sqrt(r / world) / tile)) * tile
        bounds.append(min(max(a, bounds[-1]), seq))
    bounds.append(seq)
    return bounds


def exclusive_demand_prefix(local_total: torch.Tensor, seq: int, group=None):
    """Cross-rank exclusive scan of per-key demand.

    local_total: (rows, tk_r) column sums of p over THIS rank's query rows (keys
    beyond tk_r are implicitly zero).  Returns (base, demand):
      base   (rows, tk_r): demand committed by ranks before this one,
      demand (rows, seq) : demand of all ranks, the decode accumulator.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows, tk = local_total.shape
    padded = local_total.new_zeros(rows, seq)
    padded[:, :tk] = local_total
    gathered = padded.new_empty(world, rows, seq)
    dist.all_gather(list(gathered.unbind(0)), padded, group=group)
    demand = gathered.sum(dim=0)
    base = gathered[:rank].sum(dim=0) if rank > 0 else padded.new_zeros(rows, seq)
    return base[:, :tk].contiguous(), demand


def gather_keys(k_local: torch.Tensor, v_local: torch.Tensor, bounds: list[int], group=None):
    """Bring the K/V chunks of every EARLIER rank into local memory and return the
    prefix [0, a_{rank+1}) this rank's queries can see.  k_local/v_local:
    (rows, a_{r+1}-a_r, d).

    Causality makes the exchange triangular: rank r needs the chunks of ranks
    s < r only, so it is done with point-to-point transfers of exactly those
    chunks (no padding to the longest chunk, nothing sent to ranks that cannot use
    it) instead of a symmetric all-gather.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows, _, d = k_local.shape
    end = bounds[rank + 1]
    k = k_local.new_empty(rows, end, d)
    v = v_local.new_empty(rows, end, d)
    k[:, bounds[rank]:end] = k_local
    v[:, bounds[rank]:end] = v_local
    if world == 1:
        return k, v
    mine = torch.stack((k_local, v_local)).contiguous()            # (2, rows, len_r, d)
    ops, inbox = [], {}
    for s in range(rank):                                           # receive from earlier ranks
        if bounds[s + 1] == bounds[s]:
            continue                                                # an empty chunk is never sent
        buf = mine.new_empty(2, rows, bounds[s + 1] - bounds[s], d)
        inbox[s] = buf
        ops.append(dist.P2POp(dist.irecv, buf, dist.get_global_rank(group, s) if group else s, group))
    for r in range(rank + 1, world):                                # send to later ranks
        if end > bounds[rank]:
            ops.append(dist.P2POp(dist.isend, mine, dist.get_global_rank(group, r) if group else r, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    for s, buf in inbox.items():
        a, b = bounds[s], bounds[s + 1]
        k[:, a:b] = buf[0]
        v[:, a:b] = buf[1]
    return k, v


def prefill_chunk(q_local, k_seen, v_seen, q_offset: int, dot_precision: str = "bf16",
                  demand_prefix=None, exchange=None, mark=None):
    """Forward of one contiguous query chunk against the keys it can see.

    q_local (rows, tq, d) at absolute positions q_offset..; k_seen/v_seen
    (rows, q_offset+tq, d).  `exchange(local_total)` -> base is called between
    pass 2 and pass 3 and returns the demand committed by earlier chunks (the
    cross-rank exscan, or a cached prefix); `demand_prefix` supplies it directly.
    Returns out (rows, tq, d) fp32 and local_total (rows, tk) fp32.  An empty
    chunk (tq == 0) launches nothing but still takes part in the exchange, with a
    zero total.  `mark(name)` (optional) is called at the phase boundaries.
    """
    lib = _lib.load()
    rows, tq, d = q_local.shape
    tk = k_seen.shape[1]
    dev = q_local.device
    mark = mark or (lambda name: None)
    if tq == 0:
        total = torch.zeros(rows, tk, device=dev, dtype=torch.float32)
        mark("passes_1_2")
        if exchange is not None:
            exchange(total)
        mark("exchange")
        mark("pass_3")
        return torch.empty(rows, 0, d, device=dev, dtype=torch.float32), total
    lowp, _ = K._resolve_precision(dot_precision)
    want = torch.bfloat16 if (lowp or q_local.dtype == torch.bfloat16) else torch.float32
    qf, kf, vf = (x.to(want).contiguous() for x in (q_local, k_seen, v_seen))
    code = _lib.BF16 if want == torch.bfloat16 else _lib.F32
    prec = _lib.PREC[dot_precision]
    scale = 1.0 / math.sqrt(d)
    f32 = dict(device=dev, dtype=torch.float32)
    # forward only: the coarsest spacing the kernels for this case take (an offset that is not a
    # multiple of the tile size runs on the fp32 kernels)
    carry_rows = _lib.carry_rows(code, prec, d, False) if q_offset % TILE == 0 else _lib.CARRY_ROWS
    ncb = (tq + carry_rows - 1) // carry_rows
    rmax, rden, ssum = (torch.empty(rows, tq, **f32) for _ in range(3))
    carry = torch.empty(rows, ncb, tk, **f32)
    total = torch.empty(rows, tk, **f32)
    out = torch.empty(rows, tq, d, **f32)
    st = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(lib.dilution_rowstats(qf.data_ptr(), kf.data_ptr(), code, prec, rows, tq, tk, q_offset,
                                     d, scale, rmax.data_ptr(), rden.data_ptr(), st), "dilution_rowstats")
    _lib.check(lib.dilution_colsum_scan(qf.data_ptr(), kf.data_ptr(), code, prec, rows, tq, tk, q_offset,
                                        d, scale, rmax.data_ptr(), rden.data_ptr(), None, carry_rows,
                                        carry.data_ptr(), total.data_ptr(), st), "dilution_colsum_scan")
    mark("passes_1_2")
    base = demand_prefix
    if exchange is not None:
        base = exchange(total)
    if base is not None:
        base = base.to(torch.float32).contiguous()
    mark("exchange")
    _lib.check(lib.dilution_forward_main(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), code, prec,
                                         rows, tq, tk, q_offset, d, scale, K.EPS,
                                         rmax.data_ptr(), rden.data_ptr(), carry.data_ptr(), carry_rows,
                                         None if base is None else base.data_ptr(),
                                         out.data_ptr(), ssum.data_ptr(), None, st),
               "dilution_forward_main")
    mark("pass_3")
    return out, total


def sequence_parallel_prefill(q_local, k_local, v_local, seq: int, bounds: list[int] | None = None,
                              dot_precision: str = "bf16", group=None, mark=None):
    """Sequence-parallel prefill of a (rows, seq, d) problem.

    Every rank passes ITS chunk of q, k, v (rows, a_{r+1}-a_r, d) for the
    boundaries `bounds` (default: equal_area_bounds).  Returns
      out    (rows, a_{r+1}-a_r, d) fp32 for the local query rows,
      demand (rows, seq) fp32: the decode accumulator, identical on all ranks.
    `mark(name)` (optional) is called after each phase — "gather_keys",
    "passes_1_2", "exchange", "pass_3" — so that a caller can record CUDA events.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if bounds is None:
        bounds = equal_area_bounds(seq, world)
    k_seen, v_seen = gather_keys(k_local, v_local, bounds, group)
    if mark is not None:
        mark("gather_keys")
    result = {}

    def exchange(local_total):
        base, demand = exclusive_demand_prefix(local_total, seq, group)
        result["demand"] = demand
        return base

    out, _ = prefill_chunk(q_local, k_seen, v_seen, bounds[rank], dot_precision, exchange=exchange, mark=mark)
    return out, result["demand"]


# ---- the LM with its heads sharded over ranks ------------------------------------------------
# The attention operator shards by (batch, head) rows with no exchange; a model gets those rows
# onto different GPUs by giving each rank a slice of the heads.  What follows is the usual
# tensor-parallel split of a transformer block around that: the projections that produce heads
# (c_attn; the MLP's up / gate projections) are split by output features, the ones that consume
# them (c_proj; the MLP's down projection) by input features, and ONE all-reduce follows each of
# the latter.  Embedding, LayerNorms and lm_head stay replicated.
class _CopyToRanks(torch.autograd.Function):
    """Identity forward; the backward sums the input's gradient over the ranks (every rank holds
    only its heads' contribution to it)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _SumOverRanks(torch.autograd.Function):
    """All-reduce forward (partial products of the row-split projection); identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class HeadParallelInput(torch.nn.Module):
    """`inner(x)` for an `inner` whose output features are split over the ranks."""

    def __init__(self, inner, group):
        super().__init__()
        self.inner, self.group = inner, group

    def forward(self, x):
        return self.inner(_CopyToRanks.apply(x, self.group))


class HeadParallelOutput(torch.nn.Module):
    """A projection whose INPUT features are split over the ranks: local product, all-reduce,
    then the (replicated) bias once."""

    def __init__(self, weight, bias, group):
        super().__init__()
        self.weight = torch.nn.Parameter(weight)
        self.weight.head_sharded = True
        self.bias = None if bias is None else torch.nn.Parameter(bias)
        self.group = group

    def forward(self, x):
        y = _SumOverRanks.apply(torch.nn.functional.linear(x, self.weight), self.group)
        return y if self.bias is None else y + self.bias.to(y.dtype)


def _rows_of(linear, index):
    """nn.Linear keeping the output features `index` of `linear`."""
    out = torch.nn.Linear(linear.in_features, index.numel(), bias=linear.bias is not None,
                          device=linear.weight.device, dtype=linear.weight.dtype)
    with torch.no_grad():
        out.weight.copy_(linear.weight[index])
        if linear.bias is not None:
            out.bias.copy_(linear.bias[index])
    for p in out.parameters():
        p.head_sharded = True                      # a slice: its gradient norm is a partial one
    return out


def _columns_of(linear, index, group):
    """HeadParallelOutput keeping the input features `index` of `linear`."""
    with torch.no_grad():
        weight = linear.weight[:, index].clone()
        bias = None if linear.bias is None else linear.bias.detach().clone()
    return HeadParallelOutput(weight, bias, group)


def shard_lm_heads(model, group=None):
    """Split an initialised `DilutionLM` (model.py:342-512) over the ranks of `group` IN PLACE:
    every attention layer keeps n_heads / world of its heads (the rows of `c_attn` that produce
    them, the columns of `c_proj` that consume them), every MLP hidden / world of its units, and
    one all-reduce follows `c_proj` and the MLP's last projection.  All ranks must hold the same
    weights when this is called (same seed, or a broadcast), and must feed the same tokens; every
    rank then computes the same logits and loss as the unsplit model, with 1 / world of the
    attention rows, the projection FLOPs and the KV cache.  Gradients of the replicated
    parameters (embedding, LayerNorms, biases behind an all-reduce) come out identical on every
    rank; the split weights' gradients are the matching slices of the unsplit ones.  The layers'
    `n_heads` / `d_model` attributes become the local ones, which is all `_split_heads`,
    `_merge_heads`, the caches and this library's kernels read (model.py:59-93)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world == 1:
        return model
    if getattr(model.config, "dropout", 0.0) > 0.0:
        # the replicated activations (residual stream, MLP output) would draw a different mask on
        # every rank, and the ranks' copies of the model would drift apart
        raise ValueError("a model with dropout cannot be split by heads: the ranks' dropout masks differ")
    for block in model.transformer.h:
        attn = block.attn
        if not hasattr(attn, "c_attn"):
            raise ValueError(f"cannot shard a {type(attn).__name__} layer by heads")
        if isinstance(attn.c_attn, HeadParallelInput):
            raise ValueError("this model's heads are split already")
        heads, width = attn.n_heads, attn.d_model
        if heads % world:
            raise ValueError(f"{heads} heads do not divide over {world} ranks")
        local = width // world                                     # features of this rank's heads
        dev = attn.c_attn.weight.device
        mine = torch.arange(rank * local, (rank + 1) * local, device=dev)
        attn.c_attn = HeadParallelInput(
            _rows_of(attn.c_attn, torch.cat([mine, width + mine, 2 * width + mine])), group)
        attn.c_proj = _columns_of(attn.c_proj, mine, group)
        attn.n_heads, attn.d_model = heads // world, local
        mlp = block.mlp
        ups = [name for name in ("gate_proj", "up_proj", "c_fc") if hasattr(mlp, name)]
        down = "down_proj" if hasattr(mlp, "down_proj") else "c_proj"
        hidden = getattr(mlp, down).in_features
        if hidden % world:
            raise ValueError(f"MLP width {hidden} does not divide over {world} ranks")
        units = torch.arange(rank * (hidden // world), (rank + 1) * (hidden // world), device=dev)
        for name in ups:
            setattr(mlp, name, _rows_of(getattr(mlp, name), units))
        setattr(mlp, down, _columns_of(getattr(mlp, down), units, group))
        block.mlp = HeadParallelInput(mlp, group)
    return model


def clip_grad_norm_(model, max_norm: float, group=None) -> torch.Tensor:
    """`torch.nn.utils.clip_grad_norm_` for a model split by `shard_lm_heads`: the squared norms
    of the split weights' gradients are summed over the ranks, the replicated parameters count
    once, and every rank scales by the same factor.  Returns the total norm (of the whole model)."""
    sharded = [p.grad for p in model.parameters() if p.grad is not None and getattr(p, "head_sharded", False)]
    whole = [p.grad for p in model.parameters() if p.grad is not None and not getattr(p, "head_sharded", False)]
    ref = (sharded or whole)[0]
    part = ref.new_zeros((), dtype=torch.float32)
    if sharded:
        part = torch.stack([g.float().pow(2).sum() for g in sharded]).sum()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(part, group=group)
    rest = torch.stack([g.float().pow(2).sum() for g in whole]).sum() if whole else part.new_zeros(())
    total = (part + rest).sqrt()
    factor = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for g in sharded + whole:
        g.mul_(factor.to(g.dtype))
    return total
