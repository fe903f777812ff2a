"""Parity against the CPU oracle at the sizes the benchmark quotes: the training
shape at T=16384, the long-context prefill at T=131072 and cached decode at
16384 / 131072 keys.  One (batch, head) row or a handful of rows each, so that
the oracle finishes in seconds; the kernels see the same tile counts, checkpoint
counts and chunk sizes as the full workloads (rows are independent).
Mirrors tests/test_kernels.py:109-127, 205-241 of the reference at its large sizes."""

from __future__ import annotations

import pytest
import torch

from conftest import make_inputs, rel_err, seeded
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_training_shape_t16384_out_and_grads_match_oracle(kernels):
    """B4 H16 T16384 d64 bf16 workload, one row: 128 key blocks x 512 checkpoints in the
    reverse pass.  out, dq, dk, dv <= 2e-2 max-abs against the oracle on the same
    bf16-rounded inputs, and the reference's relative metric."""
    t, d = 16384, 64
    q, k, v, dout = make_inputs(1, 1, t, d, 1339, scales=(0.5, 0.5, 1.0, 1e-2))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref = O.dilution_backward_chunked(qb.float(), kb.float(), vb.float(), dout, chunk=1024)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    out = kernels.dilution_attention(qs, ks, vs, dot_precision="bf16")
    out.backward(dout.to(DEV))
    assert (out.detach().cpu() - ref[0]).abs().max().item() < 2e-2
    assert rel_err(out.detach().cpu(), ref[0]) < 2e-2
    for name, gr, x in (("dq", ref[1], qs), ("dk", ref[2], ks), ("dv", ref[3], vs)):
        assert torch.isfinite(x.grad).all(), name
        assert (x.grad.float().cpu() - gr).abs().max().item() < 2e-2, name
        assert rel_err(x.grad.float().cpu(), gr) < 5e-2, name


def test_training_shape_t16384_unit_dout(kernels):
    """Same row with dout ~ N(0,1): gradients of order one, so the 2e-2 max-abs bound bites."""
    t, d = 16384, 64
    q, k, v, dout = make_inputs(1, 1, t, d, 1441, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref = O.dilution_backward_chunked(qb.float(), kb.float(), vb.float(), dout, chunk=1024)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    kernels.dilution_attention(qs, ks, vs, dot_precision="bf16").backward(dout.to(DEV))
    for name, gr, x in (("dq", ref[1], qs), ("dk", ref[2], ks), ("dv", ref[3], vs)):
        assert rel_err(x.grad.float().cpu(), gr) < 3e-2, name


def test_prefill_t131072_chunked_on_one_gpu(pkg):
    """B1 H16 T131072 workload, one head, cut into the 8 equal-area query chunks of the
    sequence-parallel prefill and run chunk by chunk on one GPU with the demand of the earlier
    chunks carried by hand (what the ranks exchange).  Row blocks at the start and across two
    chunk boundaries against the oracle; sum_j demand_j == T; v == 1 gives out == 1."""
    t, d = 131072, 64
    q, k, v = (seeded((1, t, d), 1340 + i).bfloat16() for i in range(3))
    bounds = pkg.partition.equal_area_bounds(t, 8)
    qd, kd, vd = (x.to(DEV) for x in (q, k, v))
    demand = torch.zeros(1, t, device=DEV)
    outs = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        out, total = pkg.partition.prefill_chunk(qd[:, a:b], kd[:, :b], vd[:, :b], a, dot_precision="bf16",
                                                 demand_prefix=demand[:, :b].contiguous())
        demand[:, :b] += total
        outs.append(out)
    out = torch.cat(outs, dim=1).cpu()
    assert torch.isfinite(out).all()
    assert abs(demand.double().sum().item() - t) / t < 1e-3
    qf, kf, vf = (x.float() for x in (q, k, v))
    ref0 = O.dilution_chunked(qf[:, :4096], kf[:, :4096], vf[:, :4096], chunk=1024)
    assert (out[:, :4096] - ref0).abs().max().item() < 2e-2
    for edge in (bounds[1], bounds[3]):
        lo, hi = edge - 128, edge + 128
        ref = O.dilution_rows(qf, kf, vf, lo, hi, chunk=1024)
        assert (out[:, lo:hi] - ref).abs().max().item() < 2e-2, edge
    front = O.demand_before(qf, kf, bounds[1], chunk=1024)
    # demand of the keys in front of the first boundary, as committed by the first chunk alone
    first_total = pkg.partition.prefill_chunk(qd[:, :bounds[1]], kd[:, :bounds[1]], vd[:, :bounds[1]], 0,
                                              dot_precision="bf16")[1]
    assert rel_err(first_total.cpu(), front) < 2e-2
    # rows of attn are normalised: the last chunk with v == 1
    a, b = bounds[-2], bounds[-1]
    ones = torch.ones(1, b, d, device=DEV, dtype=torch.bfloat16)
    prefix = demand.clone()
    out1, total = pkg.partition.prefill_chunk(qd[:, a:b], kd, ones, a, dot_precision="bf16")
    prefix -= total                                   # demand in front of the last chunk
    out1, _ = pkg.partition.prefill_chunk(qd[:, a:b], kd, ones, a, dot_precision="bf16",
                                          demand_prefix=prefix.contiguous())
    assert (out1 - 1).abs().max().item() < 1e-2


@pytest.mark.parametrize("length", [16384, 131072])
def test_decode_at_benchmark_cache_lengths(kernels, length):
    """4 rows of the batch 64 x 16 heads decode workload at its two cache lengths (the chunk
    size the launcher picks differs between them), random demand, three steps."""
    rows, d, steps = 4, 64, 3
    cap = length + steps + 2
    g = torch.Generator().manual_seed(length)
    kc = torch.randn(1, rows, cap, d, generator=g).bfloat16()
    vc = torch.randn(1, rows, cap, d, generator=g).bfloat16()
    kc[:, :, length:] = 0
    vc[:, :, length:] = 0
    committed = torch.zeros(1, rows, cap)
    committed[:, :, :length] = torch.rand(1, rows, length, generator=g) * 3.0
    newq, newk, newv = (torch.randn(steps, 1, rows, 1, d, generator=g).bfloat16() for _ in range(3))
    kd, vd, cd = kc.to(DEV), vc.to(DEV), committed.to(DEV)
    spare_k, spare_c = kd[:, :, length + steps:].clone(), cd[:, :, length + steps:].clone()
    for s in range(steps):
        pos = length + s
        kc[:, :, pos], vc[:, :, pos] = newk[s][:, :, 0], newv[s][:, :, 0]
        kd[:, :, pos], vd[:, :, pos] = newk[s][:, :, 0].to(DEV), newv[s][:, :, 0].to(DEV)
        ref = O.decode_step(newq[s], kc, vc, committed, pos + 1)
        got = kernels.dilution_decode_step(newq[s].to(DEV), kd, vd, cd, pos + 1)
        assert got.dtype == torch.bfloat16
        assert (got.float().cpu() - ref).abs().max().item() < 2e-2, s
        assert rel_err(cd[:, :, :pos + 1].cpu(), committed[:, :, :pos + 1]) < 1e-5, s
    assert torch.equal(kd[:, :, length + steps:], spare_k)
    assert torch.equal(cd[:, :, length + steps:], spare_c)
