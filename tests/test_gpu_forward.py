"""Forward / prefill parity of the CUDA path against the CPU oracle and the
reference's golden outputs.  Mirrors tests/test_kernels.py of the reference."""

from __future__ import annotations

import math

import pytest
import torch

from conftest import golden, make_inputs, rel_err, seeded
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cuda(*xs):
    return tuple(x.to(DEV) for x in xs)


@pytest.mark.parametrize("seq", [1, 8, 64, 128, 257])
@pytest.mark.parametrize("shape", [(1, 1), (2, 4)])
def test_fused_forward_matches_oracle_fp32(kernels, seq, shape):
    b, h = shape
    q, k, v, _ = make_inputs(b, h, seq, 64, seq)
    ref = O.dilution_dense(q, k, v)
    got = kernels.dilution_attention_forward(*_cuda(q, k, v)).cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 1e-3          # the reference's own bound
    assert rel_err(got, ref) < 1e-4                        # fp32 kernels: 1e-4 relative


def test_config1_golden_forward_and_backward_fp32(kernels):
    g = golden("c1_b1h4t512d64.npz")
    q, k, v, dout = make_inputs(1, 4, 512, 64, int(g["seed"]))
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = kernels.dilution_attention(qs, ks, vs, dot_precision="ieee")
    out.backward(dout.to(DEV))
    for name, got in dict(out=out.detach(), dq=qs.grad, dk=ks.grad, dv=vs.grad).items():
        assert rel_err(got.cpu(), torch.from_numpy(g[name])) < 1e-4, name


def test_reference_signature_entry_point_fp32(kernels):
    g = golden("c1_b1h4t512d64.npz")
    q, k, v, _ = make_inputs(1, 4, 512, 64, int(g["seed"]))
    got = kernels.dilution_attention_reference(*_cuda(q, k, v))
    assert got.dtype == torch.float32 and got.shape == (1, 4, 512, 64)
    assert rel_err(got.cpu(), torch.from_numpy(g["out"])) < 1e-4


@pytest.mark.parametrize("t", [1, 8, 65, 257])
def test_small_golden_cases(kernels, t):
    g = golden("small_cases.npz")
    c = {k[len(f"t{t}_"):]: torch.from_numpy(g[k]) for k in g.files if k.startswith(f"t{t}_")}
    out, aux = kernels.dilution_attention_forward(*_cuda(c["q"], c["k"], c["v"]), return_aux=True,
                                                  _save_pk=True)
    assert rel_err(out.cpu(), c["out"]) < 1e-4
    assert rel_err(aux["committed_total"].cpu(), c["demand"]) < 2e-5
    assert rel_err(aux["pk"].reshape_as(c["pk"]).cpu(), c["pk"]) < 2e-5


@pytest.mark.parametrize("head_dim", [16, 32, 64, 128])
def test_saved_query_correction_all_head_dims(kernels, head_dim):
    q, k, v, _ = make_inputs(1, 2, 257, head_dim, head_dim)
    out, aux = kernels.dilution_attention_forward(*_cuda(q, k, v), return_aux=True, _save_pk=True)
    assert rel_err(out.cpu(), O.dilution_dense(q, k, v)) < 1e-4
    torch.testing.assert_close(aux["pk"].reshape_as(q).cpu(), O.query_correction(q, k), atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("seq", [1, 65, 257, 2049])
def test_checkpoints_totals_and_row_stats(kernels, seq):
    q, k, v, _ = make_inputs(1, 2, seq, 32, seq)
    out, aux = kernels.dilution_attention_forward(*_cuda(q, k, v), return_aux=True, _save_pk=True)
    torch.testing.assert_close(out.cpu(), O.dilution_dense(q, k, v), atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(aux["committed_total"].cpu(), O.demand_totals(q, k), atol=2e-5, rtol=2e-5)
    bm = aux["bwd_block_m"]
    carry = aux["carry"].cpu()
    assert carry.shape[1] == (seq + bm - 1) // bm
    expected = O.block_carry(q, k, bm).reshape(2, -1, seq)
    for rb in range(carry.shape[1]):
        end = min((rb + 1) * bm, seq)      # only the causal key range is initialised
        torch.testing.assert_close(carry[:, rb, :end], expected[:, rb, :end], atol=2e-5, rtol=2e-5)
    rmax, rden = O.row_stats(q, k)
    lse = (aux["rmax"] + torch.log2(aux["rden"])).cpu().reshape(1, 2, seq)
    torch.testing.assert_close(lse, rmax + torch.log2(rden), atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("training", [False, True])
@pytest.mark.parametrize("seq", [64, 200, 1000])
def test_tensor_core_checkpoints_at_both_spacings(kernels, seq, training):
    """bf16, d=64: the column-sum pass stores a checkpoint every 32 rows when a backward will
    follow and every 64 rows otherwise; both against the oracle's block carry."""
    q, k, v, _ = make_inputs(1, 2, seq, 64, 60 + seq, scales=(0.7, 0.7, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    out, aux = kernels.dilution_attention_forward(*_cuda(qb, kb, vb), dot_precision="bf16", return_aux=True,
                                                  _training=training)
    bm = aux["bwd_block_m"]
    assert bm == (32 if training else 64)
    carry = aux["carry"].cpu()
    assert carry.shape[1] == (seq + bm - 1) // bm
    expected = O.block_carry(qb.float(), kb.float(), bm).reshape(2, -1, seq)
    for rb in range(carry.shape[1]):
        end = min((rb + 1) * bm, seq)      # only the causal key range is initialised
        assert (carry[:, rb, :end] - expected[:, rb, :end]).abs().max().item() < 2e-2 * max(1.0, expected.abs().max().item())
    assert (out.cpu() - O.dilution_dense(qb.float(), kb.float(), vb.float())).abs().max().item() < 2e-2


def test_bf16_inputs_against_fp32_oracle(kernels):
    q, k, v, _ = make_inputs(2, 4, 128, 64, 0)
    ref = O.dilution_dense(q, k, v)
    got = kernels.dilution_attention_forward(*(x.bfloat16() for x in _cuda(q, k, v)), dot_precision="bf16").cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 5e-2                  # reference bound, fp32 inputs
    qb, kb, vb = (x.bfloat16().float() for x in (q, k, v))        # same bf16-rounded inputs
    assert (got - O.dilution_dense(qb, kb, vb)).abs().max().item() < 2e-2


@pytest.mark.parametrize("seq", [300, 1000, 2049])
def test_bf16_tensor_path_ragged_lengths(kernels, seq):
    q, k, v, _ = make_inputs(1, 3, seq, 64, 40 + seq, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    out, aux = kernels.dilution_attention_forward(*_cuda(qb, kb, vb), dot_precision="bf16", return_aux=True,
                                                  _save_pk=True)
    ref, demand = O.dilution_chunked(qb.float(), kb.float(), vb.float(), chunk=512, return_demand=True)
    assert (out.cpu() - ref).abs().max().item() < 2e-2
    assert rel_err(aux["committed_total"].cpu(), demand) < 2e-2
    assert rel_err(aux["pk"].reshape(1, 3, seq, 64).cpu(), O.query_correction(qb.float(), kb.float())) < 2e-2


def test_bf16_forward_runs_on_the_tensor_core_kernels(pkg, kernels):
    """dot_precision="bf16" with bf16 inputs and head_dim 64 must launch the tcgen05
    kernels for all three passes (not the fp32-FMA ones), and match the oracle."""
    q, k, v, _ = make_inputs(2, 2, 700, 64, 21, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    pkg._lib.profile(True)
    pkg._lib.profile_collect()
    out, aux = kernels.dilution_attention_forward(*_cuda(qb, kb, vb), dot_precision="bf16", return_aux=True)
    torch.cuda.synchronize()
    names = set(pkg._lib.profile_collect())
    pkg._lib.profile(False)
    assert {"tc_rowstats", "tc_colsum_scan", "tc_forward_main"} <= names, names
    ref, demand = O.dilution_chunked(qb.float(), kb.float(), vb.float(), chunk=256, return_demand=True)
    assert (out.cpu() - ref).abs().max().item() < 2e-2
    assert rel_err(aux["committed_total"].cpu(), demand) < 2e-2


def test_slabbed_forward_equals_single_launch(kernels):
    q, k, v, _ = make_inputs(2, 3, 200, 64, 5)
    whole = kernels.dilution_attention_forward(*_cuda(q, k, v))
    slabs = kernels.dilution_attention_forward(*_cuda(q, k, v), scratch_budget_gib=200 * 4 * 4 * 2 / 2**30)
    assert torch.equal(whole, slabs)


@pytest.mark.parametrize("prec,tol", [("ieee", 1e-4), ("tf32", 5e-3)])
def test_non_contiguous_head_views_like_the_model(kernels, prec, tol):
    """The model hands over transposed views of the fused c_attn output (model.py:59-67)."""
    b, t, h, d = 2, 96, 4, 32
    x = seeded((b, t, 3 * h * d), 3)
    q, k, v = (y.view(b, t, h, d).transpose(1, 2) for y in x.split(h * d, dim=2))
    got = kernels.dilution_attention_forward(*_cuda(q, k, v), dot_precision=prec).cpu()
    assert rel_err(got, O.dilution_dense(q, k, v)) < tol


@pytest.mark.parametrize("prec,dtype,tol", [("ieee", torch.float32, 1e-4), ("bf16", torch.bfloat16, 2e-2)])
def test_chunked_prefill_with_offsets_equals_whole(pkg, prec, dtype, tol):
    """Query chunks at offsets with the demand of earlier chunks as carry base
    reproduce the whole-sequence operator: the sequence-parallel building block."""
    seq, d, rows = 640, 64, 3
    q, k, v, _ = make_inputs(1, rows, seq, d, 77, scales=(0.7, 0.7, 1.0, 1.0))
    q, k, v = (x[0].to(dtype) for x in (q, k, v))
    ref, demand_ref = O.dilution_chunked(q.float(), k.float(), v.float(), chunk=128, return_demand=True)
    demand = torch.zeros(rows, seq, device=DEV)
    for a, b in [(0, 128), (128, 384), (384, 640)]:
        out, total = pkg.partition.prefill_chunk(q[:, a:b].to(DEV), k[:, :b].to(DEV), v[:, :b].to(DEV), a,
                                                 dot_precision=prec, demand_prefix=demand[:, :b].contiguous())
        demand[:, :b] += total
        assert (out.cpu() - ref[:, a:b]).abs().max().item() < (tol if prec == "bf16" else 1e-4)
    assert rel_err(demand.cpu(), demand_ref) < tol


def test_size_independent_properties_at_16k(kernels):
    """T=16384, one (b,h) row, bf16: properties that need no T^2 oracle.
    (a) v == 1 gives out == 1 (rows of attn are normalised);
    (b) sum_j committed_total_j == T (every row of p sums to one);
    (c) the operator is linear in v."""
    t, d = 16384, 64
    q, k, v, v2 = make_inputs(1, 1, t, d, 9, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb = q.bfloat16().to(DEV), k.bfloat16().to(DEV)
    ones = torch.ones(1, 1, t, d, device=DEV, dtype=torch.bfloat16)
    out1, aux = kernels.dilution_attention_forward(qb, kb, ones, dot_precision="bf16", return_aux=True)
    assert (out1 - 1).abs().max().item() < 1e-2
    assert abs(aux["committed_total"].double().sum().item() - t) / t < 1e-3
    va, vb = v.bfloat16().to(DEV), (v2 * 0.5).bfloat16().to(DEV)
    oa = kernels.dilution_attention_forward(qb, kb, va, dot_precision="bf16")
    ob = kernels.dilution_attention_forward(qb, kb, vb, dot_precision="bf16")
    oab = kernels.dilution_attention_forward(qb, kb, (va.float() + vb.float()).bfloat16(), dot_precision="bf16")
    assert (oab - (oa + ob)).abs().max().item() < 2e-2
    # sampled rows against the chunked oracle restricted to the needed prefix
    ref = O.dilution_chunked(qb.float().cpu()[..., :2048, :], kb.float().cpu()[..., :2048, :],
                             va.float().cpu()[..., :2048, :], chunk=512)
    assert (oa.cpu()[..., :2048, :] - ref).abs().max().item() < 2e-2
