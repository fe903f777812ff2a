"""The CPU oracle against the reference's golden outputs (no GPU needed)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from conftest import golden, make_inputs, rel_err
from oracle import dilution_oracle as O

SMALL = [(1, (1, 2, 32)), (8, (2, 2, 64)), (65, (1, 2, 32)), (257, (1, 2, 64))]


def _small(t):
    g = golden("small_cases.npz")
    return {k[len(f"t{t}_"):]: torch.from_numpy(g[k]) for k in g.files if k.startswith(f"t{t}_")}


def test_config1_inputs_regenerate_bit_exact():
    g = golden("c1_b1h4t512d64.npz")
    q, k, v, dout = make_inputs(1, 4, 512, 64, int(g["seed"]))
    fp = np.array([float(x.double().sum()) for x in (q, k, v, dout)] +
                  [float(x.flatten()[0]) for x in (q, k, v, dout)])
    assert np.array_equal(fp, g["fingerprint"])


def test_config1_dense_forward_and_autograd_match_reference():
    g = golden("c1_b1h4t512d64.npz")
    q, k, v, dout = make_inputs(1, 4, 512, 64, int(g["seed"]))
    out, dq, dk, dv = O.dilution_backward(q, k, v, dout)
    for name, got in dict(out=out, dq=dq, dk=dk, dv=dv).items():
        assert rel_err(got, torch.from_numpy(g[name])) < 1e-6, name


def test_config1_analytic_backward_matches_reference():
    g = golden("c1_b1h4t512d64.npz")
    q, k, v, dout = make_inputs(1, 4, 512, 64, int(g["seed"]))
    dq, dk, dv, aux = O.dilution_backward_analytic(q, k, v, dout)
    assert rel_err(aux["out"], torch.from_numpy(g["out"])) < 1e-5
    for name, got in dict(dq=dq, dk=dk, dv=dv).items():
        assert rel_err(got, torch.from_numpy(g[name])) < 1e-4, name


@pytest.mark.parametrize("t,shape", SMALL)
def test_small_cases_all_quantities(t, shape):
    c = _small(t)
    out, dq, dk, dv = O.dilution_backward(c["q"], c["k"], c["v"], c["dout"])
    assert rel_err(out, c["out"]) < 1e-6
    for name, got in dict(dq=dq, dk=dk, dv=dv).items():
        assert rel_err(got, c[name]) < 1e-5, name
    assert rel_err(O.demand_totals(c["q"], c["k"]), c["demand"]) < 1e-6
    assert rel_err(O.query_correction(c["q"], c["k"]), c["pk"]) < 1e-6
    adq, adk, adv, _ = O.dilution_backward_analytic(c["q"], c["k"], c["v"], c["dout"])
    for name, got in dict(dq=adq, dk=adk, dv=adv).items():
        assert rel_err(got, c[name]) < 2e-4, name


@pytest.mark.parametrize("t,shape", SMALL)
@pytest.mark.parametrize("chunk", [1, 7, 64, 1024])
def test_chunked_equals_dense(t, shape, chunk):
    c = _small(t)
    out, demand = O.dilution_chunked(c["q"], c["k"], c["v"], chunk=chunk, return_demand=True)
    assert rel_err(out, c["out"]) < 2e-5
    assert rel_err(demand, c["demand"]) < 2e-6


def test_row_stats_rebuild_bids():
    c = _small(257)
    rmax, rden = O.row_stats(c["q"], c["k"])
    d = c["q"].shape[-1]
    z = (c["q"] @ c["k"].transpose(-2, -1)) * (1.4426950408889634 / math.sqrt(d))
    p = torch.exp2(z - rmax[..., None]) / rden[..., None]
    p = p * torch.ones(257, 257).tril()
    assert rel_err(p, O.bids(c["q"], c["k"])) < 1e-5


def test_block_carry_is_exclusive_prefix():
    c = _small(257)
    carry = O.block_carry(c["q"], c["k"], 64)
    p = O.bids(c["q"], c["k"])
    assert carry.shape[-2] == 5
    assert torch.equal(carry[..., 0, :], torch.zeros_like(carry[..., 0, :]))
    assert rel_err(carry[..., 3, :], p[..., :192, :].sum(-2)) < 1e-6


def test_decode_steps_match_reference_rows():
    g = golden("decode_b2h4d32.npz")
    q, k, v, rows = (torch.from_numpy(g[n]) for n in ("q", "k", "v", "rows"))
    prefix = int(g["prefix"])
    total = q.shape[2]
    cap = total + 3
    kc = torch.zeros(2, 4, cap, 32)
    vc = torch.zeros(2, 4, cap, 32)
    kc[:, :, :prefix], vc[:, :, :prefix] = k[:, :, :prefix], v[:, :, :prefix]
    committed = torch.zeros(2, 4, cap)
    committed[:, :, :prefix] = torch.from_numpy(g["demand_prefix"])
    for t in range(prefix, total):
        kc[:, :, t], vc[:, :, t] = k[:, :, t], v[:, :, t]
        y = O.decode_step(q[:, :, t:t + 1], kc, vc, committed, t + 1)
        assert (y[:, :, 0] - rows[:, :, t]).abs().max().item() < 1e-5
    assert rel_err(committed[:, :, :total], torch.from_numpy(g["demand_final"])) < 1e-5
    assert committed[:, :, total:].abs().max().item() == 0


def test_fp32_reference_rounding_is_far_inside_tolerance():
    """fp64 restatement: the fp32 reference's own error, the floor for the 1e-4 bound."""
    c = _small(257)
    hi = O.dilution_dense(c["q"].double(), c["k"].double(), c["v"].double())
    assert rel_err(c["out"], hi) < 1e-5


def test_equal_area_bounds():
    b = O.equal_area_bounds(131072, 8)
    assert b[0] == 0 and b[-1] == 131072 and all(x % 128 == 0 for x in b)
    areas = [b[i + 1] ** 2 - b[i] ** 2 for i in range(8)]
    assert max(areas) / min(areas) < 1.05


@pytest.mark.parametrize("chunk", [7, 64, 1024])
def test_chunked_backward_matches_reference_goldens(chunk):
    """The row-chunked closed-form backward against the reference's autograd gradients."""
    g = golden("c1_b1h4t512d64.npz")
    q, k, v, dout = make_inputs(1, 4, 512, 64, int(g["seed"]))
    out, dq, dk, dv = O.dilution_backward_chunked(q, k, v, dout, chunk=chunk)
    assert rel_err(out, torch.from_numpy(g["out"])) < 1e-5
    for name, got in dict(dq=dq, dk=dk, dv=dv).items():
        assert rel_err(got, torch.from_numpy(g[name])) < 1e-4, name
    for t, _ in SMALL:
        c = _small(t)
        res = O.dilution_backward_chunked(c["q"], c["k"], c["v"], c["dout"], chunk=chunk)
        for name, got in zip(("out", "dq", "dk", "dv"), res):
            assert rel_err(got, c[name]) < 2e-4, (t, name)


def test_chunked_backward_matches_dense_autograd_at_4096():
    """One (b,h) row at T=4096 with the benchmark's value scales: chunked == dense autograd."""
    q, k, v, dout = make_inputs(1, 1, 4096, 64, 1339, scales=(0.5, 0.5, 1.0, 1e-2))
    ref = O.dilution_backward(q, k, v, dout)
    got = O.dilution_backward_chunked(q, k, v, dout, chunk=512)
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, ref):
        assert rel_err(a, b) < 1e-4, name


def test_row_block_helpers_match_dense():
    c = _small(257)
    assert rel_err(O.demand_before(c["q"], c["k"], 100, chunk=32),
                   O.bids(c["q"], c["k"])[..., :100, :100].sum(-2)) < 1e-6
    assert rel_err(O.dilution_rows(c["q"], c["k"], c["v"], 100, 180, chunk=32), c["out"][..., 100:180, :]) < 2e-5
    assert rel_err(O.dilution_rows(c["q"], c["k"], c["v"], 0, 64), c["out"][..., :64, :]) < 2e-5


def test_rope_and_softmax_attention_match_reference_modules():
    """The oracle's RoPE (rope.py:26-44) and softmax attention (model.py:96-117) against
    outputs of the reference's RopeModule and of F.scaled_dot_product_attention."""
    g = golden("layers_b2t24h2d32.npz")
    q, k, v = (torch.from_numpy(g[n]) for n in "qkv")
    theta = float(g["theta"])
    for off in (0, 9):
        assert torch.equal(O.rope(q, off, theta), torch.from_numpy(g[f"rope_f32_off{off}"]))
        assert torch.equal(O.rope(q.bfloat16(), off, theta).float(), torch.from_numpy(g[f"rope_bf16_off{off}"]))
    assert rel_err(O.softmax_attention(q, k, v), torch.from_numpy(g["sdpa"])) < 1e-6
    # the head split of a fused projection: the three parts, per head, q and k rotated
    b, h, t, d = q.shape
    qkv = torch.cat([x.transpose(1, 2).reshape(b, t, h * d) for x in (q, k, v)], dim=2)
    sq, sk, sv = O.split_heads(qkv, h, 9, theta)
    assert torch.equal(sq, torch.from_numpy(g["rope_f32_off9"])) and torch.equal(sv, v)
    assert torch.equal(sk, O.rope(k, 9, theta))


from conftest import SHIFT, VARIANTS, variant_case  # noqa: E402


@pytest.mark.parametrize("key,bid,share", VARIANTS)
def test_variants_match_reference_goldens(key, bid, share):
    """The bid / share restatements against kernels_bid.dilution_attention_reference and its
    autograd gradients (stored by tests/golden/make_golden.py)."""
    c = variant_case(key)
    out, dq, dk, dv = O.variant_backward(c["q"], c["k"], c["v"], c["dout"], bid, share, SHIFT)
    assert rel_err(out, c["out"]) < 1e-5
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert rel_err(got, c[name]) < 1e-4, name
    assert rel_err(O.variant_bids(c["q"], c["k"], bid, SHIFT).sum(-2), c["demand"]) < 1e-6


def test_variant_operator_is_the_operator():
    q, k, v, _ = make_inputs(1, 2, 50, 32, 9)
    assert torch.equal(O.variant_dense(q, k, v, "softmax", True), O.dilution_dense(q, k, v))


@pytest.mark.parametrize("key,bid,share", VARIANTS)
def test_variant_decode_steps_reproduce_dense_rows(key, bid, share):
    """Token-by-token decoding from an empty cache gives the rows of the dense operator and
    leaves the column totals of p in the accumulator (the property the reference's decode test
    checks, tests/test_kernels.py:211-243, for the variant's maths of kernels_bid.py:905-950)."""
    c = variant_case(key)
    q, k, v = c["q"], c["k"], c["v"]
    seq = q.shape[2]
    committed = torch.zeros(*q.shape[:2], seq)
    rows = [O.variant_decode_step(q[:, :, t:t + 1], k, v, committed, t + 1, bid, share, SHIFT) for t in range(seq)]
    got = torch.cat(rows, dim=2)
    assert rel_err(got, c["out"]) < 1e-4
    assert rel_err(committed, c["demand"]) < 1e-5
