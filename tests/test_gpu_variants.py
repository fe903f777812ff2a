"""The bid / share ablations (the reference's kernels_bid.py) through `kernels_bid` of this
package: parity with the reference's goldens and with the CPU oracle for the forward, the
gradients, the demand totals and the cached decode step, and the reference's model configured
with them (model.py:133-156).  Mirrors tests/test_kernels.py:349-395 of the reference, which
checks the same entry points against `dilution_attention_reference(..., bid=, share_cumsum=)`."""

from __future__ import annotations

import os
import sys

import pytest
import torch

from conftest import ROOT, SHIFT, VARIANTS, load_package, make_inputs, rel_err, variant_case
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.fixture(scope="module")
def KB():
    return load_package().kernels_bid


def check_grads(share, got, want, tol):
    """dq, dk, dv against the reference's autograd.  With the exclusive share step every row
    collapses onto its diagonal key (committed is exactly 0 there, so that entry wins by 1/eps):
    the true dq and dk are ~1e-9 and what any fp32 evaluation returns for them is rounding noise
    on cancelling 1e9-scale terms, in the reference's kernels too — its own test compares the
    output and dv only (tests/test_kernels.py:378-416).  Here as there, plus: the noise is
    finite."""
    for name, g, w in zip(("dq", "dk", "dv"), got, want):
        g = g.float().cpu()
        if share == "exclusive" and name != "dv":
            assert torch.isfinite(g).all(), name
        else:
            assert rel_err(g, w) < tol, name


@pytest.mark.parametrize("key,bid,share", VARIANTS)
def test_goldens_forward_and_backward_fp32(KB, key, bid, share):
    c = variant_case(key)
    qs, ks, vs = (c[n].to(DEV).requires_grad_(True) for n in "qkv")
    out = KB.dilution_attention(qs, ks, vs, dot_precision="ieee", bid=bid, share_cumsum=share, shift=SHIFT)
    out.backward(c["dout"].to(DEV))
    assert out.dtype == torch.float32 and rel_err(out.detach().cpu(), c["out"]) < 1e-4
    check_grads(share, (qs.grad, ks.grad, vs.grad), (c["dq"], c["dk"], c["dv"]), 1e-4)


@pytest.mark.parametrize("key,bid,share", VARIANTS)
def test_reference_signature_and_demand_totals(KB, key, bid, share):
    c = variant_case(key)
    q, k, v = (c[n].to(DEV) for n in "qkv")
    out = KB.dilution_attention_reference(q, k, v, bid=bid, share_cumsum=share, shift=SHIFT)
    assert rel_err(out.cpu(), c["out"]) < 1e-4
    out2, aux = KB.dilution_attention_forward(q, k, v, return_aux=True, bid=bid, share_cumsum=share, shift=SHIFT)
    assert rel_err(out2.cpu(), c["out"]) < 1e-4
    assert rel_err(aux["committed_total"].cpu(), c["demand"]) < 1e-5
    assert aux["bid"] == bid and aux["share_cumsum"] == share
    assert (aux["rmax"] is None) == (bid in ("sigmoid", "expshift", "sigshift"))


@pytest.mark.parametrize("key,bid,share", VARIANTS)
@pytest.mark.parametrize("seq,head_dim", [(257, 64), (700, 32), (130, 128)])
def test_ragged_lengths_against_oracle(KB, key, bid, share, seq, head_dim):
    """fp32 tensors under "ieee" and "tf32".  The f(a) / rowsum(f) bids carry a Jacobian factor
    1 / (row mass) that is unbounded where a row has one barely positive key; the reference bounds
    their "ieee" gradients at 2e-3 (relu2, which squares the affinities: 5e-3) and does not test
    them under "tf32" (tests/test_kernels.py:296-316).  Same bounds here.  Under "tf32" a rounded
    product can land on the other side of relu's kink, and a row whose only positive affinities
    are small sees them move by several percent (twice that after relu2's square) with the
    gradient of exactly those rows the largest of the tensor: relu and relu2 are held to the
    output (2e-2, relu2 1e-1) and to finite gradients there; the same kernels with the same tf32
    products are held to 2e-2 on outputs AND gradients by test_bf16_tensors, whose bf16 values
    tf32 carries without rounding."""
    q, k, v, dout = make_inputs(2, 2, seq, head_dim, 300 + seq)
    ref, rdq, rdk, rdv = O.variant_backward(q, k, v, dout, bid, share, SHIFT)
    row_sum = bid in ("relu", "relu2", "softplus", "minshift")
    kinked = bid in ("relu", "relu2")
    ieee_grad = 5e-3 if bid == "relu2" else 2e-3 if row_sum else 1e-4
    for prec, tol, gtol in (("ieee", 1e-4, ieee_grad),
                            ("tf32", 1e-1 if bid == "relu2" else 2e-2 if kinked else 5e-3, None if kinked else 5e-3)):
        qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
        out = KB.dilution_attention(qs, ks, vs, dot_precision=prec, bid=bid, share_cumsum=share, shift=SHIFT)
        out.backward(dout.to(DEV))
        assert rel_err(out.detach().cpu(), ref) < tol, prec
        if gtol is None:
            assert all(torch.isfinite(x.grad).all() for x in (qs, ks, vs))
        else:
            check_grads(share, (qs.grad, ks.grad, vs.grad), (rdq, rdk, rdv), gtol)


@pytest.mark.parametrize("key,bid,share", VARIANTS)
def test_bf16_tensors(KB, key, bid, share):
    q, k, v, dout = make_inputs(1, 3, 300, 64, 77, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref, rdq, rdk, rdv = O.variant_backward(qb.float(), kb.float(), vb.float(), dout, bid, share, SHIFT)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    out = KB.dilution_attention(qs, ks, vs, dot_precision="bf16", bid=bid, share_cumsum=share, shift=SHIFT)
    out.backward(dout.to(DEV))
    assert (out.detach().cpu() - ref).abs().max().item() < 2e-2
    assert qs.grad.dtype == ks.grad.dtype == vs.grad.dtype == torch.bfloat16
    check_grads(share, (qs.grad, ks.grad, vs.grad), (rdq, rdk, rdv), 2e-2)


ROW_SUM = ("relu", "relu2", "softplus", "minshift")     # f(a) / rowsum(f): the tile kernels, always


@pytest.mark.parametrize("seq", [300, 1100, 2049])
@pytest.mark.parametrize("key,bid,share", [x for x in VARIANTS if x[1] not in ROW_SUM])
def test_bf16_head_dim_64_runs_on_the_tensor_core_kernels(KB, key, bid, share, seq):
    """bf16 tensors with heads of 64 under "bf16": the tcgen05 kernels instantiated for the bid and
    share step (not the tile kernels), forward and backward, at ragged lengths."""
    pkg = load_package()
    q, k, v, dout = make_inputs(2, 2, seq, 64, 31 + seq, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref, rdq, rdk, rdv = O.variant_backward(qb.float(), kb.float(), vb.float(), dout, bid, share, SHIFT)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    pkg._lib.profile(True)
    pkg._lib.profile_collect()
    out = KB.dilution_attention(qs, ks, vs, dot_precision="bf16", bid=bid, share_cumsum=share, shift=SHIFT)
    out.backward(dout.to(DEV))
    torch.cuda.synchronize()
    names = set(pkg._lib.profile_collect())
    pkg._lib.profile(False)
    assert {"tc_forward_main", "tc_backward_main"} <= names, names
    assert not any(n.startswith("simt_") for n in names), names
    assert ("tc_colsum_scan" in names) == (share is not False)      # nothing reads checkpoints without a share step
    assert ("tc_rowstats_pk" in names) == (bid == "softmax" and share is not False)
    assert ("tc_backward_key_correction" in names) == (bid == "softmax" and share is not False)
    assert (out.detach().cpu() - ref).abs().max().item() < 2e-2
    check_grads(share, (qs.grad, ks.grad, vs.grad), (rdq, rdk, rdv), 2e-2)
    # forward only, with the demand totals
    out2, aux = KB.dilution_attention_forward(qs.detach(), ks.detach(), vs.detach(), dot_precision="bf16",
                                              return_aux=True, bid=bid, share_cumsum=share, shift=SHIFT)
    assert (out2.cpu() - ref).abs().max().item() < 2e-2
    assert rel_err(aux["committed_total"].cpu(), O.variant_bids(qb.float(), kb.float(), bid, SHIFT).sum(-2)) < 2e-2


@pytest.mark.parametrize("key,bid,share", [x for x in VARIANTS if x[1] in ROW_SUM])
def test_row_sum_bids_on_bf16_heads_of_64_take_the_tile_kernels(KB, key, bid, share):
    """The four f(a) / rowsum(f) bids have no tcgen05 instantiation: bf16 tensors with heads of 64
    run on the tile kernels (tf32 products, exact on bf16 values), with the row statistics, the
    saved jac K product and the key correction of a row-normalised bid."""
    pkg = load_package()
    q, k, v, dout = make_inputs(2, 2, 520, 64, 71, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref, rdq, rdk, rdv = O.variant_backward(qb.float(), kb.float(), vb.float(), dout, bid, share, SHIFT)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    pkg._lib.profile(True)
    pkg._lib.profile_collect()
    out = KB.dilution_attention(qs, ks, vs, dot_precision="bf16", bid=bid, share_cumsum=share, shift=SHIFT)
    out.backward(dout.to(DEV))
    torch.cuda.synchronize()
    names = set(pkg._lib.profile_collect())
    pkg._lib.profile(False)
    assert "simt_backward_main" in names and not any(n.startswith("tc_") for n in names), names
    # under a share step ghat comes from a sweep of its own and is subtracted before the (unbounded)
    # Jacobian factor multiplies: no correction pass afterwards
    assert ("simt_backward_ghat" in names) == (share is not False)
    assert "simt_backward_dk_correction" not in names
    assert (out.detach().cpu() - ref).abs().max().item() < 2e-2
    check_grads(share, (qs.grad, ks.grad, vs.grad), (rdq, rdk, rdv), 2e-2)


def test_the_operator_itself_goes_to_the_production_kernels(KB):
    pkg = load_package()
    q, k, v, _ = make_inputs(1, 2, 300, 64, 5, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16().to(DEV) for x in (q, k, v))
    pkg._lib.profile(True)
    pkg._lib.profile_collect()
    got = KB.dilution_attention_forward(qb, kb, vb, dot_precision="bf16", bid="softmax", share_cumsum=True)
    torch.cuda.synchronize()
    names = set(pkg._lib.profile_collect())
    pkg._lib.profile(False)
    assert "tc_forward_main" in names, names
    assert torch.equal(got, pkg.kernels.dilution_attention_forward(qb, kb, vb, dot_precision="bf16"))


def test_unknown_bids_raise(KB):
    q, k, v, _ = make_inputs(1, 1, 16, 32, 1)
    q, k, v = (x.to(DEV) for x in (q, k, v))
    with pytest.raises(ValueError, match="bid must be one of"):
        KB.dilution_attention(q, k, v, bid="tanh")
    with pytest.raises(ValueError, match="dot_precision must be one of"):
        KB.dilution_attention_forward(q, k, v, dot_precision="fp8", bid="sigmoid")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("key,bid,share", VARIANTS)
def test_decode_steps_from_a_prefilled_cache(KB, key, bid, share, dtype, tol):
    """Prefill with return_aux, then cached steps: each step's row and the accumulator against
    the oracle's decode step on the same cache (kernels_bid.py:962-1012)."""
    b, h, d, prefix, steps, cap = 2, 3, 64, 150, 5, 160
    q, k, v, _ = make_inputs(b, h, prefix + steps, d, 4100, scales=(0.5, 0.5, 1.0, 1.0))
    q, k, v = (x.to(dtype) for x in (q, k, v))
    _, aux = KB.dilution_attention_forward(q[:, :, :prefix].to(DEV), k[:, :, :prefix].to(DEV), v[:, :, :prefix].to(DEV),
                                           dot_precision="ieee" if dtype == torch.float32 else "bf16",
                                           return_aux=True, bid=bid, share_cumsum=share, shift=SHIFT)
    demand = O.variant_bids(q[:, :, :prefix], k[:, :, :prefix], bid, SHIFT).sum(-2)
    assert rel_err(aux["committed_total"].cpu(), demand) < (1e-5 if dtype == torch.float32 else 2e-2)
    kc = torch.zeros(b, h, cap, d, dtype=dtype)
    vc = torch.zeros(b, h, cap, d, dtype=dtype)
    kc[:, :, :prefix + steps], vc[:, :, :prefix + steps] = k, v
    committed = torch.zeros(b, h, cap)
    committed[:, :, :prefix] = demand
    kd, vd, cd = kc.to(DEV), vc.to(DEV), committed.to(DEV)
    for s in range(steps):
        length = prefix + s + 1
        q1 = q[:, :, length - 1:length]
        want = O.variant_decode_step(q1, kc, vc, committed, length, bid, share, SHIFT)
        got = KB.dilution_decode_step(q1.to(DEV), kd, vd, cd, length, bid=bid, share_cumsum=share, shift=SHIFT)
        assert got.dtype == dtype and got.shape == (b, h, 1, d)
        assert rel_err(got.float().cpu(), want) < tol, s
    assert rel_err(cd.cpu(), committed) < 1e-5
    assert cd[:, :, prefix + steps:].abs().max().item() == 0


@pytest.mark.parametrize("bid", ["relu", "relu2", "softplus", "minshift", "sigmoid", "expshift", "sigshift"])
def test_bid_model_kernel_matches_eager(bid):
    """tests/test_kernels.py:361-376 of the reference, as it stands there: an fp32 model with a
    dilution layer under each bid and a softmax layer, eager logits against the kernel path."""
    if not os.path.isdir(os.path.join(REF, "dilution")):
        pytest.skip("no installed copy of the reference under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from dilution.config import ModelConfig
    from dilution.model import DilutionLM
    pkg = load_package()
    torch.manual_seed(7)
    cfg = ModelConfig(vocab_size=128, n_layers=2, d_model=64, n_heads=2, context_length=96,
                      layer_attention=["dilution", "softmax"], bid=bid)
    model = DilutionLM(cfg).to(DEV).eval()
    idx = torch.randint(0, 128, (2, 96), device=DEV)
    pkg.install()
    try:
        with torch.no_grad():
            eager, _ = model(idx)
            before = pkg._lib.launch_count()
            model.enable_dilution_kernel()
            fused, _ = model(idx)
        assert pkg._lib.launch_count() > before
        assert (eager - fused).abs().max().item() < 5e-2
    finally:
        pkg.uninstall()


@pytest.mark.parametrize("dtype,d,length", [(torch.bfloat16, 64, 5000), (torch.float32, 32, 2100), (torch.float32, 128, 1)])
@pytest.mark.parametrize("bid,share", [("relu", True), ("relu2", "exclusive"), ("softplus", True), ("minshift", True),
                                       ("minshift", False), ("sigshift", True)])
def test_decode_long_rows_many_chunks(KB, bid, share, dtype, d, length):
    """Rows split over many key chunks: the chunk statistics of an f(a) / rowsum(f) bid — (minimum,
    mass) — are combined across chunks, random demand, spare rows untouched, caches read-only.
    A single-key row has no mass under minshift: the uniform fall-back (kernels_bid.py:944)."""
    b, h, cap = 2, 3, length + 5
    g = torch.Generator().manual_seed(length + d)
    kc = torch.randn(b, h, cap, d, generator=g).mul(0.5).to(dtype)
    vc = torch.randn(b, h, cap, d, generator=g).to(dtype)
    q1 = torch.randn(b, h, 1, d, generator=g).mul(0.5).to(dtype)
    committed = torch.rand(b, h, cap, generator=g)
    committed[:, :, length - 1:] = 0
    want_c = committed.clone()
    want = O.variant_decode_step(q1, kc, vc, want_c, length, bid, share, SHIFT)
    dk, dv, dc = kc.to(DEV), vc.to(DEV), committed.to(DEV)
    got = KB.dilution_decode_step(q1.to(DEV), dk, dv, dc, length, bid=bid, share_cumsum=share, shift=SHIFT)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert rel_err(got.float().cpu(), want) < tol
    assert rel_err(dc.cpu(), want_c) < 1e-5
    assert torch.equal(dc[:, :, length:].cpu(), committed[:, :, length:])
    assert torch.equal(dk.cpu(), kc) and torch.equal(dv.cpu(), vc)


def test_variant_decode_appends_through_the_c_abi():
    """k1 / v1 given: the call writes the new token's rows and treats its demand as zero."""
    pkg = load_package()
    lib, L = pkg._lib.load(), pkg._lib
    n, d, cap, length = 6, 32, 64, 41
    g = torch.Generator().manual_seed(3)
    kc = torch.randn(1, n, cap, d, generator=g) * 0.5
    vc = torch.randn(1, n, cap, d, generator=g)
    q1 = torch.randn(1, n, 1, d, generator=g)
    committed = torch.rand(1, n, cap, generator=g)
    committed[:, :, length - 1:] = 0
    k_new, v_new = kc[:, :, length - 1].clone(), vc[:, :, length - 1].clone()
    want_c = committed.clone()
    want = O.variant_decode_step(q1, kc, vc, want_c, length, "sigmoid", "exclusive")
    kd, vd = kc.clone(), vc.clone()
    kd[:, :, length - 1], vd[:, :, length - 1] = 7.0, 7.0           # stale rows the call must overwrite
    kd, vd, cd = kd.to(DEV), vd.to(DEV), committed.clone().to(DEV)
    cd[:, :, length - 1] = 5.0                                      # stale demand the call must ignore
    out = torch.empty(n, d, device=DEV)
    scratch = torch.empty(lib.dilution_decode_scratch_bytes(n, length, d), device=DEV, dtype=torch.uint8)
    qd, k1, v1 = q1.reshape(n, d).to(DEV), k_new.reshape(n, d).to(DEV), v_new.reshape(n, d).to(DEV)
    L.check(lib.dilution_variant_decode(qd.data_ptr(), k1.data_ptr(), v1.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                                        L.F32, n, cap, length, d, d ** -0.5, 1e-9, L.BID["sigmoid"], 2, 1.0,
                                        cd.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream), "dilution_variant_decode")
    assert rel_err(out.cpu().view(1, n, 1, d), want) < 1e-4
    assert rel_err(cd.cpu(), want_c) < 1e-5
    assert torch.equal(kd.cpu()[:, :, length - 1], k_new) and torch.equal(vd.cpu()[:, :, length - 1], v_new)


@pytest.mark.parametrize("bid,share", [("sigmoid", True), ("sigmoid", "exclusive"), ("softmax", "exclusive"),
                                       ("softmax", False), ("sigshift", True), ("expshift", True),
                                       ("relu", True), ("softplus", True), ("relu2", False)])
def test_reference_model_with_a_variant_configuration(bid, share):
    """The unmodified DilutionLM configured with an ablation binds dilution.kernels_bid
    (model.py:145-156): after install() its kernel path runs here and must reproduce the eager
    logits, in the full forward and in prefill + cached steps.  (minshift is left to the
    operator-level tests: the key at a row's minimum gets no mass at all, so in a row of three
    keys a near-tie that the model's "tf32" products resolve the other way moves the output by
    O(1) — in the reference's kernels as much as here; under "ieee" the same tensors agree to 1e-7.)"""
    if not os.path.isdir(os.path.join(REF, "dilution")):
        pytest.skip("no installed copy of the reference under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from dilution.config import ModelConfig
    from dilution.model import DilutionLM
    pkg = load_package()
    cfg = ModelConfig(context_length=128, vocab_size=256, n_layers=2, n_heads=4, d_model=128,
                      attention="dilution", bid=bid, share_cumsum=share)
    torch.manual_seed(0)
    model = DilutionLM(cfg).to(DEV).eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 48), device=DEV)
    prefix = 40

    def run():
        logits, caches = model.prefill(tokens[:, :prefix])
        outs = [logits[:, -1]]
        for pos in range(prefix, tokens.shape[1]):
            outs.append(model.decode_step(tokens[:, pos:pos + 1], pos, caches)[:, -1])
        return torch.stack(outs, dim=1)

    pkg.install()
    try:
        with torch.no_grad():
            eager_full, _ = model(tokens, tokens)
            eager_steps = run()
            before = pkg._lib.launch_count()
            model.enable_dilution_kernel()
            kernel_full, _ = model(tokens, tokens)
            kernel_steps = run()
        assert pkg._lib.launch_count() > before
        assert (kernel_full - eager_full).abs().max().item() < 2e-2
        assert (kernel_steps - eager_steps).abs().max().item() < 2e-2
    finally:
        pkg.uninstall()
