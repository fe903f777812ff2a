"""Pass 1 with a product (tcgen05): the saved query correction pk, the backward that uses
it, and causal softmax attention on the same kernel.  Mirrors tests/test_kernels.py:46-59
(pk against softmax(q k^T) k), :109-127 (gradients) and :349-357 (share_cumsum=False is plain
attention) of the reference."""

from __future__ import annotations

import math

import pytest
import torch
import torch.nn.functional as F

from conftest import make_inputs, rel_err
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[True, False], ids=["saved_pk", "recomputed_pk"])
def pk_mode(kernels, request):
    old = kernels.TC_SAVE_PK
    kernels.TC_SAVE_PK = request.param
    yield request.param
    kernels.TC_SAVE_PK = old


@pytest.mark.parametrize("seq,scale", [(1, 1.0), (64, 1.0), (129, 1.0), (257, 1.0), (1100, 0.5), (2048, 1.0),
                                       (1024, 4.0), (1024, 8.0)])
def test_saved_pk_and_row_statistics_match_oracle(pkg, kernels, seq, scale):
    """pk = scale * softmax(q k^T) k and the log-sum-exp of every row, also for peaked scores
    (standard deviation 16 and 64), where the lazily moved reference maximum has to rescale."""
    q, k, v, _ = make_inputs(1, 3, seq, 64, 40 + seq, scales=(scale, scale, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    _, aux = kernels.dilution_attention_forward(qb.to(DEV), kb.to(DEV), vb.to(DEV), dot_precision="bf16",
                                                return_aux=True, _save_pk=True)
    ref = O.query_correction(qb.float(), kb.float())
    assert rel_err(aux["pk"].reshape(1, 3, seq, 64).cpu(), ref) < 1e-2
    rmax, rden = O.row_stats(qb.float(), kb.float())
    lse = (aux["rmax"] + torch.log2(aux["rden"])).reshape(1, 3, seq).cpu()
    assert (lse - (rmax + torch.log2(rden))).abs().max().item() < 2e-3
    # (rmax alone is the pass's reference exponent, which lags behind the exact row maximum)
    # the plain row pass gives the same statistics
    _, aux2 = kernels.dilution_attention_forward(qb.to(DEV), kb.to(DEV), vb.to(DEV), dot_precision="bf16",
                                                 return_aux=True)
    lse2 = (aux2["rmax"] + torch.log2(aux2["rden"])).reshape(1, 3, seq).cpu()
    assert (lse - lse2).abs().max().item() < 1e-3


@pytest.mark.parametrize("seq,scales", [(257, (1.0, 1.0, 1.0, 1.0)), (1100, (0.5, 0.5, 1.0, 1e-2)),
                                        (2049, (0.5, 0.5, 1.0, 1.0)), (1024, (4.0, 4.0, 1.0, 1e-1)),
                                        (63, (1.0, 1.0, 1.0, 1.0)), (192, (1.0, 1.0, 1.0, 1.0))])
def test_backward_parity_with_and_without_saved_pk(kernels, pk_mode, seq, scales):
    q, k, v, dout = make_inputs(1, 2, seq, 64, 700 + seq, scales=scales)
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref = O.dilution_backward(qb.float(), kb.float(), vb.float(), dout)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    out = kernels.dilution_attention(qs, ks, vs, dot_precision="bf16")
    out.backward(dout.to(DEV))
    assert (out.detach().cpu() - ref[0]).abs().max().item() < 2e-2
    for name, gr, t in (("dq", ref[1], qs), ("dk", ref[2], ks), ("dv", ref[3], vs)):
        assert torch.isfinite(t.grad).all(), name
        assert rel_err(t.grad.float().cpu(), gr) < 3e-2, name


def test_training_shape_row_at_16384_with_saved_pk(kernels, pk_mode):
    t, d = 16384, 64
    q, k, v, dout = make_inputs(1, 1, t, d, 1551, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref = O.dilution_backward_chunked(qb.float(), kb.float(), vb.float(), dout, chunk=1024)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    kernels.dilution_attention(qs, ks, vs, dot_precision="bf16").backward(dout.to(DEV))
    for name, gr, x in (("dq", ref[1], qs), ("dk", ref[2], ks), ("dv", ref[3], vs)):
        assert rel_err(x.grad.float().cpu(), gr) < 3e-2, name


@pytest.mark.parametrize("seq,scale", [(1, 1.0), (200, 1.0), (513, 1.0), (2048, 0.5), (1024, 6.0)])
def test_softmax_attention_forward_matches_sdpa_semantics(kernels, seq, scale):
    """model.py:96-117: softmax layers call F.scaled_dot_product_attention(is_causal=True)."""
    q, k, v, _ = make_inputs(2, 3, seq, 64, 900 + seq, scales=(scale, scale, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref = O.softmax_attention(qb.float(), kb.float(), vb.float())
    sdpa = F.scaled_dot_product_attention(qb.float(), kb.float(), vb.float(), is_causal=True)
    assert (ref - sdpa).abs().max().item() < 1e-5
    got, lse = kernels.softmax_attention_forward(qb.to(DEV), kb.to(DEV), vb.to(DEV), return_lse=True)
    assert got.dtype == torch.bfloat16 and got.shape == (2, 3, seq, 64)
    assert (got.float().cpu() - ref).abs().max().item() < 2e-2
    rmax, rden = O.row_stats(qb.float(), kb.float())
    ref_lse = (rmax + torch.log2(rden)) * math.log(2.0)
    assert (lse.cpu() - ref_lse).abs().max().item() < 2e-3


def test_softmax_attention_on_model_views(kernels):
    """Transposed views of a fused qkv projection, as the model hands them over (model.py:59-67)."""
    b, t, h, d = 2, 300, 4, 64
    g = torch.Generator().manual_seed(5)
    x = torch.randn(b, t, 3 * h * d, generator=g).bfloat16()
    q, k, v = (y.view(b, t, h, d).transpose(1, 2) for y in x.split(h * d, dim=2))
    got = kernels.softmax_attention_forward(q.to(DEV), k.to(DEV), v.to(DEV))
    assert (got.float().cpu() - O.softmax_attention(q.float(), k.float(), v.float())).abs().max().item() < 2e-2
