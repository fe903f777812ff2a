"""The key-stationary training forward (dilution_forward_fused: passes 2 and 3 in one sweep)
against the column-sum pass + query-stationary main pass it replaces and against the oracle:
output, share row sums, demand totals and every checkpoint a backward reads."""

from __future__ import annotations

import math

import pytest
import torch

from conftest import load_package, make_inputs, rel_err
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _both_paths(qb, kb, vb):
    """(out, aux) of a training forward with and without the fused sweep."""
    K = load_package().kernels
    res = {}
    for fused in (True, False):
        saved, K.TC_FUSED_FORWARD = K.TC_FUSED_FORWARD, fused
        try:
            res[fused] = K.dilution_attention_forward(qb, kb, vb, dot_precision="bf16", return_aux=True,
                                                      _save_pk=True, _training=True)
        finally:
            K.TC_FUSED_FORWARD = saved
    torch.cuda.synchronize()
    return res[True], res[False]


@pytest.mark.parametrize("seq", [64, 130, 256, 257, 700, 1025, 2049])
def test_fused_forward_matches_the_two_pass_forward_and_the_oracle(seq):
    pkg = load_package()
    q, k, v, _ = make_inputs(2, 3, seq, 64, 900 + seq, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16().to(DEV) for x in (q, k, v))
    pkg._lib.profile(True)
    pkg._lib.profile_collect()
    (out_f, aux_f), (out_u, aux_u) = _both_paths(qb, kb, vb)
    names = set(pkg._lib.profile_collect())
    pkg._lib.profile(False)
    assert {"tc_forward_fused", "tc_colsum_scan", "tc_forward_main"} <= names, names
    ref, demand = O.dilution_chunked(qb.float().cpu(), kb.float().cpu(), vb.float().cpu(), chunk=512,
                                     return_demand=True)
    assert (out_f.cpu() - ref).abs().max().item() < 2e-2
    assert (out_f - out_u).abs().max().item() < 1e-2           # both round their shares to bf16
    assert rel_err(aux_f["committed_total"].cpu(), demand) < 2e-2
    assert rel_err(aux_f["committed_total"].cpu(), aux_u["committed_total"].cpu()) < 1e-4
    assert rel_err(aux_f["ssum"].cpu(), aux_u["ssum"].cpu()) < 1e-2
    assert aux_f["bwd_block_m"] == aux_u["bwd_block_m"] == 32
    # every checkpoint a consumer reads: row block rb, keys a query of that block can see
    cf, cu = aux_f["carry"].cpu(), aux_u["carry"].cpu()
    scale = max(1.0, cu[:, -1, :].abs().max().item())
    for rb in range(cf.shape[1]):
        end = min((rb + 1) * 32, seq)
        assert (cf[:, rb, :end] - cu[:, rb, :end]).abs().max().item() < 1e-4 * scale, rb


@pytest.mark.parametrize("seq", [300, 1100])
def test_training_step_through_the_fused_forward(seq):
    """Gradients with the fused forward in front of the unchanged backward."""
    K = load_package().kernels
    assert K.TC_FUSED_FORWARD
    q, k, v, dout = make_inputs(1, 4, seq, 64, 40 + seq, scales=(0.5, 0.5, 1.0, 1e-2))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    ref, rdq, rdk, rdv = O.dilution_backward(qb.float(), kb.float(), vb.float(), dout)
    qs, ks, vs = (x.to(DEV).requires_grad_(True) for x in (qb, kb, vb))
    out = K.dilution_attention(qs, ks, vs, dot_precision="bf16")
    out.backward(dout.to(DEV))
    assert (out.detach().cpu() - ref).abs().max().item() < 2e-2
    for name, r, t in (("dq", rdq, qs), ("dk", rdk, ks), ("dv", rdv, vs)):
        assert rel_err(t.grad.float().cpu(), r) < 3e-2, name


def test_fused_forward_refuses_what_it_is_not_built_for():
    pkg = load_package()
    lib, L = pkg._lib.load(), pkg._lib
    x = torch.zeros(1, 64, 128, device=DEV)
    s = torch.zeros(1, 64, device=DEV)
    rc = lib.dilution_forward_fused(x.data_ptr(), x.data_ptr(), x.data_ptr(), L.F32, L.PREC["ieee"], 1, 64, 128,
                                    1.0 / math.sqrt(128), 1e-9, s.data_ptr(), s.data_ptr(), x.data_ptr(),
                                    s.data_ptr(), x.data_ptr(), s.data_ptr(), None)
    assert rc == 2 and b"head_dim 64" in lib.dilution_last_error()
