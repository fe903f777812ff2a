"""The model's other attention pieces on this library: the fused head split with RoPE
(model.py:59-67, rope.py:26-44), the cached step of a softmax layer (model.py:112-117) and
the patched reference model end to end."""

from __future__ import annotations

import os
import sys

import pytest
import torch

from conftest import ROOT, load_package, rel_err
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF = os.path.join(ROOT, "baseline", "_ref")


class _Rope:            # what split_heads_rope reads of a RopeModule
    def __init__(self, dim, theta=10000.0):
        self.dim, self.theta = dim, theta


@pytest.mark.parametrize("heads,d,seq,offset,with_rope", [(4, 64, 130, 0, True), (2, 32, 33, 17, True),
                                                          (2, 128, 65, 5, True), (3, 64, 50, 0, False)])
def test_split_heads_rope_forward_and_backward(pkg, heads, d, seq, offset, with_rope):
    L = pkg.layers
    g = torch.Generator().manual_seed(seq)
    qkv = torch.randn(2, seq, 3 * heads * d, generator=g).bfloat16()
    theta = 10000.0 if with_rope else None
    rq, rk, rv = O.split_heads(qkv, heads, offset, theta)
    x = qkv.to(DEV).requires_grad_(True)
    q, k, v = L.split_heads_rope(x, heads, _Rope(d) if with_rope else None, offset)
    assert q.is_contiguous() and q.shape == (2, heads, seq, d)
    assert torch.equal(v.cpu(), rv)
    # the kernel follows the reference's bf16 arithmetic operation by operation
    for got, ref in ((q, rq), (k, rk)):
        diff = (got.float().cpu() - ref.float()).abs()
        assert diff.max().item() <= 2 ** -7 * ref.float().abs().max().item()
        assert (diff > 0).float().mean().item() < 1e-3
    # backward: the transpose of the rotation, against fp32 autograd through the oracle
    gq, gk, gv = (torch.randn(2, heads, seq, d, generator=g).bfloat16() for _ in range(3))
    (q.float() * gq.to(DEV).float()).sum().backward(retain_graph=True)
    xr = qkv.float().requires_grad_(True)
    oq, ok, ov = O.split_heads(xr, heads, offset, theta)
    ((oq * gq.float()).sum()).backward()
    assert rel_err(x.grad.float().cpu(), xr.grad) < 2e-2
    x.grad = None
    (k.float() * gk.to(DEV).float()).sum().backward(retain_graph=True)
    (v.float() * gv.to(DEV).float()).sum().backward()
    xr.grad = None
    oq, ok, ov = O.split_heads(xr, heads, offset, theta)
    ((ok * gk.float()).sum() + (ov * gv.float()).sum()).backward()
    assert rel_err(x.grad.float().cpu(), xr.grad) < 2e-2


@pytest.mark.parametrize("dtype,d,prefix", [(torch.bfloat16, 64, 300), (torch.float32, 32, 40)])
def test_softmax_decode_append_matches_attention_rows(pkg, dtype, d, prefix):
    b, h, steps = 2, 3, 6
    total = prefix + steps
    g = torch.Generator().manual_seed(prefix)
    q, k, v = (torch.randn(b, h, total, d, generator=g).to(dtype) for _ in range(3))
    rows = O.softmax_attention(q.float(), k.float(), v.float())
    cache = {"k": torch.zeros(b, h, total + 2, d, device=DEV, dtype=dtype), "len": prefix}
    cache["v"] = torch.zeros_like(cache["k"])
    cache["k"][:, :, :prefix], cache["v"][:, :, :prefix] = k[:, :, :prefix].to(DEV), v[:, :, :prefix].to(DEV)
    for t in range(prefix, total):
        y = pkg.layers.softmax_decode_append_step(q[:, :, t:t + 1].to(DEV), k[:, :, t:t + 1].to(DEV),
                                                  v[:, :, t:t + 1].to(DEV), cache)
        assert cache["len"] == t + 1 and y.dtype == dtype
        assert (y[:, :, 0].float().cpu() - rows[:, :, t]).abs().max().item() < (1e-4 if dtype == torch.float32 else 2e-2)
    assert torch.equal(cache["k"][:, :, :total].cpu(), k) and torch.equal(cache["v"][:, :, :total].cpu(), v)
    assert cache["k"][:, :, total:].abs().max().item() == 0


def test_patched_alternating_model_matches_eager(pkg):
    """install() + install_layers() on the reference's model: an alternating softmax+RoPE /
    dilution stack under bf16 autocast — prefill, cached greedy steps and a training step stay
    within bf16 noise of the unpatched eager model."""
    if not os.path.isdir(os.path.join(REF, "dilution")):
        pytest.skip("no installed copy of the reference under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from dilution.config import ModelConfig
    from dilution.model import DilutionLM
    cfg = ModelConfig(context_length=400, vocab_size=512, n_layers=4, n_heads=4, d_model=256,
                      layer_attention=["softmax", "dilution"] * 2, positional="rope_alt", mlp="swiglu",
                      ffn_hidden=512)
    torch.manual_seed(2)
    model = DilutionLM(cfg).to(DEV).eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 330), device=DEV)
    prefix = 300

    def run():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            logits, caches = model.prefill(tokens[:, :prefix])
            outs = [logits[:, -1].float()]
            for pos in range(prefix, tokens.shape[1]):
                logits = model.decode_step(tokens[:, pos:pos + 1], pos, caches)
                outs.append(logits[:, -1].float())
        return torch.stack(outs, dim=1)

    def train():
        model.train()
        model.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        model.eval()
        return loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters()}

    eager = run()
    eager_loss, eager_grads = train()
    pkg.install(fused_decode=True)
    pkg.layers.install_layers()
    try:
        model.enable_dilution_kernel()
        before = pkg._lib.launch_count()
        pkg._lib.profile(True)
        pkg._lib.profile_collect()
        got = run()
        loss, grads = train()
        torch.cuda.synchronize()
        names = set(pkg._lib.profile_collect())
        pkg._lib.profile(False)
    finally:
        pkg.layers.uninstall_layers()
        pkg.uninstall()
    assert {"split_heads_rope", "merge_heads_rope_grad", "tc_softmax_forward", "decode_scores"} <= names, names
    assert pkg._lib.launch_count() > before
    assert torch.isfinite(got).all()
    assert (got - eager).abs().max().item() < 6e-2
    assert abs(loss - eager_loss) < 2e-2
    for n, gr in eager_grads.items():
        err = (grads[n] - gr).abs().max().item() / (gr.abs().max().item() + 1e-12)
        assert err < 1e-1, (n, err)


def test_graphed_decode_replays_the_layer_loop(pkg):
    """GraphedDecode: the model's decode_step recorded once into a CUDA graph (length and position
    read from the device) against the same model stepping launch by launch — same logits, same
    caches, same demand; and the model's own decode_step takes over again after close()."""
    if not os.path.isdir(os.path.join(REF, "dilution")):
        pytest.skip("no installed copy of the reference under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from dilution.config import ModelConfig
    from dilution.model import DilutionLM
    cfg = ModelConfig(context_length=400, vocab_size=512, n_layers=4, n_heads=4, d_model=256,
                      layer_attention=["softmax", "dilution"] * 2, positional="rope_alt", mlp="swiglu",
                      ffn_hidden=512)
    torch.manual_seed(5)
    model = DilutionLM(cfg).to(DEV).eval()
    tokens = torch.randint(0, cfg.vocab_size, (3, 340), device=DEV)
    prefix, graphed_until = 300, 330
    pkg.install(fused_decode=True)
    pkg.layers.install_layers()
    try:
        model.enable_dilution_kernel()
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            # launch by launch
            logits, caches = model.prefill(tokens[:, :prefix], capacity=360)
            want = []
            for pos in range(prefix, tokens.shape[1]):
                want.append(model.decode_step(tokens[:, pos:pos + 1], pos, caches)[:, -1].float())
            # recorded
            logits, caches_g = model.prefill(tokens[:, :prefix], capacity=360)
        dec = pkg.GraphedDecode(model, caches_g)
        before = pkg._lib.launch_count()
        got = [dec.step(tokens[:, pos:pos + 1])[:, -1].float().clone() for pos in range(prefix, graphed_until)]
        assert dec.graph is not None and int(dec.pos_dev.item()) == graphed_until == dec.position
        # replays launch nothing through the library's host code: the eager step and the recorded one only
        assert pkg._lib.launch_count() - before <= 2 * 4 * 5
        dec.close()
        assert all("pos_dev" not in c and c["len"] == graphed_until for c in caches_g)
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            for pos in range(graphed_until, tokens.shape[1]):       # the model's own loop again
                got.append(model.decode_step(tokens[:, pos:pos + 1], pos, caches_g)[:, -1].float())
        torch.cuda.synchronize()
    finally:
        pkg.layers.uninstall_layers()
        pkg.uninstall()
    got, want = torch.stack(got, 1), torch.stack(want, 1)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() < 2e-2
    for c, e in zip(caches_g, caches):
        assert c["len"] == e["len"] == tokens.shape[1]
        assert (c["k"].float() - e["k"].float()).abs().max().item() < 2e-2
        if "committed" in c:
            assert (c["committed"] - e["committed"]).abs().max().item() < 1e-2
    with pytest.raises(ValueError, match="ignores the position"):
        pkg.GraphedDecode(DilutionLM(ModelConfig(context_length=64, vocab_size=64, n_layers=1, n_heads=2, d_model=64,
                                                 positional="learned")), [{"k": caches[0]["k"], "len": 1}])
