"""The reference's own model on these kernels: `install()` onto the real
`dilution.kernels`, `DilutionLM.enable_dilution_kernel()`, and the reference's two
model-level parity tests (tests/test_kernels.py:79-95 and :245-273) with the
unmodified `DilutionLM` — kernel logits against eager logits, fused decode against
eager decode against the full forward — which drive `begin_cache`, `step_cache`,
`_alloc_cache` and `_append_kv` (model.py:76-93, 198-240).

The reference package is not part of this repository.  An installed copy is looked
for under baseline/_ref (pip --target of the reference checkout); without it these
tests are skipped.
"""

from __future__ import annotations

import os
import sys

import pytest
import torch

from conftest import ROOT, load_package

pytestmark = pytest.mark.gpu
REF = os.path.join(ROOT, "baseline", "_ref")
DEV = "cuda"


@pytest.fixture()
def ref():
    """The reference package with this backend installed; put back afterwards."""
    if not os.path.isdir(os.path.join(REF, "dilution")):
        pytest.skip("no installed copy of the reference under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import dilution.kernels as rk
    from dilution.config import ModelConfig
    from dilution.model import DilutionLM
    pkg = load_package()
    pkg.install()
    assert rk.dilution_attention is pkg.kernels.dilution_attention and rk.HAS_TRITON is True
    yield dict(kernels=rk, ModelConfig=ModelConfig, DilutionLM=DilutionLM, pkg=pkg)
    pkg.uninstall()


def _launches(pkg):
    return pkg._lib.launch_count()


def test_model_kernel_path_matches_eager(ref):
    """tests/test_kernels.py:79-95: enable_dilution_kernel() must not change eval logits."""
    cfg = ref["ModelConfig"](context_length=128, vocab_size=256, n_layers=2, n_heads=4,
                             d_model=128, attention="dilution")
    torch.manual_seed(0)
    model = ref["DilutionLM"](cfg).to(DEV).eval()
    idx = torch.randint(0, cfg.vocab_size, (2, 128), device=DEV)
    with torch.no_grad():
        eager_logits, _ = model(idx, idx)
        before = _launches(ref["pkg"])
        model.enable_dilution_kernel()
        kernel_logits, _ = model(idx, idx)
    assert _launches(ref["pkg"]) >= before + 2 * 3          # three passes per dilution layer ran here
    assert torch.isfinite(kernel_logits).all()
    assert (kernel_logits - eager_logits).abs().max().item() < 2e-2


@pytest.mark.parametrize("fused", [False, True])
def test_model_kernel_decode_matches_eager_decode(ref, fused):
    """tests/test_kernels.py:245-273: prefill + cached steps on the kernels reproduce the eager
    cached steps and the full forward.  fused=True also replaces step_cache by the version that
    hands the new token's k, v to the decode kernels instead of calling _append_kv first."""
    cfg = ref["ModelConfig"](context_length=128, vocab_size=256, n_layers=2, n_heads=4,
                             d_model=128, attention="dilution")
    torch.manual_seed(0)
    model = ref["DilutionLM"](cfg).to(DEV).eval()
    tokens = torch.randint(0, cfg.vocab_size, (2, 40), device=DEV)
    prefix = 24

    def run():
        logits, caches = model.prefill(tokens[:, :prefix])
        outs = [logits[:, -1]]
        for pos in range(prefix, tokens.shape[1]):
            logits = model.decode_step(tokens[:, pos:pos + 1], pos, caches)
            outs.append(logits[:, -1])
        return torch.stack(outs, dim=1), caches

    with torch.no_grad():
        eager, eager_caches = run()
        if fused:
            ref["pkg"].install(fused_decode=True)
        before = _launches(ref["pkg"])
        model.enable_dilution_kernel()
        got, caches = run()
        full, _ = model(tokens, tokens)
    assert _launches(ref["pkg"]) > before
    assert torch.isfinite(got).all()
    assert (got - eager).abs().max().item() < 2e-2
    assert (got - full[:, prefix - 1:]).abs().max().item() < 2e-2
    for c, e in zip(caches, eager_caches):          # the cache dict the model owns (model.py:76-83, 224-228)
        assert c["len"] == e["len"] == tokens.shape[1]
        # layer 0 sees identical inputs; later layers see the earlier layers' outputs
        assert (c["k"] - e["k"]).abs().max().item() < 1e-3 and (c["v"] - e["v"]).abs().max().item() < 1e-3
        assert c["k"][:, :, c["len"]:].abs().max().item() == 0
        assert (c["committed"] - e["committed"]).abs().max().item() < 1e-4
        assert c["committed"][:, :, c["len"]:].abs().max().item() == 0


def test_alternating_model_bf16_autocast_trains_on_the_tensor_core_kernels(ref):
    """An alt-style stack (softmax with RoPE / dilution, heads of 64) under bf16 autocast, as the
    end-to-end LM workload runs it: the dilution layers receive bf16 transposed views of the
    fused c_attn output, run forward and backward on the tcgen05 kernels, and logits, loss and
    parameter gradients stay within bf16 noise of the eager model."""
    cfg = ref["ModelConfig"](context_length=512, vocab_size=512, n_layers=4, n_heads=4, d_model=256,
                             layer_attention=["softmax", "dilution"] * 2, positional="rope_alt",
                             mlp="swiglu", ffn_hidden=512)
    torch.manual_seed(1)
    model = ref["DilutionLM"](cfg).to(DEV).train()
    idx = torch.randint(0, cfg.vocab_size, (2, 512), device=DEV)
    tgt = torch.randint(0, cfg.vocab_size, (2, 512), device=DEV)

    def step():
        model.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, loss = model(idx, tgt)
        loss.backward()
        grads = {n: p.grad.detach().float().clone() for n, p in model.named_parameters()}
        return logits.detach().float(), loss.item(), grads

    eager_logits, eager_loss, eager_grads = step()
    pkg = ref["pkg"]
    pkg._lib.profile(True)
    pkg._lib.profile_collect()
    model.enable_dilution_kernel()
    logits, loss, grads = step()
    torch.cuda.synchronize()
    names = set(pkg._lib.profile_collect())
    pkg._lib.profile(False)
    assert "tc_backward_main" in names and \
        ({"tc_forward_fused"} <= names or {"tc_colsum_scan", "tc_forward_main"} <= names), names
    assert names & {"tc_rowstats", "tc_rowstats_pk"} and \
        names & {"tc_backward_correction", "tc_backward_key_correction"}, names
    assert not any(n.startswith("simt_") for n in names), names
    assert torch.isfinite(logits).all()
    assert (logits - eager_logits).abs().max().item() < 5e-2
    assert abs(loss - eager_loss) < 2e-2
    for n, gr in eager_grads.items():
        err = (grads[n] - gr).abs().max().item() / (gr.abs().max().item() + 1e-12)
        assert err < 1e-1, (n, err)                      # the reference's bf16-mode bound


def test_generate_greedy_matches_eager_tokens(ref):
    """DilutionLM.generate (model.py:472-512) end to end on the kernels: same greedy tokens."""
    cfg = ref["ModelConfig"](context_length=96, vocab_size=64, n_layers=2, n_heads=2, d_model=64,
                             attention="dilution")
    torch.manual_seed(3)
    model = ref["DilutionLM"](cfg).to(DEV).eval()
    prompt = torch.randint(0, cfg.vocab_size, (3, 30), device=DEV)
    eager = model.generate(prompt, 20)
    ref["pkg"].install(fused_decode=True)
    model.enable_dilution_kernel()
    fused = model.generate(prompt, 20)
    agree = (eager == fused).float().mean().item()
    assert agree > 0.95, agree       # near-ties in fp32 logits may flip a late token
