"""Call patterns around the operator rather than its arithmetic: streams, partial gradients,
strided upstream gradients, and a first call from a thread that has no CUDA context yet."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

from conftest import make_inputs, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(kernels, q, k, v, dout):
    qs, ks, vs = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = kernels.dilution_attention(qs, ks, vs, dot_precision="bf16")
    out.backward(dout)
    return out.detach(), qs.grad, ks.grad, vs.grad


def test_side_stream_matches_default_stream(kernels):
    """The library launches on the caller's current stream and nowhere else."""
    q, k, v, dout = make_inputs(2, 2, 700, 64, 11, scales=(0.5, 0.5, 1.0, 1e-1))
    q, k, v = (x.bfloat16().to(DEV) for x in (q, k, v))
    dout = dout.to(DEV)
    ref = _run(kernels, q, k, v, dout)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = _run(kernels, q, k, v, dout)
    side.synchronize()
    assert torch.equal(got[0], ref[0])
    assert torch.equal(got[3], ref[3])
    # dq and ghat (hence dk) are accumulated across key blocks with floating-point reductions
    # whose order varies between runs: equal up to the last bits, not bitwise
    assert rel_err(got[1].float().cpu(), ref[1].float().cpu()) < 2e-2
    assert rel_err(got[2].float().cpu(), ref[2].float().cpu()) < 2e-3


def test_partial_gradients_and_strided_upstream_gradient(kernels):
    """Only q requires a gradient; the upstream gradient is a bf16, non-contiguous view."""
    q, k, v, dout = make_inputs(1, 2, 333, 64, 12, scales=(0.5, 0.5, 1.0, 1e-1))
    q, k, v = (x.bfloat16().to(DEV) for x in (q, k, v))
    ref = _run(kernels, q, k, v, dout.bfloat16().float().to(DEV))
    qs = q.clone().requires_grad_(True)
    out = kernels.dilution_attention(qs, k, v, dot_precision="bf16")
    strided = dout.bfloat16().to(DEV).transpose(2, 3).contiguous().transpose(2, 3)
    assert not strided.is_contiguous()
    out.backward(strided)
    assert k.grad is None and v.grad is None
    assert rel_err(qs.grad.float().cpu(), ref[1].float().cpu()) < 2e-2


def test_first_call_in_a_fresh_process(kernels):
    """The backward's first tensor-core call comes from the autograd engine thread, which has
    selected the device but made no CUDA call of its own: encoding the TMA descriptors there
    needs the context to be bound first."""
    code = (
        "import importlib, sys, torch\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "K = importlib.import_module('dilution-attention_b200').kernels\n"
        "g = torch.Generator().manual_seed(0)\n"
        "q, k, v = (torch.randn(1, 3, 1, 64, generator=g).bfloat16().cuda().requires_grad_(True) for _ in range(3))\n"
        "out = K.dilution_attention(q, k, v, dot_precision='bf16')\n"
        "out.backward(torch.ones_like(out))\n"
        "torch.cuda.synchronize()\n"
        "assert torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all() and torch.isfinite(v.grad).all()\n"
        "print('fresh-process ok')\n"
    )
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "fresh-process ok" in res.stdout, res.stderr[-2000:]
