"""Failure detection without a GPU fault: a device-side wait that can never be
satisfied gives up after its limit, reports through the status word, and leaves
the context usable for the next launch."""

from __future__ import annotations

import pytest
import torch

from conftest import make_inputs, rel_err
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu


def test_wait_that_nothing_satisfies_gives_up_and_reports(pkg, kernels):
    lib = pkg._lib.load()
    assert lib.dilution_device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.dilution_selftest_bounded_wait(flag.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()                       # the kernel returned by itself
    assert flag.item() == 1                        # ... because its wait ran out
    rc = lib.dilution_device_status()
    assert rc == 4 and b"bounded wait" in lib.dilution_last_error()
    assert lib.dilution_device_status() == 0       # reported once, then cleared
    # the context is intact: a normal tensor-core forward still matches the oracle
    q, k, v, _ = make_inputs(1, 2, 260, 64, 3, scales=(0.5, 0.5, 1.0, 1.0))
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    out = kernels.dilution_attention_forward(qb.cuda(), kb.cuda(), vb.cuda(), dot_precision="bf16")
    assert (out.cpu() - O.dilution_dense(qb.float(), kb.float(), vb.float())).abs().max().item() < 2e-2
