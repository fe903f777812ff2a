"""dilution_decode_static: the decode step with its scratch inside the library.

Some callers cannot allocate device memory when a token is due: the device heap
already belongs to their KV-cache pool, or an allocation would stall the token
loop, or they bind the C ABI from a host without a device allocator.  They call
dilution_decode_static, which takes no scratch pointer.  This test drives it
through the C ABI exactly as such a host would (raw pointers, no torch
allocation between the calls), twice in a row on the same caches, and requires
the same outputs and the same advanced demand as dilution_decode with
caller-provided scratch, and as the CPU oracle's decode step.  One case sits at
the limits of the built-in array (128 rows, head_dim 128, rows x keys = 2^21).
It is collected last so that a failure here cannot
hide any other test.
"""

from __future__ import annotations

import math

import pytest
import torch

from conftest import load_package
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, name, q1, kc, vc, com, out, length, scratch=None):
    n, cap, d = kc.shape
    code = 1 if q1.dtype == torch.bfloat16 else 0
    args = [q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), code, n, cap, length, d,
            1.0 / math.sqrt(d), 1e-9, com.data_ptr(), out.data_ptr()]
    if scratch is not None:
        args.append(scratch.data_ptr())
    args.append(torch.cuda.current_stream().cuda_stream)
    return getattr(lib, name)(*args)


@pytest.mark.parametrize("dtype,d,n,length", [(torch.bfloat16, 64, 8, 3000), (torch.float32, 32, 5, 77),
                                              (torch.bfloat16, 128, 128, 16383)])
def test_static_scratch_decode_equals_decode_with_scratch_twice(dtype, d, n, length):
    pkg = load_package()
    lib = pkg._lib.load()
    cap = length + 4
    g = torch.Generator().manual_seed(length)
    kc_h = torch.randn(n, cap, d, generator=g).to(dtype)
    vc_h = torch.randn(n, cap, d, generator=g).to(dtype)
    kc, vc = kc_h.to(DEV), vc_h.to(DEV)
    qs_h = [torch.randn(n, d, generator=g).to(dtype) for _ in range(2)]
    qs = [x.to(DEV) for x in qs_h]
    com0 = torch.rand(n, cap, generator=g)
    com0[:, length - 1:] = 0
    com_ref = com0.clone()
    com_a, com_b = com0.to(DEV), com0.to(DEV)
    out_a = torch.empty(n, d, device=DEV, dtype=dtype)
    out_b = torch.empty_like(out_a)
    scratch = pkg.kernels.decode_scratch(n, cap, d, DEV)
    tol = 1e-5 if dtype == torch.float32 else 2e-2      # the decode tests' tolerances
    for step in range(2):                                # second call reuses the shared array
        ln = length + step
        assert _call(lib, "dilution_decode", qs[step], kc, vc, com_a, out_a, ln, scratch) == 0
        rc = _call(lib, "dilution_decode_static", qs[step], kc, vc, com_b, out_b, ln)
        assert rc == 0, lib.dilution_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(out_b.float()).all()
        assert (out_a.float() - out_b.float()).abs().max().item() <= tol
        assert (com_a - com_b).abs().max().item() <= 1e-6
        assert com_b[:, ln:].abs().max().item() == 0
        ref = O.decode_step(qs_h[step].view(1, n, 1, d), kc_h.view(1, n, cap, d), vc_h.view(1, n, cap, d),
                            com_ref.view(1, n, cap), ln)
        assert (out_b.float().cpu() - ref.view(n, d)).abs().max().item() <= max(tol, 1e-4)
        assert (com_b.cpu() - com_ref).abs().max().item() <= 1e-5 * max(1.0, com_ref.abs().max().item())


def test_static_scratch_decode_refuses_sizes_beyond_its_array():
    lib = load_package()._lib.load()
    one = 256  # never dereferenced: the size check comes first
    rc = lib.dilution_decode_static(one, one, one, 1, 129, 64, 64, 64, 0.125, 1e-9, one, one, None)
    assert rc == 1 and b"exceeds the built-in scratch" in lib.dilution_last_error()
    rc = lib.dilution_decode_static(one, one, one, 1, 64, 1 << 17, 1 << 17, 64, 0.125, 1e-9, one, one, None)
    assert rc == 1 and b"exceeds the built-in scratch" in lib.dilution_last_error()
