"""Cached decode parity.  Mirrors tests/test_kernels.py:205-241 of the reference."""

from __future__ import annotations

import pytest
import torch

from conftest import golden, make_inputs, rel_err
from oracle import dilution_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_matches_reference_rows(kernels, dtype):
    g = golden("decode_b2h4d32.npz")
    q, k, v, rows = (torch.from_numpy(g[n]) for n in ("q", "k", "v", "rows"))
    prefix, total = int(g["prefix"]), q.shape[2]
    prec = "bf16" if dtype == torch.bfloat16 else "ieee"
    _, aux = kernels.dilution_attention_forward(
        q[:, :, :prefix].to(DEV, dtype), k[:, :, :prefix].to(DEV, dtype), v[:, :, :prefix].to(DEV, dtype),
        dot_precision=prec, return_aux=True)
    capacity = total + 3          # spare rows: the kernel must never touch them
    kc = torch.zeros(2, 4, capacity, 32, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    kc[:, :, :prefix] = k[:, :, :prefix].to(DEV, dtype)
    vc[:, :, :prefix] = v[:, :, :prefix].to(DEV, dtype)
    committed = torch.zeros(2, 4, capacity, device=DEV)
    committed[:, :, :prefix] = aux["committed_total"]
    tol = 1e-3 if dtype == torch.float32 else 5e-2
    for t in range(prefix, total):
        kc[:, :, t] = k[:, :, t].to(DEV, dtype)
        vc[:, :, t] = v[:, :, t].to(DEV, dtype)
        out = kernels.dilution_decode_step(q[:, :, t:t + 1].to(DEV, dtype), kc, vc, committed, t + 1)
        assert out.dtype == dtype and out.shape == (2, 4, 1, 32)
        assert torch.isfinite(out).all()
        err = (out[:, :, 0].float().cpu() - rows[:, :, t]).abs().max().item()
        assert err < tol, f"t={t} max abs err {err}"
    assert committed[:, :, total - 1].abs().max().item() > 0
    assert committed[:, :, total:].abs().max().item() == 0
    if dtype == torch.float32:
        assert rel_err(committed[:, :, :total].cpu(), torch.from_numpy(g["demand_final"])) < 1e-4


@pytest.mark.parametrize("dtype,d,length", [(torch.bfloat16, 64, 5000), (torch.float32, 128, 700),
                                            (torch.bfloat16, 16, 1), (torch.float32, 16, 33),
                                            (torch.bfloat16, 128, 4097)])
def test_decode_long_rows_many_chunks(kernels, dtype, d, length):
    """Lengths that span several key chunks, every head_dim/dtype layout, random demand."""
    b, h, cap = 2, 3, length + 5
    g = torch.Generator().manual_seed(length)
    kc = torch.randn(b, h, cap, d, generator=g).to(dtype)
    vc = torch.randn(b, h, cap, d, generator=g).to(dtype)
    q1 = torch.randn(b, h, 1, d, generator=g).to(dtype)
    committed = torch.rand(b, h, cap, generator=g)
    committed[:, :, length - 1:] = 0
    ref_c = committed.clone()
    ref = O.decode_step(q1, kc, vc, ref_c, length)
    dc = committed.to(DEV)
    dk, dv = kc.to(DEV), vc.to(DEV)
    scratch = kernels.decode_scratch(b * h, cap, d, DEV)
    out = kernels.dilution_decode_step(q1.to(DEV), dk, dv, dc, length, scratch=scratch)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert (out.float().cpu() - ref).abs().max().item() < tol
    assert rel_err(dc.cpu(), ref_c) < 1e-5
    assert torch.equal(dc[:, :, length:].cpu(), committed[:, :, length:])
    assert torch.equal(dk.cpu(), kc) and torch.equal(dv.cpu(), vc)


def test_decode_sequence_of_steps_bf16_d64(kernels):
    """Prefill with the bf16 tensor path, then 16 steps, against the dense oracle rows."""
    b, h, d, prefix, steps = 1, 4, 64, 300, 16
    total = prefix + steps
    q, k, v, _ = make_inputs(b, h, total, d, 31)
    qb, kb, vb = (x.bfloat16() for x in (q, k, v))
    rows = O.dilution_dense(qb.float(), kb.float(), vb.float())
    _, aux = kernels.dilution_attention_forward(qb[:, :, :prefix].to(DEV), kb[:, :, :prefix].to(DEV),
                                                vb[:, :, :prefix].to(DEV), dot_precision="bf16", return_aux=True)
    kc = torch.zeros(b, h, total, d, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kc[:, :, :prefix], vc[:, :, :prefix] = kb[:, :, :prefix].to(DEV), vb[:, :, :prefix].to(DEV)
    committed = torch.zeros(b, h, total, device=DEV)
    committed[:, :, :prefix] = aux["committed_total"]
    for t in range(prefix, total):
        kc[:, :, t], vc[:, :, t] = kb[:, :, t].to(DEV), vb[:, :, t].to(DEV)
        out = kernels.dilution_decode_step(qb[:, :, t:t + 1].to(DEV), kc, vc, committed, t + 1)
        assert (out[:, :, 0].float().cpu() - rows[:, :, t]).abs().max().item() < 2e-2
    assert rel_err(committed.cpu(), O.demand_totals(qb.float(), kb.float())) < 2e-2


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 64), (torch.float32, 32)])
def test_fused_append_equals_append_then_step(kernels, dtype, d):
    """dilution_decode_append_step == the model's _append_kv (model.py:85-93) followed by
    dilution_decode_step, over a run of tokens that crosses a key-chunk boundary; caches,
    demand and outputs must agree, and the dict's len must advance."""
    b, h, prefix, steps = 2, 3, 250, 12
    cap = prefix + steps + 2
    g = torch.Generator().manual_seed(17)
    k = torch.randn(b, h, cap, d, generator=g).to(dtype)
    v = torch.randn(b, h, cap, d, generator=g).to(dtype)
    k[:, :, prefix:], v[:, :, prefix:] = 0, 0
    com = torch.zeros(b, h, cap)
    com[:, :, :prefix] = torch.rand(b, h, prefix, generator=g)
    a = {"k": k.to(DEV), "v": v.to(DEV), "len": prefix, "committed": com.to(DEV)}
    f = {"k": k.to(DEV), "v": v.to(DEV), "len": prefix, "committed": com.to(DEV)}
    # the fused path must not depend on what the demand buffer holds at the new position
    f["committed"][:, :, prefix:] = 7.0
    ck, cv, cc = k.clone(), v.clone(), com.clone()
    for s in range(steps):
        q1, k1, v1 = (torch.randn(b, h, 1, d, generator=g).to(dtype) for _ in range(3))
        t = a["len"]
        a["k"][:, :, t], a["v"][:, :, t] = k1[:, :, 0].to(DEV), v1[:, :, 0].to(DEV)
        a["len"] = t + 1
        ya = kernels.dilution_decode_step(q1.to(DEV), a["k"], a["v"], a["committed"], t + 1)
        yf = kernels.dilution_decode_append_step(q1.to(DEV), k1.to(DEV), v1.to(DEV), f)
        assert f["len"] == t + 1
        # the appended key joins the chunk's sums last instead of in key order
        assert (ya.float() - yf.float()).abs().max().item() <= (1e-5 if dtype == torch.float32 else 2e-2), s
        ck[:, :, t], cv[:, :, t] = k1[:, :, 0], v1[:, :, 0]
        ref = O.decode_step(q1, ck, cv, cc, t + 1)
        assert (yf.float().cpu() - ref).abs().max().item() < (1e-4 if dtype == torch.float32 else 2e-2)
    n = prefix + steps
    assert torch.equal(a["k"], f["k"]) and torch.equal(a["v"], f["v"])
    assert rel_err(a["committed"][:, :, :n], f["committed"][:, :, :n]) < 1e-5
    assert (f["committed"][:, :, n:] == 7.0).all()          # rows past the length stay untouched
    assert rel_err(f["committed"][:, :, :n].cpu(), cc[:, :, :n]) < 1e-5


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("position", [0, 31, 32, 2047, 2048, 4095, 4998])
def test_step_with_the_length_on_the_device(kernels, dtype, tol, position):
    """cache["pos_dev"]: the launches read the new token's position from device memory and run with
    the geometry of the full cache (dilution_decode_append_at) — against the oracle's step, with
    the spare rows of the caches and of the demand untouched, at positions around chunk edges."""
    b, h, d, cap = 1, 3, 64, 5000
    g = torch.Generator().manual_seed(700 + position)
    kc = torch.randn(b, h, cap, d, generator=g).mul(0.5).to(dtype)
    vc = torch.randn(b, h, cap, d, generator=g).to(dtype)
    kc[:, :, position + 1:], vc[:, :, position + 1:] = 0, 0
    q1 = torch.randn(b, h, 1, d, generator=g).mul(0.5).to(dtype)
    committed = torch.rand(b, h, cap, generator=g)
    committed[:, :, position:] = 0
    want_c = committed.clone()
    want = O.decode_step(q1, kc, vc, want_c, position + 1)
    k1, v1 = kc[:, :, position:position + 1].clone(), vc[:, :, position:position + 1].clone()
    kd, vd = kc.clone(), vc.clone()
    kd[:, :, position], vd[:, :, position] = 3.0, 3.0            # stale rows the step must overwrite
    cache = {"k": kd.to(DEV), "v": vd.to(DEV), "len": position, "committed": committed.clone().to(DEV),
             "pos_dev": torch.tensor([position], device=DEV, dtype=torch.int32)}
    cache["committed"][:, :, position] = 9.0                     # stale demand the step must ignore
    got = kernels.dilution_decode_append_step(q1.to(DEV), k1.to(DEV), v1.to(DEV), cache)
    assert got.dtype == dtype and cache["len"] == position + 1
    assert rel_err(got.float().cpu(), want) < tol
    assert rel_err(cache["committed"].cpu(), want_c) < 1e-5
    assert torch.equal(cache["k"].cpu()[:, :, position], k1[:, :, 0]) and torch.equal(cache["v"].cpu()[:, :, position], v1[:, :, 0])
    assert cache["k"][:, :, position + 1:].abs().max().item() == 0 and cache["committed"][:, :, position + 1:].abs().max().item() == 0


def test_position_past_the_capacity_stays_inside_the_cache(kernels, pkg):
    """The C-ABI step with the position on the device holds a position outside [0, capacity) at the
    nearest row: the result is the caller's problem, the memory around the caches is not touched
    (dilution_decode_append_at, dilution_softmax_decode_append_at)."""
    from importlib import import_module
    _lib = import_module(pkg.__name__ + "._lib")
    lib = _lib.load()
    n, d, cap, pad = 3, 64, 300, 64
    g = torch.Generator().manual_seed(77)

    def guarded(rows, width, dtype):            # a cache with sentinel rows on both sides
        buf = torch.full((pad + rows + pad, width), 7.0, dtype=dtype, device=DEV)
        buf[pad:pad + rows] = torch.randn(rows, width, generator=g).to(dtype).to(DEV)
        return buf, buf[pad:pad + rows]

    kbuf, kc = guarded(n * cap, d, torch.bfloat16)
    vbuf, vc = guarded(n * cap, d, torch.bfloat16)
    cbuf, committed = guarded(n * cap, 1, torch.float32)
    committed.copy_(torch.rand(n * cap, 1, generator=g).to(DEV))
    q1, k1, v1 = (torch.randn(n, d, generator=g).to(torch.bfloat16).to(DEV) for _ in range(3))
    out = torch.empty(n, d, device=DEV, dtype=torch.bfloat16)
    scratch = kernels.decode_scratch(n, cap, d, DEV)
    stream = torch.cuda.current_stream().cuda_stream
    for position in (cap, cap + 5, 1 << 20, -3):
        pos = torch.tensor([position], device=DEV, dtype=torch.int32)
        rc = lib.dilution_decode_append_at(q1.data_ptr(), k1.data_ptr(), v1.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                           _lib.BF16, n, cap, pos.data_ptr(), d, d ** -0.5, 1e-9, committed.data_ptr(),
                                           out.data_ptr(), scratch.data_ptr(), stream)
        assert rc == 0
        rc = lib.dilution_softmax_decode_append_at(q1.data_ptr(), k1.data_ptr(), v1.data_ptr(), kc.data_ptr(),
                                                   vc.data_ptr(), _lib.BF16, n, cap, pos.data_ptr(), d, d ** -0.5,
                                                   out.data_ptr(), scratch.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        for buf, rows in ((kbuf, n * cap), (vbuf, n * cap), (cbuf, n * cap)):
            assert (buf[:pad] == 7.0).all() and (buf[pad + rows:] == 7.0).all()
        # the row the step wrote is the nearest one inside the cache
        row = cap - 1 if position >= cap else 0
        got_k = kc.view(n, cap, d)[:, row]
        assert torch.equal(got_k, k1)
