"""Sequence-parallel prefill across GPUs (NCCL), one process per GPU.

Needs at least two CUDA devices; skipped otherwise.  Every rank owns a contiguous
query chunk, all-gathers K/V, runs passes 1-2, takes part in the cross-rank
exclusive scan of per-key demand and finishes with pass 3.  The result must equal
the single-sequence operator.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, seq, prec, q):
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        pkg = importlib.import_module("dilution-attention_b200")
        from oracle import dilution_oracle as O
        P = pkg.partition
        g = torch.Generator().manual_seed(5)
        rows, d = 4, 64
        dt = torch.bfloat16 if prec == "bf16" else torch.float32
        qq, kk, vv = (torch.randn(rows, seq, d, generator=g).mul_(0.7).to(dt) for _ in range(3))
        bounds = P.equal_area_bounds(seq, world)
        a, b = bounds[rank], bounds[rank + 1]
        dev = torch.device("cuda", rank)
        out, demand = P.sequence_parallel_prefill(qq[:, a:b].to(dev), kk[:, a:b].to(dev), vv[:, a:b].to(dev),
                                                  seq, bounds, dot_precision=prec)
        torch.cuda.synchronize()
        ref, dref = O.dilution_chunked(qq.float(), kk.float(), vv.float(), chunk=512, return_demand=True)
        tol = 2e-2 if prec == "bf16" else 1e-4
        err = (out.cpu() - ref[:, a:b]).abs().max().item()
        derr = (demand.cpu() - dref).abs().max().item() / dref.abs().max().item()
        status = pkg._lib.load().dilution_device_status()
        assert err < tol and derr < tol and status == 0, (err, derr, status)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("prec", ["bf16", "ieee"])
def test_sequence_parallel_prefill_matches_single_sequence(prec):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    seq = 2048 if prec == "bf16" else 1024
    procs = [ctx.Process(target=_worker, args=(r, world, port, seq, prec, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results


REF = os.path.join(ROOT, "baseline", "_ref")


def _lm_worker(rank, world, port, q):
    """The reference's DilutionLM with its heads over the ranks and every kernel of this library
    installed, against the whole model on the same GPU: logits, loss, a decode run."""
    import copy
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, REF)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = importlib.import_module("dilution-attention_b200")
        from dilution.config import ModelConfig
        from dilution.model import DilutionLM
        pkg.install(fused_decode=True)
        pkg.install_layers()
        cfg = ModelConfig(vocab_size=512, n_layers=4, d_model=256, n_heads=4, context_length=400,
                          layer_attention=["softmax", "dilution"] * 2, positional="rope_alt",
                          mlp="swiglu", ffn_hidden=512)
        torch.manual_seed(9)
        whole = DilutionLM(cfg).to(dev)
        split = pkg.partition.shard_lm_heads(copy.deepcopy(whole))
        whole.enable_dilution_kernel(), split.enable_dilution_kernel()
        idx = torch.randint(0, 512, (2, 321), generator=torch.Generator().manual_seed(3)).to(dev)
        before = pkg._lib.launch_count()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            lw, loss_w = whole(idx[:, :-1], idx[:, 1:])
            ls, loss_s = split(idx[:, :-1], idx[:, 1:])
        assert pkg._lib.launch_count() > before
        assert (ls.float() - lw.float()).abs().max().item() < 5e-2
        assert abs(loss_s.item() - loss_w.item()) < 2e-2
        loss_s.backward()
        norm = pkg.partition.clip_grad_norm_(split, 1.0)
        assert torch.isfinite(norm)
        whole.eval(), split.eval()
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            pw, cw = whole.prefill(idx[:, :300], capacity=320)
            ps, cs = split.prefill(idx[:, :300], capacity=320)
            assert (ps.float() - pw.float()).abs().max().item() < 5e-2
            assert cs[1]["k"].shape[1] == 4 // world
            for t in range(300, 308):
                sw = whole.decode_step(idx[:, t:t + 1], t, cw)
                ss = split.decode_step(idx[:, t:t + 1], t, cs)
                assert (ss.float() - sw.float()).abs().max().item() < 5e-2, t
        torch.cuda.synchronize()
        assert pkg._lib.load().dilution_device_status() == 0
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()[-800:]))
    finally:
        try:
            pkg.uninstall_layers()
            pkg.uninstall()
        except Exception:  # noqa: BLE001
            pass
        dist.destroy_process_group()


def test_lm_with_heads_over_gpus_matches_the_whole_model():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    if not os.path.isdir(os.path.join(REF, "dilution")):
        pytest.skip("no installed copy of the reference under baseline/_ref")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_lm_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results
