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
