"""world_size-2 and -4 gloo tests of the cross-rank demand exchange (CPU)."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, seq, q):
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        P = importlib.import_module("dilution-attention_b200").partition
        from oracle import dilution_oracle as O
        g = torch.Generator().manual_seed(11)
        rows, d = 3, 16
        qq, kk, vv = (torch.randn(rows, seq, d, generator=g) for _ in range(3))
        bounds = P.equal_area_bounds(seq, world, tile=8)
        a, b = bounds[rank], bounds[rank + 1]
        # the K/V all-gather reassembles exactly the visible prefix
        k_seen, v_seen = P.gather_keys(kk[:, a:b].contiguous(), vv[:, a:b].contiguous(), bounds)
        assert torch.equal(k_seen, kk[:, :b]) and torch.equal(v_seen, vv[:, :b])
        # local column sums of p over this rank's rows (oracle maths), then the exscan
        p = O.bids(qq[:, a:b], kk[:, :b], q_offset=a)
        base, demand = P.exclusive_demand_prefix(p.sum(-2), seq)
        full = O.bids(qq, kk)
        assert torch.allclose(base, full[:, :a, :b].sum(-2), atol=1e-5)
        assert torch.allclose(demand, full.sum(-2), atol=1e-5)
        # chunk output with that base == rows [a, b) of the whole-sequence operator
        committed = base[:, None, :] + p.cumsum(-2) - p
        share = p / (committed + p + O.EPS)
        out = (share / (share.sum(-1, keepdim=True) + O.EPS)) @ vv[:, :b]
        ref = O.dilution_dense(qq, kk, vv)[:, a:b]
        assert torch.allclose(out, ref, atol=2e-5)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,seq", [(2, 96), (4, 96), (4, 16)])
def test_sequence_parallel_exchange_matches_whole_sequence(world, seq):
    """seq=16 on four ranks leaves two ranks with an empty query chunk: they must still take
    part in both exchanges instead of leaving the others waiting."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, seq, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results
