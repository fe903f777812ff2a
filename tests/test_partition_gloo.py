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


REF = os.path.join(ROOT, "baseline", "_ref")


def _lm_worker(rank, world, port, variant, q):
    """The reference's DilutionLM on CPU (its eager paths), whole and with its heads split over
    the ranks by partition.shard_lm_heads: same logits, loss, decode steps and gradients."""
    import copy
    import importlib
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, REF)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        P = importlib.import_module("dilution-attention_b200").partition
        from dilution.config import ModelConfig
        from dilution.model import DilutionLM
        kw = dict(vocab_size=96, n_layers=4, d_model=64, n_heads=4, context_length=48,
                  layer_attention=["softmax", "dilution"] * 2)
        if variant == "swiglu_rope":
            kw.update(positional="rope_alt", mlp="swiglu", ffn_hidden=96)
        else:
            kw.update(positional="learned", mlp="gelu", bias=True)
        torch.manual_seed(5)                       # every rank builds the same weights
        whole = DilutionLM(ModelConfig(**kw))
        if variant != "swiglu_rope":               # biases start at zero: make them count
            with torch.no_grad():
                for p in whole.parameters():
                    if p.ndim == 1:
                        p.add_(0.1 * torch.randn(p.shape, generator=torch.Generator().manual_seed(p.numel())))
        split = P.shard_lm_heads(copy.deepcopy(whole))
        assert split.transformer.h[0].attn.n_heads == 4 // world
        try:                                       # dropout masks would differ between the ranks
            P.shard_lm_heads(DilutionLM(ModelConfig(**dict(kw, dropout=0.1))))
            raise AssertionError("a model with dropout was split")
        except ValueError:
            pass
        idx = torch.randint(0, 96, (2, 41), generator=torch.Generator().manual_seed(6))
        # training step: logits, loss, gradients
        lw, loss_w = whole(idx[:, :-1], idx[:, 1:])
        ls, loss_s = split(idx[:, :-1], idx[:, 1:])
        assert torch.allclose(ls, lw, atol=2e-5), (ls - lw).abs().max()
        assert abs(loss_s.item() - loss_w.item()) < 1e-5
        loss_w.backward()
        loss_s.backward()
        gw = dict(whole.named_parameters())
        lo, hi = rank * (64 // world), (rank + 1) * (64 // world)
        for name, p in split.named_parameters():
            g = p.grad
            assert g is not None, name
            if name in gw and gw[name].shape == p.shape:   # replicated: embedding, LayerNorms, biases
                assert torch.allclose(g, gw[name].grad, atol=2e-5), name
        a0 = split.transformer.h[1].attn
        w0 = whole.transformer.h[1].attn
        rows = torch.cat([torch.arange(lo, hi) + part * 64 for part in range(3)])
        assert torch.allclose(a0.c_attn.inner.weight.grad, w0.c_attn.weight.grad[rows], atol=2e-5)
        assert torch.allclose(a0.c_proj.weight.grad, w0.c_proj.weight.grad[:, lo:hi], atol=2e-5)
        if w0.c_proj.bias is not None:
            assert torch.allclose(a0.c_proj.bias.grad, w0.c_proj.bias.grad, atol=2e-5)
        # the gradient norm of the whole model, from the split one
        want = torch.nn.utils.clip_grad_norm_(whole.parameters(), 0.05)
        got = P.clip_grad_norm_(split, 0.05)
        assert abs(got.item() - want.item()) < 1e-5 * max(1.0, want.item())
        assert torch.allclose(a0.c_proj.weight.grad, w0.c_proj.weight.grad[:, lo:hi], atol=2e-6)
        # cached decode: prefill + steps (model.py:451-470)
        whole.eval(), split.eval()
        with torch.no_grad():
            pw, cw = whole.prefill(idx[:, :30], capacity=40)
            ps, cs = split.prefill(idx[:, :30], capacity=40)
            assert torch.allclose(ps, pw, atol=2e-5)
            assert cs[1]["k"].shape[1] == 4 // world and cs[1]["committed"].shape[1] == 4 // world
            for t in range(30, 36):
                sw = whole.decode_step(idx[:, t:t + 1], t, cw)
                ss = split.decode_step(idx[:, t:t + 1], t, cs)
                assert torch.allclose(ss, sw, atol=2e-5), t
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()[-600:] or repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,variant", [(2, "swiglu_rope"), (4, "swiglu_rope"), (2, "gelu_bias_learned")])
def test_lm_with_heads_split_over_ranks_equals_the_whole_model(world, variant):
    if not os.path.isdir(os.path.join(REF, "dilution")):
        pytest.skip("no installed copy of the reference under baseline/_ref")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_lm_worker, args=(r, world, port, variant, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results
