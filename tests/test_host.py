"""Host-side logic that needs no GPU: precision resolution, argument errors,
partition arithmetic, the plug-in switch."""

from __future__ import annotations

import types

import pytest
import torch

from conftest import load_package


def test_resolve_precision_matches_reference_contract():
    K = load_package().kernels
    assert K._resolve_precision("bf16") == (1, "tf32")
    assert K._resolve_precision("ieee") == (0, "ieee")
    assert K._resolve_precision("tf32") == (0, "tf32")
    with pytest.raises(ValueError, match="dot_precision must be one of ieee, tf32, bf16"):
        K._resolve_precision("fp8")


def test_cpu_tensors_raise_instead_of_falling_back():
    K = load_package().kernels
    q = torch.randn(1, 1, 8, 64)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        K.dilution_attention_forward(q, q, q)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        K.dilution_attention(q, q, q, dot_precision="ieee")
    with pytest.raises(ValueError):
        K.dilution_attention(q, q, q, dot_precision="nope")


def test_decode_argument_errors_match_reference():
    K = load_package().kernels
    q2 = torch.randn(1, 1, 2, 32)
    cache = torch.zeros(1, 1, 8, 32)
    com = torch.zeros(1, 1, 8)
    with pytest.raises(ValueError, match="exactly one query row"):
        K.dilution_decode_step(q2, cache, cache, com, 1)
    with pytest.raises(ValueError, match="power of two"):
        K.dilution_decode_step(torch.randn(1, 1, 1, 24), torch.zeros(1, 1, 8, 24), torch.zeros(1, 1, 8, 24), com, 1)
    with pytest.raises(ValueError, match="outside cache capacity"):
        K.dilution_decode_step(torch.randn(1, 1, 1, 32), cache, cache, com, 9)
    with pytest.raises(ValueError, match="outside cache capacity"):
        K.dilution_decode_step(torch.randn(1, 1, 1, 32), cache, cache, com, 0)


def test_install_swaps_entry_points_on_a_module():
    pkg = load_package()
    fake = types.SimpleNamespace(HAS_TRITON=False)
    pkg.install(fake)
    assert fake.dilution_attention is pkg.kernels.dilution_attention
    assert fake.dilution_decode_step is pkg.kernels.dilution_decode_step
    assert fake.HAS_TRITON is True
    pkg.uninstall(fake)
    assert fake.HAS_TRITON is False


def test_fused_append_refuses_a_full_cache_like_append_kv():
    """model.py:88-89: a step past the capacity is a ValueError before anything runs."""
    K = load_package().kernels
    cache = {"k": torch.zeros(1, 1, 4, 32), "v": torch.zeros(1, 1, 4, 32), "len": 4,
             "committed": torch.zeros(1, 1, 4)}
    x = torch.randn(1, 1, 1, 32)
    with pytest.raises(ValueError, match="past the cache capacity"):
        K.dilution_decode_append_step(x, x, x, cache)
    assert cache["len"] == 4


def test_row_shard_covers_rows_exactly():
    P = load_package().partition
    for n, w in [(64, 8), (64, 3), (5, 8), (1024, 4)]:
        spans = [P.row_shard(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1


def test_equal_area_bounds_balance_and_agree_with_oracle():
    P = load_package().partition
    from oracle import dilution_oracle as O
    for seq, w in [(131072, 8), (131072, 4), (131072, 2), (4096, 8)]:
        b = P.equal_area_bounds(seq, w)
        assert b == O.equal_area_bounds(seq, w)
        assert b[0] == 0 and b[-1] == seq and all(x % 128 == 0 for x in b)
    b = P.equal_area_bounds(131072, 8)
    areas = [b[i + 1] ** 2 - b[i] ** 2 for i in range(8)]
    assert max(areas) / (sum(areas) / 8) < 1.03   # speed-up ceiling > 7.7x, not 4.27x


def test_variant_codes_and_errors_follow_the_reference_module():
    """kernels_bid.py:84-91, 123-127 of the reference: bid names, share codes, ValueError."""
    KB = load_package().kernels_bid
    assert KB.BID_TYPES == ("softmax", "relu", "relu2", "softplus", "minshift", "sigmoid", "expshift", "sigshift")
    assert [KB._bid_code(b) for b in KB.BUILT_BIDS] == [KB.BID_TYPES.index(b) for b in KB.BUILT_BIDS]
    assert KB._share_code(True) == 1 and KB._share_code(False) == 0 and KB._share_code("exclusive") == 2
    with pytest.raises(ValueError, match="bid must be one of"):
        KB._bid_code("tanh")
    assert KB.BUILT_BIDS == KB.BID_TYPES                                 # every bid of the reference is built
    q = torch.randn(1, 1, 8, 64)
    with pytest.raises(RuntimeError, match="no CPU fallback"):          # the variants have none either
        KB.dilution_attention_forward(q, q, q, bid="sigmoid")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        KB.dilution_attention(q, q, q, dot_precision="ieee", bid="softmax", share_cumsum="exclusive")
    with pytest.raises(ValueError, match="exactly one query row"):
        KB.dilution_decode_step(torch.randn(1, 1, 2, 32), torch.zeros(1, 1, 8, 32), torch.zeros(1, 1, 8, 32),
                                torch.zeros(1, 1, 8), 1, bid="sigmoid")


def test_variant_install_routes_every_bid_here_and_uninstall_puts_the_module_back():
    """After install() every bid of the reference reaches this backend (none is left to the
    module's original functions); uninstall() puts everything back."""
    KB = load_package().kernels_bid
    calls = []

    def original(*args, bid="softmax", **kwargs):
        calls.append(bid)
        return "original"

    fake = types.SimpleNamespace(HAS_TRITON=False, dilution_attention_forward=original,
                                 dilution_attention=original, dilution_decode_step=original)
    KB.install(fake)
    assert fake.HAS_TRITON is True
    q = torch.randn(1, 1, 8, 64)
    for bid in ("relu2", "sigshift", "minshift"):
        with pytest.raises(RuntimeError, match="no CPU fallback"):      # this backend, which needs CUDA
            fake.dilution_attention_forward(q, q, q, bid=bid, shift=8.0)
    with pytest.raises(ValueError, match="bid must be one of"):
        fake.dilution_attention(q, q, q, bid="tanh")
    assert calls == []
    KB.uninstall(fake)
    assert fake.dilution_attention is original and fake.HAS_TRITON is False
