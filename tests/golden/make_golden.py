"""Generate the golden fixtures in this folder from the UNMODIFIED reference.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/Dilution-Attention

It imports `dilution.kernels.dilution_attention_reference` (src/dilution/kernels.py:40-68)
from the checkout, feeds it inputs drawn from a CPU `torch.Generator` (so the
same bits can be regenerated anywhere), and stores the reference's outputs and
its autograd gradients.  The fixtures travel with the repository; the reference
does not, so nothing else reads the checkout.

Fixture layout (all fp32 unless noted):
  c1_b1h4t512d64.npz   config-1 golden: out, dq, dk, dv  (+ input fingerprint)
  small_cases.npz      T in {1, 8, 65, 257}: q, k, v, dout, out, dq, dk, dv,
                       demand (= p.sum(-2)) and pk (= p@k/sqrt(D))
  decode_b2h4d32.npz   prefix 37 + 6 steps: q, k, v and the reference rows
  layers_b2t24h2d32.npz  the model's softmax layer pieces: RopeModule outputs at two offsets
                       (bf16 and fp32 inputs) and softmax-attention rows
                       (F.scaled_dot_product_attention, is_causal) for the same q, k, v
  variants_b1h2t80d32.npz  the bid / share ablations of src/dilution/kernels_bid.py:130-166
                       ("softmax" / "sigmoid" / "expshift" / "sigshift" bids x inclusive / "exclusive" /
                       no share step, shift 80):
                       q, k, v, dout and per variant out, dq, dk, dv and demand (= p.sum(-2))

`--only variants` writes just the last one.
"""

from __future__ import annotations

import argparse
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def seeded(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32) * scale


def make_inputs(b, h, t, d, seed):
    """q, k, v, dout ~ N(0,1) from consecutive seeds; identical on every host."""
    return tuple(seeded((b, h, t, d), seed + i) for i in range(4))


def fingerprint(*tensors):
    return np.array([float(x.double().sum()) for x in tensors] +
                    [float(x.flatten()[0]) for x in tensors], dtype=np.float64)


def ref_fwd_bwd(ref, q, k, v, dout):
    qs, ks, vs = (x.clone().requires_grad_(True) for x in (q, k, v))
    out = ref(qs, ks, vs)
    out.backward(dout)
    return out.detach(), qs.grad, ks.grad, vs.grad


VARIANTS = [("softmax", "exclusive"), ("softmax", False), ("sigmoid", True), ("sigmoid", "exclusive"),
            ("sigmoid", False), ("expshift", True), ("sigshift", True), ("sigshift", False),
            ("relu", True), ("relu2", True), ("softplus", True), ("minshift", True), ("relu", False),
            ("softplus", "exclusive")]
SHIFT = 80.0      # the shifted bids' divisor: the model passes its context length (model.py:152-156)


def variant_key(bid, share):
    return f"{bid}_{ {True: 'inclusive', False: 'none'}.get(share, share) }"


def make_variants():
    from dilution.kernels_bid import bids_from_affinity, dilution_attention_reference as ref_bid
    b, h, t, d = 1, 2, 80, 32
    q, k, v, dout = make_inputs(b, h, t, d, 7070)
    data = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), dout=dout.numpy(), shift=np.array(SHIFT))
    aff = (q @ k.transpose(-2, -1)) / math.sqrt(d)
    causal = torch.ones(t, t, dtype=torch.bool).tril()
    for bid, share in VARIANTS:
        out, dq, dk, dv = ref_fwd_bwd(lambda a, b_, c: ref_bid(a, b_, c, bid=bid, share_cumsum=share, shift=SHIFT), q, k, v, dout)
        p = bids_from_affinity(aff, causal, bid, SHIFT)
        for name, x in dict(out=out, dq=dq, dk=dk, dv=dv, demand=p.sum(-2)).items():
            data[f"{variant_key(bid, share)}_{name}"] = x.numpy()
    np.savez(os.path.join(HERE, "variants_b1h2t80d32.npz"), **data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", choices=("all", "variants"), default="all")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from dilution.kernels import dilution_attention_reference as ref

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    make_variants()
    if args.only == "variants":
        print("wrote the variants fixture to", HERE)
        return

    # config 1: B1 H4 T512 d64, fp32 N(0,1), seed 1338 (1337 + config index)
    q, k, v, dout = make_inputs(1, 4, 512, 64, 1338)
    out, dq, dk, dv = ref_fwd_bwd(ref, q, k, v, dout)
    np.savez(os.path.join(HERE, "c1_b1h4t512d64.npz"),
             out=out.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
             fingerprint=fingerprint(q, k, v, dout), seed=np.array(1338))

    # small ragged cases, inputs stored
    small = {}
    for t, (b, h, d) in [(1, (1, 2, 32)), (8, (2, 2, 64)), (65, (1, 2, 32)), (257, (1, 2, 64))]:
        q, k, v, dout = make_inputs(b, h, t, d, 100 + t)
        out, dq, dk, dv = ref_fwd_bwd(ref, q, k, v, dout)
        aff = (q @ k.transpose(-2, -1)) / math.sqrt(d)
        causal = torch.ones(t, t, dtype=torch.bool).tril()
        p = aff.masked_fill(~causal, float("-inf")).softmax(-1)
        for name, x in dict(q=q, k=k, v=v, dout=dout, out=out, dq=dq, dk=dk, dv=dv,
                            demand=p.sum(-2), pk=(p @ k) / math.sqrt(d)).items():
            small[f"t{t}_{name}"] = x.numpy()
    np.savez(os.path.join(HERE, "small_cases.npz"), **small)

    # decode: the reference's own decode test shape (tests/test_kernels.py:211-215)
    b, h, d, prefix, steps = 2, 4, 32, 37, 6
    total = prefix + steps
    q, k, v, _ = make_inputs(b, h, total, d, 4242)
    rows = ref(q, k, v)
    aff = (q @ k.transpose(-2, -1)) / math.sqrt(d)
    causal = torch.ones(total, total, dtype=torch.bool).tril()
    p = aff.masked_fill(~causal, float("-inf")).softmax(-1)
    np.savez(os.path.join(HERE, "decode_b2h4d32.npz"),
             q=q.numpy(), k=k.numpy(), v=v.numpy(), rows=rows.numpy(),
             demand_prefix=p[:, :, :prefix].sum(-2)[..., :prefix].numpy(),
             demand_final=p.sum(-2).numpy(), prefix=np.array(prefix))
    # the softmax layers' pieces (src/dilution/rope.py, model.py:96-117)
    from dilution.rope import RopeModule
    b, h, t, d = 2, 2, 24, 32
    q, k, v, _ = make_inputs(b, h, t, d, 5151)
    rope = RopeModule(d, theta=10000.0)
    qb = q.bfloat16()
    sdpa = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    np.savez(os.path.join(HERE, "layers_b2t24h2d32.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
             rope_f32_off0=rope(q, 0).numpy(), rope_f32_off9=rope(q, 9).numpy(),
             rope_bf16_off0=rope(qb, 0).float().numpy(), rope_bf16_off9=rope(qb, 9).float().numpy(),
             sdpa=sdpa.numpy(), theta=np.array(10000.0))
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
