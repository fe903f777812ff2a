"""The reference model's attention layers on this library, beyond the dilution operator.

The reference's alternating stacks (config `layer_attention`, `positional="rope_alt"`) interleave
dilution layers with softmax layers that call `F.scaled_dot_product_attention`
(model.py:96-117) and rotate q and k with RoPE in `_split_heads` (model.py:59-67,
rope.py:26-44).  This module puts those pieces on the same kernels:

    split_heads_rope(qkv, n_heads, rope, offset)   the head split of the fused c_attn output with
                                                   the rotation applied on the way, differentiable:
                                                   one pass over qkv instead of split + view +
                                                   transpose + the rotation's elementwise chain +
                                                   three .contiguous() copies
    softmax_attention_forward(q, k, v)             kernels.py of this package (tcgen05 row pass + P V)
    softmax_decode_append_step(q1, k1, v1, cache)  the cached step of a softmax layer with the
                                                   token append fused in (model.py:112-117)
    install_layers() / uninstall_layers()          patch `dilution.model` accordingly

Everything falls back to the model's own code whenever a tensor is not bf16 on a CUDA device,
the head size is not supported, or (for the softmax forward) gradients are required: there is
no backward kernel for the softmax layers, training keeps using SDPA for them.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from . import kernels as K

_ROPE_DIMS = (32, 64, 128)


_TABLE_CACHE: dict = {}


def rope_tables(rope, seq: int, offset: int, device, dtype):
    """cos / sin tables (seq, dim/2) exactly as RopeModule.forward builds them (rope.py:33-39):
    fp32 angles, cast to the activation dtype.  The last table per (dim, theta, device, dtype) is
    kept: every rotated layer of a model asks for the same positions within a forward pass or a
    decode step."""
    key = (rope.dim, float(rope.theta), str(device), dtype)
    hit = _TABLE_CACHE.get(key)
    if hit is not None and hit[0] == (seq, offset):
        return hit[1], hit[2]
    positions = torch.arange(offset, offset + seq, device=device, dtype=torch.float32)
    inv_freq = 1.0 / (rope.theta ** (torch.arange(0, rope.dim, 2, device=device, dtype=torch.float32) / rope.dim))
    freqs = torch.outer(positions, inv_freq)
    cos, sin = freqs.cos().to(dtype).contiguous(), freqs.sin().to(dtype).contiguous()
    _TABLE_CACHE[key] = ((seq, offset), cos, sin)
    return cos, sin


class _SplitHeadsRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, heads, cos, sin):
        lib = _lib.load()
        batch, seq, width = qkv.shape
        d = width // (3 * heads)
        qkv = qkv.contiguous()
        q, k, v = (torch.empty(batch, heads, seq, d, device=qkv.device, dtype=qkv.dtype) for _ in range(3))
        _lib.check(lib.dilution_split_heads_rope(qkv.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                 K._ptr(cos), K._ptr(sin), batch, seq, heads, d, 0,
                                                 K._stream(qkv.device)), "dilution_split_heads_rope")
        ctx.save_for_backward(cos, sin) if cos is not None else None
        ctx.has_rope = cos is not None
        ctx.heads = heads
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        lib = _lib.load()
        cos, sin = ctx.saved_tensors if ctx.has_rope else (None, None)
        batch, heads, seq, d = dq.shape
        dq, dk, dv = (x.contiguous() for x in (dq, dk, dv))
        dqkv = torch.empty(batch, seq, 3 * heads * d, device=dq.device, dtype=dq.dtype)
        _lib.check(lib.dilution_split_heads_rope(dqkv.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                                 K._ptr(cos), K._ptr(sin), batch, seq, heads, d, 1,
                                                 K._stream(dq.device)), "dilution_split_heads_rope")
        return dqkv, None, None, None


def split_heads_rope(qkv: torch.Tensor, n_heads: int, rope=None, offset: int = 0):
    """q, k, v (B, H, T, D) contiguous from the fused projection qkv (B, T, 3*H*D), q and k
    rotated by `rope` (a RopeModule or None) at positions offset.. (model.py:59-67).
    bf16 CUDA tensors with D in {32, 64, 128}; differentiable."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16):
        raise ValueError("split_heads_rope takes bfloat16 CUDA tensors")
    d = qkv.shape[-1] // (3 * n_heads)
    if d not in _ROPE_DIMS:
        raise ValueError(f"head_dim {d} not in {_ROPE_DIMS}")
    cos = sin = None
    if rope is not None:
        cos, sin = rope_tables(rope, qkv.shape[1], offset, qkv.device, qkv.dtype)
    return _SplitHeadsRope.apply(qkv, n_heads, cos, sin)


def split_heads_at(layer, x1, cache):
    """`_split_heads` of ONE token per batch row whose position is read from the device
    (cache["pos_dev"], a one-element int32 tensor): the launch takes no host-side position, so
    it can be recorded into a CUDA graph.  layer: the attention module; x1: (B, 1, C).
    bf16 projections only."""
    lib = _lib.load()
    qkv = layer.c_attn(x1)
    if qkv.dtype != torch.bfloat16:
        raise ValueError("a step with the position on the device takes bfloat16 activations (autocast)")
    batch, one, width = qkv.shape
    heads = layer.n_heads
    d = width // (3 * heads)
    if one != 1 or d not in _ROPE_DIMS:
        raise ValueError(f"one token per row and head_dim in {_ROPE_DIMS}")
    qkv = qkv.contiguous()
    q, k, v = (torch.empty(batch, heads, 1, d, device=qkv.device, dtype=qkv.dtype) for _ in range(3))
    cos = sin = None
    if layer.rope is not None:
        # tables for every position the cache can hold, kept with the cache: a recorded graph
        # holds their addresses, so they must live as long as the cache does
        tables = cache.get("rope_tables")
        if tables is None:
            tables = cache["rope_tables"] = rope_tables(layer.rope, cache["k"].shape[2], 0, qkv.device, qkv.dtype)
        cos, sin = tables
    _lib.check(lib.dilution_split_heads_rope_at(qkv.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                K._ptr(cos), K._ptr(sin),
                                                0 if cos is None else cos.shape[0], batch, heads, d,
                                                cache["pos_dev"].data_ptr(), K._stream(qkv.device)),
               "dilution_split_heads_rope_at")
    return q, k, v


def softmax_decode_append_step(q1, k1, v1, cache: dict, scratch=None, out=None):
    """One cached token of a softmax layer: `_append_kv(cache, k1, v1)` followed by attention of
    q1 over the first len+1 cache rows (model.py:112-117), as three launches that stream K and V
    once.  q1, k1, v1: (B, H, 1, D); cache: the model's dict {"k", "v", "len"}.  Returns
    (B, H, 1, D) in q1.dtype; cache["len"] grows by one.  With cache["pos_dev"] the length is
    read from the device (see GraphedDecode)."""
    lib = _lib.load()
    t = cache["len"]
    k_cache, v_cache = cache["k"], cache["v"]
    if t >= k_cache.shape[2]:
        raise ValueError("decode step past the cache capacity (context_length)")
    batch, heads, one, d = q1.shape
    if one != 1:
        raise ValueError("decode step takes exactly one query row per (batch, head)")
    if q1.dtype not in (torch.float32, torch.bfloat16) or k_cache.dtype != q1.dtype or v_cache.dtype != q1.dtype:
        raise ValueError("caches must have q1's dtype (float32 or bfloat16)")
    n, capacity = batch * heads, k_cache.shape[2]
    qf, kn, vn = (K._rows(x, n, d) for x in (q1, k1, v1))
    if out is None:
        out = torch.empty(n, d, device=q1.device, dtype=q1.dtype)
    pos_dev = cache.get("pos_dev")
    need = lib.dilution_decode_scratch_bytes(n, capacity if pos_dev is not None else t + 1, d)
    if scratch is None or scratch.numel() * scratch.element_size() < need:
        scratch = torch.empty(need, device=q1.device, dtype=torch.uint8)
    code = _lib.BF16 if q1.dtype == torch.bfloat16 else _lib.F32
    if pos_dev is not None:
        _lib.check(lib.dilution_softmax_decode_append_at(
            qf.data_ptr(), kn.data_ptr(), vn.data_ptr(), k_cache.view(n, capacity, d).data_ptr(),
            v_cache.view(n, capacity, d).data_ptr(), code, n, capacity, pos_dev.data_ptr(), d, 1.0 / math.sqrt(d),
            out.data_ptr(), scratch.data_ptr(), K._stream(q1.device)), "dilution_softmax_decode_append_at")
    else:
        _lib.check(lib.dilution_softmax_decode_append(
            qf.data_ptr(), kn.data_ptr(), vn.data_ptr(), k_cache.view(n, capacity, d).data_ptr(),
            v_cache.view(n, capacity, d).data_ptr(), code, n, capacity, t + 1, d, 1.0 / math.sqrt(d),
            out.data_ptr(), scratch.data_ptr(), K._stream(q1.device)), "dilution_softmax_decode_append")
    cache["len"] = t + 1
    return out.view(batch, heads, 1, d)


class GraphedDecode:
    """The model's per-token layer loop (`DilutionLM.decode_step`, model.py:464-470) recorded ONCE
    into a CUDA graph and replayed per token.

    A step's launches normally take the cache length and the token's position as host scalars,
    which a graph would freeze.  Here every cache of the model shares one int32 device scalar
    (`cache["pos_dev"]`, the new token's position); the decode and head-split launches read it
    (`dilution_decode_append_at`, `dilution_softmax_decode_append_at`,
    `dilution_split_heads_rope_at`), and the recorded step ends by adding one to it.

    Needs `install(fused_decode=True)` and `install_layers()` (every attention layer's cached
    step on this library's kernels), bf16 autocast, and a model whose embedding does not use the
    position (positional "none", "rope" or "rope_alt": `_embed`, model.py:386-393).  Usage:

        logits, caches = model.prefill(prompt, capacity=...)
        dec = GraphedDecode(model, caches)
        logits = dec.step(token)          # (B, 1) int64 -> (B, 1, vocab); the first call records

    The caches stay the model's own dicts; their "len" entries are kept in step with the device
    scalar, so `model.decode_step` can take over again after `dec.close()`.
    """

    def __init__(self, model, caches, autocast_dtype=torch.bfloat16):
        if model.config.positional == "learned":
            raise ValueError("GraphedDecode needs a model whose embedding ignores the position")
        self.model, self.caches, self.dtype = model, caches, autocast_dtype
        dev = caches[0]["k"].device
        self.capacity = min(c["k"].shape[2] for c in caches)
        self.position = caches[0]["len"]
        if any(c["len"] != self.position for c in caches):
            raise ValueError("all layers' caches must hold the same number of tokens")
        self.pos_dev = torch.tensor([self.position], device=dev, dtype=torch.int32)
        for c in caches:
            c["pos_dev"] = self.pos_dev
        self.graph = None
        self.token = None
        self.logits = None

    def _one_step(self):
        with torch.no_grad(), torch.autocast("cuda", dtype=self.dtype):
            logits = self.model.decode_step(self.token, 0, self.caches)
        self.pos_dev.add_(1)
        return logits

    def step(self, token):
        """One token for every sequence: (B, 1) int64 ids -> (B, 1, vocab) logits (a view of a
        buffer that the next call overwrites)."""
        if self.position >= self.capacity:
            raise ValueError("decode step past the cache capacity (context_length)")
        if self.graph is None:
            # the first step runs eagerly (it also warms up every library this step touches), the
            # second is recorded; recording executes nothing, so it is replayed right away
            if self.token is None:
                self.token = token.clone()
                logits = self._one_step()
                self.position += 1
                return logits
            self.token.copy_(token)
            for c in self.caches:                 # the recorded step must not move the host-side lengths
                c["len"] = self.position
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.logits = self._one_step()
        else:
            self.token.copy_(token)
        self.graph.replay()
        self.position += 1
        for c in self.caches:
            c["len"] = self.position
        return self.logits

    def close(self):
        """Detach the device-side position: the caches are the model's plain dicts again."""
        for c in self.caches:
            c.pop("pos_dev", None)
            c.pop("rope_tables", None)
            c["len"] = self.position
        self.graph = None


# ---- patches of dilution.model -------------------------------------------------------------
def _fast_split_ok(self, x):
    d = self.d_model // self.n_heads
    return x.is_cuda and d in _ROPE_DIMS


def _split_heads(self, x, offset: int = 0):
    """_AttentionBase._split_heads (model.py:59-67) with the split, the transposition and the
    rotation in one kernel when the projection comes out in bf16 on a CUDA device."""
    if _fast_split_ok(self, x):
        qkv = self.c_attn(x)
        if qkv.dtype == torch.bfloat16:
            return split_heads_rope(qkv, self.n_heads, self.rope, offset)
        batch, seq, _ = x.shape
        q, k, v = qkv.split(self.d_model, dim=2)
        shape = (batch, seq, self.n_heads, self.d_model // self.n_heads)
        q, k, v = (q.view(shape).transpose(1, 2), k.view(shape).transpose(1, 2), v.view(shape).transpose(1, 2))
        if self.rope is not None:
            q, k = self.rope(q, offset), self.rope(k, offset)
        return q, k, v
    return self._b200_split_heads(x, offset)


def _softmax_forward(self, x):
    """CausalSelfAttention.forward (model.py:99-105); the tcgen05 kernel when no gradient is
    needed, the model's SDPA call otherwise."""
    if torch.is_grad_enabled() or not x.is_cuda or self.d_model // self.n_heads != 64:
        return self._b200_forward(x)
    batch, seq, _ = x.shape
    q, k, v = self._split_heads(x)
    if q.dtype != torch.bfloat16:
        return self._b200_forward(x)
    y = K.softmax_attention_forward(q, k, v)
    return self._merge_heads(y, batch, seq)


def _softmax_begin_cache(self, x, capacity=None):
    """CausalSelfAttention.begin_cache (model.py:107-110) with one head split instead of two."""
    if torch.is_grad_enabled() or not x.is_cuda or self.d_model // self.n_heads != 64:
        return self._b200_begin_cache(x, capacity)
    batch, seq, _ = x.shape
    q, k, v = self._split_heads(x)
    if q.dtype != torch.bfloat16:
        return self._b200_begin_cache(x, capacity)
    y = K.softmax_attention_forward(q, k, v)
    return self._merge_heads(y, batch, seq), self._alloc_cache(k, v, capacity)


def _softmax_step_cache(self, x1, cache):
    """CausalSelfAttention.step_cache (model.py:112-117) on the streaming decode kernels."""
    if not x1.is_cuda or (self.d_model // self.n_heads) not in (16, 32, 64, 128):
        return self._b200_step_cache(x1, cache)
    batch = x1.shape[0]
    if cache.get("pos_dev") is not None:       # the position lives on the device (a captured step)
        q1, k1, v1 = split_heads_at(self, x1, cache)
        return self._merge_heads(softmax_decode_append_step(q1, k1, v1, cache), batch, 1)
    q1, k1, v1 = self._split_heads(x1, offset=cache["len"])
    if q1.dtype not in (torch.float32, torch.bfloat16) or cache["k"].dtype != q1.dtype:
        t = self._append_kv(cache, k1, v1)
        y = torch.nn.functional.scaled_dot_product_attention(q1, cache["k"][:, :, :t], cache["v"][:, :, :t])
        return self._merge_heads(y, batch, 1)
    y = softmax_decode_append_step(q1, k1, v1, cache)
    return self._merge_heads(y, batch, 1)


_PATCHES = (
    ("_AttentionBase", "_split_heads", _split_heads),
    ("CausalSelfAttention", "forward", _softmax_forward),
    ("CausalSelfAttention", "begin_cache", _softmax_begin_cache),
    ("CausalSelfAttention", "step_cache", _softmax_step_cache),
)


def install_layers(model_module=None):
    """Patch `dilution.model` (or the given module): fused head split + RoPE for every attention
    layer, and the softmax layers' inference forward / prefill / cached step on this library's
    kernels.  The originals stay reachable as `_b200_<name>` and are used whenever a fast path
    does not apply.  Training of the softmax layers is untouched (SDPA)."""
    if model_module is None:
        import dilution.model as model_module
    for cls_name, name, fn in _PATCHES:
        cls = getattr(model_module, cls_name)
        saved = "_b200_" + name.lstrip("_")
        if saved not in cls.__dict__:
            setattr(cls, saved, cls.__dict__[name])
            setattr(cls, name, fn)
    return model_module


def uninstall_layers(model_module=None):
    if model_module is None:
        import sys
        model_module = sys.modules.get("dilution.model")
        if model_module is None:
            return None
    for cls_name, name, _ in _PATCHES:
        cls = getattr(model_module, cls_name)
        saved = "_b200_" + name.lstrip("_")
        if saved in cls.__dict__:
            setattr(cls, name, cls.__dict__[saved])
            delattr(cls, saved)
    return model_module
