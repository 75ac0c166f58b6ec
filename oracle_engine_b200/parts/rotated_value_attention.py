"""Mixer `rotated_value_attention`: grouped-query attention over the paged cache whose queries and keys are normed
per head before they are turned, whose values are normed and turned too, and whose softmax has a learned sink.

    q = Wq h + bq [H, dk],  k = Wk h + bk [G, dk],  v = Wv h + bv [G, dv]
    q, k <- q / sqrt(mean(q^2) + eps) * wq,  k / sqrt(mean(k^2) + eps) * wk      per head, weights shared by the heads
    q, k: the first `rot` dimensions turned by the token's position, dimension i < rot/2 paired with i + rot/2 (the
          position encoding's cos/sin table; its frequencies may be rescaled); the other dimensions pass
    v <- v / sqrt(mean(v^2) + eps) per head (no weight), then ALL dv dimensions turned by the position of the key's
          token, m paired with m + dv/2, frequencies base^(-2m/dv) (a table of its own, never rescaled)
    s_j = scale * q . k_j for the keys pos - window < j <= pos (all j <= pos when window is 0)
    p_j = exp(s_j) / (exp(sink_h) + sum_j exp(s_j))          the sink: a learned score per head with no key, no value
    o = sum_j p_j v_j, turned back by the QUERY's position;    x += Wo concat_heads(o)
Query head i reads key/value head i // (H / G).  Turning the values by their own position and the sum back by the
query's makes the output depend on the values through relative positions.  Every one of bias, q/k norm, key
rotation, value norm, value rotation, window and sink is a parameter that can be off.

The cache keeps per token two tensors, as stored after norm and turn: "k" (G, dk) and "v" (G, dv).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import CacheNeed, TensorDecl

_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_bias": "mix.q.b", "k_bias": "mix.k.b",
          "v_bias": "mix.v.b", "q_norm": "mix.q.norm", "k_norm": "mix.k.norm", "sink": "mix.sink"}


@MIXERS.register("rotated_value_attention")
class RotatedValueAttention(Part):
    graph_safe = True
    can_overwrite = True
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale, eps, window (0 or None: all keys),
    position (a `rotary` encoding whose head_dim is the number of turned key dimensions, or None), value_position (a
    `rotary` encoding of head_dim = value_dim, or None: values are not turned), bias, qk_norm, value_norm, sink
    (booleans, default True), tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.G = int(self._need("num_kv_heads"))
        self.dk = int(self._need("key_dim"))
        self.dv = int(self._need("value_dim"))
        self.scale = float(self._need("scale"))
        self.eps = float(self._need("eps"))
        self.window = int(self.params.get("window") or 0)
        self.position = self.params.get("position")
        self.value_position = self.params.get("value_position")
        if isinstance(self.value_position, str):
            self.value_position = self.params["position_table"][self.value_position]
        self.bias = bool(self.params.get("bias", True))
        self.qk_norm = bool(self.params.get("qk_norm", True))
        self.value_norm = bool(self.params.get("value_norm", True))
        self.sink = bool(self.params.get("sink", True))
        if self.H % self.G:
            raise ValueError(f"rotated_value_attention: {self.H} heads are not a multiple of {self.G} key heads")
        if not (1 <= self.dk <= ops.MAX_HEAD_DIM and 1 <= self.dv <= ops.MAX_HEAD_DIM):
            raise ValueError(f"rotated_value_attention: head sizes up to {ops.MAX_HEAD_DIM} are supported")
        self.rot = 0 if self.position is None else int(self.position.head_dim)
        if self.rot % 2 or self.rot > self.dk:
            raise ValueError(f"rotated_value_attention: {self.rot} turned dimensions must be even and at most key_dim {self.dk}")
        if self.value_position is not None and (self.dv % 2 or int(self.value_position.head_dim) != self.dv):
            raise ValueError("rotated_value_attention: the values' rotation spans all of an even value_dim")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_qkv = self.w_o = self.biases = self.norm_w = self.sinks = None

    def tensors(self):
        n = self.names
        out = [TensorDecl(n["q"], (self.H * self.dk, self.D)), TensorDecl(n["k"], (self.G * self.dk, self.D)),
               TensorDecl(n["v"], (self.G * self.dv, self.D)), TensorDecl(n["o"], (self.D, self.H * self.dv))]
        if self.bias:
            out += [TensorDecl(n["q_bias"], (self.H * self.dk,)), TensorDecl(n["k_bias"], (self.G * self.dk,)),
                    TensorDecl(n["v_bias"], (self.G * self.dv,))]
        if self.qk_norm:
            out += [TensorDecl(n["q_norm"], (self.dk,), "ones_normal"), TensorDecl(n["k_norm"], (self.dk,), "ones_normal")]
        if self.sink:
            out.append(TensorDecl(n["sink"], (self.H,)))
        return out

    def load(self, get):
        to, f32, n = self.rt.to_compute, self.rt.to_f32, self.names
        self.w_qkv = torch.cat([to(get(n["q"])), to(get(n["k"])), to(get(n["v"]))], 0).contiguous()
        self.w_o = to(get(n["o"]))
        self.biases = tuple(f32(get(n[k])) for k in ("q_bias", "k_bias", "v_bias")) if self.bias else None
        self.norm_w = (f32(get(n["q_norm"])), f32(get(n["k_norm"]))) if self.qk_norm else None
        self.sinks = f32(get(n["sink"])) if self.sink else None

    def cache_need(self):
        return CacheNeed("window" if self.window else "full",
                         (("k", (self.G, self.dk)), ("v", (self.G, self.dv))), self.window)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o) if t is not None)

    def cache_bytes_per_query(self, context):
        seen = min(context, self.window) if self.window else context
        return seen * self.G * (self.dk + self.dv) * (2 if self.rt.dtype == torch.bfloat16 else 4)

    def flops(self, start, count):
        products = 2.0 * self.D * (self.H * self.dk + self.G * (self.dk + self.dv) + self.H * self.dv)
        first, last = start + 1, start + count
        tri = lambda a, b: (a + b) * (b - a + 1) / 2.0 if b >= a else 0.0      # noqa: E731
        if self.window:
            w = self.window
            seen = tri(first, min(last, w)) + w * max(0, last - max(first, w + 1) + 1)
        else:
            seen = tri(first, last)
        return count * products + 2.0 * self.H * (self.dk + self.dv) * seen

    def first_weights(self):
        return self.w_qkv

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        if not owns_cache:
            raise ValueError("rotated_value_attention: reading another entry's cache is not supported")
        T = h.shape[0]
        proj = self.rt.buffer("rva.proj", T, self.H * self.dk + self.G * (self.dk + self.dv), dtype=torch.float32)
        matmul_nt(self.rt, proj, h, self.w_qkv)                   # float32 out: the norms read unrounded sums
        kc, vc = cache.tensors["k"], cache.tensors["v"]
        q = self.rt.buffer("rva.q", T, self.H * self.dk)
        key_tables = self.position.tables() if self.rot else None
        value_tables = self.value_position.tables() if self.value_position is not None else None
        ops.qkv_norm_rot_write(q, kc, vc, proj, self.biases, self.norm_w, self.eps, key_tables, self.rot, value_tables,
                               self.value_norm, cache.tables, ctx.tok_seq, ctx.tok_pos, self.H, self.G, self.dk, self.dv)
        o = self.rt.buffer("rva.o", T, self.H * self.dv)
        from . import attention_dispatch as ad
        ad.split_attend(self.rt, o, q, kc, vc, cache.tables, ctx, self.H, self.G, self.dk, self.dv, self.window, self.scale,
                        0.0, self.sinks, unrotate=value_tables)      # the turn back happens where the result is stored
        matmul_nt(self.rt, residual, o, self.w_o, accumulate=not overwrite)
