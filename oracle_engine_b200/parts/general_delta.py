"""Mixer `general_delta`: a generalized delta rule, a recurrent layer whose memory is one matrix S [d, d] per head
and sequence, with a decay and a removal rate per key channel.

With h the layer's input, per token and head:
    r = Wr h, k = Wk h, v = Wv h
    w = exp(-c * sigmoid(W2 tanh(W1 h) + w0))          the decay, one per key channel; c a constant of the design
    a = sigmoid(Wa h + ba)                             the removal rate, one per key channel
    u = k / sqrt(|k|^2 + 1e-6)                         the unit key
    S <- diag(w) S - (a * u) (u^T S) + k v^T           (both terms read the old S);    o = S^T r
    x += Wo (o / sqrt(mean(o^2) + eps) * w_norm * sigmoid(Wg h))        the read-out normed per head

The six projections are one matrix product whose output is float32 (decays, rates, unit keys and everything the
recurrence reads stay in float32); the small product with W2 is done in float32 inside the kernel that prepares
the scan's vectors.  S is per-sequence state (float32, zero when a sequence starts).  Prompts, pieces of prompts and
single tokens run the same kernels.
"""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import StateNeed, TensorDecl

_NAMES = {"r": "mix.r", "k": "mix.k", "v": "mix.v", "g": "mix.g", "a": "mix.a", "a_bias": "mix.a.b", "w1": "mix.w1",
          "w2": "mix.w2", "w0": "mix.w0", "norm": "mix.norm", "o": "mix.o"}


@MIXERS.register("general_delta")
class GeneralDelta(Part):
    graph_safe = True
    can_overwrite = True
    """params: hidden_size, num_heads, head_dim, eps (of the read-out's norm), decay_coef (c above; default
    exp(-1/2)), rank (of the decay's two-matrix projection; None: the file gives it), tensor_names (optional
    overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.d = int(self._need("head_dim"))
        self.eps = float(self._need("eps"))
        self.decay_coef = float(self.params.get("decay_coef") or math.exp(-0.5))
        self.rank = int(self.params.get("rank") or -1)
        if not 1 <= self.d <= 256:
            raise ValueError("general_delta: head sizes up to 256 are supported")
        self.C = self.H * self.d
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_in = self.w_o = None

    def tensors(self):
        n, C = self.names, self.C
        return [TensorDecl(n["r"], (C, self.D)), TensorDecl(n["k"], (C, self.D)), TensorDecl(n["v"], (C, self.D)),
                TensorDecl(n["g"], (C, self.D)), TensorDecl(n["a"], (C, self.D)), TensorDecl(n["a_bias"], (C,)),
                TensorDecl(n["w1"], (self.rank, self.D)), TensorDecl(n["w2"], (C, self.rank)), TensorDecl(n["w0"], (C,)),
                TensorDecl(n["norm"], (C,), "ones_normal"), TensorDecl(n["o"], (self.D, C))]

    def load(self, get):
        to, f32, n = self.rt.to_compute, self.rt.to_f32, self.names
        w1 = to(get(n["w1"]))
        self.rank = int(w1.shape[0])
        self.w_in = torch.cat([to(get(n[k])) for k in ("r", "k", "v", "g", "a")] + [w1], 0).contiguous()
        self.w2, self.w0, self.a_bias = f32(get(n["w2"])), f32(get(n["w0"])), f32(get(n["a_bias"]))
        if self.w2.shape[1] != self.rank:
            raise ValueError(f"general_delta: {n['w2']} has {self.w2.shape[1]} columns, {n['w1']} has {self.rank} rows")
        self.norm_w = f32(get(n["norm"]))
        self.w_o = to(get(n["o"]))

    def state_need(self):
        return {"S": StateNeed((self.H, self.d, self.d), torch.float32)}

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o) if t is not None)

    def state_bytes_per_query(self) -> int:
        """Bytes of state one sequence's token reads and writes."""
        return 2 * 4 * self.H * self.d * self.d

    def cache_bytes_per_query(self, context):
        return self.state_bytes_per_query()

    def flops(self, start, count):
        rank = max(self.rank, 0)
        products = 2.0 * self.D * (6 * self.C + rank) + 2.0 * self.C * rank
        return count * (products + 8.0 * self.H * self.d * self.d)

    def first_weights(self):
        return self.w_in

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T, f32, C = h.shape[0], torch.float32, self.C
        buf = self.rt.buffer
        proj = buf("gdelta.proj", T, 5 * C + self.rank, dtype=f32)
        matmul_nt(self.rt, proj, h, self.w_in)
        dkp = ops.gdelta_padded_dk(self.d)
        packed = buf("gdelta.packed", T, self.H, 5 * dkp + 4, dtype=f32)
        ops.gdelta_prepare(packed, proj, 0, C, 4 * C, 5 * C, self.rank, self.w2, self.w0, self.a_bias, self.decay_coef,
                           ctx.tok_seq, self.H, self.d)
        o = buf("gdelta.o", T, C, dtype=f32)
        ops.gdelta_scan(o, state["S"], packed, proj[:, 2 * C:3 * C], ctx, self.H, self.d, self.d)
        y = buf("gdelta.y", T, C)
        ops.head_gate(y, o, proj[:, 3 * C:4 * C], self.norm_w, self.H, self.d, True, "sigmoid", self.eps)
        matmul_nt(self.rt, residual, y, self.w_o, accumulate=not overwrite)
