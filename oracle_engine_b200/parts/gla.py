"""Mixer `gated_linear_attention`: linear attention with a data-dependent decay per key channel; a recurrent layer
whose memory is one matrix S [dk, dv] per head and sequence.

    q = (Wq h) dk^(-1/2), k = Wk h [H, dk], v = Wv h [H, dv]                                    (no bias)
    alpha = sigmoid(Wa2 (Wa1 h) + b)^(1/tau) [H, dk]            (two thin matrices; the rank is the file's)
    S <- diag(alpha) S + k v^T;   o = S^T q                     per head, S starts at zero; o reads the new S
    x += Wo (concat_h (o_h / sqrt(mean(o_h^2) + eps) * wn) * silu(Wg h))       wn [dv], shared by the heads
The projections leave their products as float32 on both paths, so nothing that enters the recurrence is rounded to
16 bits; the decay (sigmoid, its power), S and the read-out's norm are float32.  The scan (csrc/gla.cu) takes a
step's tokens one by one in order, whatever their number.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import StateNeed, TensorDecl

_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}


SEGMENTS_FROM = 256         # a step whose longest sequence brings this many tokens runs them as segments side by side
SEGMENT_MIN = 32            # tokens of the shortest segment
SEGMENT_BLOCKS = 2368       # blocks of the scan that keep the GPU busy (16 per SM)


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Part):
    graph_safe = True
    can_overwrite = True
    """params: hidden_size, num_heads, key_dim, value_dim, tau, eps (of the read-out's norm), decay_rank (None: the
    shape of `a1` in the file gives it), tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.dk = int(self._need("key_dim"))
        self.dv = int(self._need("value_dim"))
        self.tau = float(self._need("tau"))
        self.eps = float(self._need("eps"))
        self.rank = int(self.params.get("decay_rank") or -1)
        if not 1 <= self.dk <= 256:
            raise ValueError("gated_linear_attention: key_dim up to 256 is supported")
        if not self.tau > 0:
            raise ValueError("gated_linear_attention: tau must be positive")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_in = self.w_a1 = self.w_a2 = self.w_o = self.bias = self.norm_w = None

    def tensors(self):
        n, qk, vv = self.names, self.H * self.dk, self.H * self.dv
        return [TensorDecl(n["q"], (qk, self.D)), TensorDecl(n["k"], (qk, self.D)), TensorDecl(n["v"], (vv, self.D)),
                TensorDecl(n["g"], (vv, self.D)), TensorDecl(n["o"], (self.D, vv)),
                TensorDecl(n["norm"], (self.dv,), "ones_normal"), TensorDecl(n["a1"], (self.rank, self.D)),
                TensorDecl(n["a2"], (qk, self.rank)), TensorDecl(n["a2_bias"], (qk,))]

    def load(self, get):
        to, f32, n = self.rt.to_compute, self.rt.to_f32, self.names
        a1 = to(get(n["a1"]))
        self.w_a2 = to(get(n["a2"]))
        self.rank = int(a1.shape[0])
        if self.w_a2.shape[1] != self.rank:
            raise ValueError(f"{n['a2']}: {self.w_a2.shape[1]} columns, but {n['a1']} has {self.rank} rows")
        self.w_a1 = a1
        # one product with float32 output for what enters the recurrence and the gate: [q | k | v | g]
        self.w_in = torch.cat([to(get(n[k])) for k in ("q", "k", "v", "g")], 0).contiguous()
        self.w_o = to(get(n["o"]))
        self.bias, self.norm_w = f32(get(n["a2_bias"])), f32(get(n["norm"]))

    def state_need(self):
        return {"S": StateNeed((self.H, self.dk, self.dv), torch.float32)}

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_a1, self.w_a2, self.w_o) if t is not None)

    def cache_bytes_per_query(self, context):
        return 2 * 4 * self.H * self.dk * self.dv          # the state, read and written

    def flops(self, start, count):
        qk, vv = self.H * self.dk, self.H * self.dv
        return count * (2.0 * self.D * (2 * qk + 3 * vv + max(self.rank, 0)) + 2.0 * max(self.rank, 0) * qk +
                        4.0 * self.H * self.dk * self.dv)

    def first_weights(self):
        return self.w_in

    def _segments(self, ctx):
        """How a step with long prompts cuts its sequences into segments that run side by side (csrc/gla.cu), or None
        for the one walk.  float32 serving keeps the one walk: there a position's logits are the same bits under
        every cut of the prompt into steps."""
        longest = int(ctx.max_qlen)
        if self.rt.dtype != torch.bfloat16 or longest < SEGMENTS_FROM or torch.cuda.is_current_stream_capturing():
            return None             # (a captured step's longest sequence is a bound, not a length)
        pairs = -(-SEGMENT_BLOCKS // (self.H * -(-self.dv // 32)))         # (sequence, segment) pairs that fill the GPU
        n_seg = max(1, min(-(-pairs // max(1, ctx.n_seqs)), longest // SEGMENT_MIN))
        seg_len = -(-(-(-longest // n_seg)) // 8) * 8
        n_seg = -(-longest // seg_len)
        if n_seg < 2:
            return None
        seg_state = self.rt.buffer("gla.seg_state", ctx.n_seqs * n_seg, self.H, self.dk * self.dv, dtype=torch.float32)
        seg_decay = self.rt.buffer("gla.seg_decay", ctx.n_seqs * n_seg, self.H, self.dk, dtype=torch.float32)
        return seg_len, n_seg, seg_state, seg_decay

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T, f32, buf = h.shape[0], torch.float32, self.rt.buffer
        qk, vv = self.H * self.dk, self.H * self.dv
        proj = buf("gla.in", T, 2 * qk + 2 * vv, dtype=f32)
        matmul_nt(self.rt, proj, h, self.w_in)
        low = buf("gla.low", T, self.rank)             # the second thin product's operand, in the compute dtype
        matmul_nt(self.rt, low, h, self.w_a1)
        z = buf("gla.z", T, qk, dtype=f32)
        matmul_nt(self.rt, z, low, self.w_a2)
        o = buf("gla.o", T, vv, dtype=f32)
        ops.gla_scan(o, state["S"], proj, 0, qk, 2 * qk, z, self.bias, ctx, self.H, self.dk, self.dv, self.dk ** -0.5,
                     self.tau, segments=self._segments(ctx))
        y = buf("gla.y", T, vv)
        ops.head_gate(y, o, proj[:, 2 * qk + vv:2 * qk + 2 * vv], self.norm_w, self.H, self.dv, True, "silu", self.eps)
        matmul_nt(self.rt, residual, y, self.w_o, accumulate=not overwrite)
