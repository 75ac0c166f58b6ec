"""Mixer `latent_attention`: attention whose keys and values are projections of one small latent per token, so
that the latent (and one shared, turned key part) is all the cache keeps.

    q_h = (Wq h)_h                                      or, with a query latent (q_rank),  (Wuq (R(Wdq h) * wq))_h
          laid out per head as [dk dimensions without position | rd turned dimensions]
    d = Wdkv h:  c = R(d[:r]) * wc  (the latent),  kr = turn(d[r:], position)  (rd values shared by all heads)
    k_h,j = [Wuk_h c_j | kr_j],  v_h,j = Wuv_h c_j,  s_j = scale * q_h . k_h,j for j <= t,  softmax,  o_h = sum_j p_j v_h,j
    x += Wo (concat_h o_h [* sigmoid(Wg h)])
R(u) = u / sqrt(mean(u^2) + eps); turn: pairs (2i, 2i + 1), i < dims/2, by the angle position * base^(-2i/dims).

How it is computed: keys and values are never expanded.  The query goes through the key projection first,
qa_h = Wuk_h^T q_h[:dk] (r values), so that s_j = scale * (qa_h . c_j + turn(q_h[dk:]) . kr_j) reads the cache rows
[c_j | kr_j] directly, the same rows for every head; the heads' sums u_h = sum_j p_j c_j (r values) go through the
value projection afterwards, o_h = Wuv_h u_h.  A prompt, a piece of one and a decoded token take the same path.
A layer with `cache_from` in its schedule entry has no Wdkv: it reads the rows another layer wrote for the same
tokens, with projections of its own.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import MIXERS, Part
from .spec import CacheNeed, TensorDecl

_NAMES = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
          "uv": "uv", "g": "g", "o": "o"}
HEAD_MATMUL_MAX_TOKENS = 16       # up to here the per-head products run as one launch that streams the weights once


@MIXERS.register("latent_attention")
class LatentAttention(Part):
    graph_safe = True
    can_overwrite = True
    """params: hidden_size, num_heads, key_dim (per head, without position), value_dim, kv_rank, scale, eps,
    rot_dim (0 or None: no turned part), position (a `rotary_pairs` encoding; its dims <= rot_dim), q_rank (0 or None:
    queries straight from the input), gate (sigmoid output gate), reads_cache (the layer owns no down projection: it
    reads another entry's cache), tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.H = int(self._need("num_heads"))
        self.dk = int(self._need("key_dim"))
        self.dv = int(self._need("value_dim"))
        self.r = int(self._need("kv_rank"))
        self.scale = float(self._need("scale"))
        self.eps = float(self._need("eps"))
        self.rd = int(self.params.get("rot_dim") or 0)
        self.q_rank = int(self.params.get("q_rank") or 0)
        self.gate = bool(self.params.get("gate", False))
        self.reads_cache = bool(self.params.get("reads_cache", False))
        self.position = self.params.get("position") if self.rd else None
        self.dims = 0 if self.position is None else int(self.position.dims)
        if self.dims > self.rd:
            raise ValueError(f"latent_attention: {self.dims} turned dimensions exceed rot_dim {self.rd}")
        if not 1 <= self.r <= 512:
            raise ValueError("latent_attention: kv_rank up to 512 is supported")
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w = {}

    @property
    def R(self):
        return self.r + self.rd

    def tensors(self):
        n, qd = self.names, self.H * (self.dk + self.rd)
        out = []
        if self.q_rank:
            out += [TensorDecl(n["dq"], (self.q_rank, self.D)), TensorDecl(n["dq_norm"], (self.q_rank,), "ones_normal"),
                    TensorDecl(n["uq"], (qd, self.q_rank))]
        else:
            out.append(TensorDecl(n["q"], (qd, self.D)))
        if not self.reads_cache:
            out += [TensorDecl(n["dkv"], (self.R, self.D)), TensorDecl(n["dkv_norm"], (self.r,), "ones_normal")]
        out += [TensorDecl(n["uk"], (self.H * self.dk, self.r)), TensorDecl(n["uv"], (self.H * self.dv, self.r))]
        if self.gate:
            out.append(TensorDecl(n["g"], (self.H * self.dv, self.D)))
        out.append(TensorDecl(n["o"], (self.D, self.H * self.dv)))
        return out

    def load(self, get):
        to, f32, n = self.rt.to_compute, self.rt.to_f32, self.names
        w = {}
        # one product with float32 output for everything that is normed, turned or gated in float32: [dq | dkv | g]
        first = []
        if self.q_rank:
            first.append(to(get(n["dq"])))
            w["uq"] = to(get(n["uq"]))
            self.dq_norm = f32(get(n["dq_norm"]))
        else:
            w["q"] = to(get(n["q"]))
        self.off_dkv = sum(t.shape[0] for t in first)
        if not self.reads_cache:
            first.append(to(get(n["dkv"])))
            self.dkv_norm = f32(get(n["dkv_norm"]))
        self.off_g = sum(t.shape[0] for t in first)
        if self.gate:
            first.append(to(get(n["g"])))
        if first:
            w["in"] = torch.cat(first, 0).contiguous()
        uk = to(get(n["uk"])).reshape(self.H, self.dk, self.r)
        w["uk_t"] = uk.transpose(1, 2).contiguous()                       # [H, r, dk]: qa_h = uk_t[h] @ q_h
        w["uv"] = to(get(n["uv"])).reshape(self.H, self.dv, self.r).contiguous()      # [H, dv, r]: o_h = uv[h] @ u_h
        w["o"] = to(get(n["o"]))
        self.w = w

    def cache_need(self):
        return CacheNeed("full", (("latent", (self.R,)),))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.w.values())

    def cache_bytes_per_query(self, context):
        return context * self.R * (2 if self.rt.dtype == torch.bfloat16 else 4)

    def flops(self, start, count):
        qd = self.H * (self.dk + self.rd)
        products = 2.0 * self.D * ((self.q_rank or qd) + (0 if self.reads_cache else self.R) +
                                   (self.H * self.dv if self.gate else 0) + self.H * self.dv)
        products += 2.0 * self.q_rank * qd + 2.0 * self.H * self.r * (self.dk + self.dv)
        first, last = start + 1, start + count
        seen = (first + last) * (last - first + 1) / 2.0
        return count * products + 2.0 * self.H * (self.R + self.r) * seen

    def first_weights(self):
        return self.w.get("in") if self.w.get("in") is not None else self.w.get("q")

    def _per_head(self, out, a, w):
        """out[:, h, :] = w[h] @ a[:, h, :].  bfloat16: one launch for all heads, a kernel that streams the weights once
        for a handful of tokens, the tensor cores for more; else a product per head (float32: the CUDA-core product
        whose sums do not depend on the batch)."""
        T = a.shape[0]
        if self.rt.dtype == torch.bfloat16 and T <= HEAD_MATMUL_MAX_TOKENS:
            ops.head_matmul(out, a, w)
            return
        if self.rt.dtype == torch.bfloat16 and self.rt.tensor_cores:
            from ..csrc import ops_tc
            if ops_tc.head_matmul_supported(a, w, out):
                ops_tc.head_matmul(out, a, w)
                return
        for h in range(self.H):
            matmul_nt(self.rt, out[:, h, :], a[:, h, :], w[h])

    def forward(self, h, residual, ctx, cache, state, owns_cache=True, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        if owns_cache == self.reads_cache:
            raise ValueError("latent_attention: a layer without a down projection must read another entry's cache "
                             "(and one with it must own its cache)")
        T, f32, buf = h.shape[0], torch.float32, self.rt.buffer
        H, dk, dv, r, rd, R = self.H, self.dk, self.dv, self.r, self.rd, self.R
        qd = H * (dk + rd)
        proj = None
        if "in" in self.w:
            proj = buf("latent.in", T, self.w["in"].shape[0], dtype=f32)
            matmul_nt(self.rt, proj, h, self.w["in"])
        q = buf("latent.q", T, qd)
        if self.q_rank:
            cq = buf("latent.cq", T, self.q_rank)
            ops.group_rmsnorm(cq, proj[:, :self.q_rank], self.dq_norm, self.eps, 1)
            matmul_nt(self.rt, q, cq, self.w["uq"])
        else:
            matmul_nt(self.rt, q, h, self.w["q"])
        qfull = buf("latent.qfull", T, H * R)
        freq = self.position.tables()[0] if self.dims else None
        rows = cache.tensors["latent"]
        ops.latent_write(None if self.reads_cache else proj[:, self.off_dkv:self.off_dkv + R],
                         None if self.reads_cache else self.dkv_norm, self.eps, q, qfull, freq, self.dims,
                         rows, cache.tables, ctx, H, dk, r, rd, owns_cache)
        self._per_head(qfull.view(T, H, R)[:, :, :r], q.view(T, H, dk + rd)[:, :, :dk], self.w["uk_t"])
        u = buf("latent.u", T, H * r)
        from . import attention_dispatch as ad
        ad.latent_core(self.rt, u, qfull, rows, cache.tables, ctx, H, r, rd, self.scale)
        # with a gate the heads' outputs stay float32 until the gate has been applied
        o = buf("latent.o", T, H * dv, dtype=f32 if self.gate else None)
        self._per_head(o.view(T, H, dv), u.view(T, H, r), self.w["uv"])
        if self.gate:
            y = buf("latent.y", T, H * dv)
            ops.head_gate(y, o, proj[:, self.off_g:self.off_g + H * dv], None, H, dv, False, "sigmoid")
            o = y
        matmul_nt(self.rt, residual, o, self.w["o"], accumulate=not overwrite)
