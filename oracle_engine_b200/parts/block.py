"""Arrangements of a layer's parts.  `pre_norm`: x += mixer(norm(x)); x += ffn(norm(x)),
the reference's layer (core/model.cpp:361-474).  The mixer and the feed-forward add their
outputs into the float32 residual stream themselves (fused into their last product).
`norm_after`: x += norm(mixer(x)); x += norm(ffn(x)): the sublayers read the residual stream itself and
their OUTPUT is normed before it is added; a sublayer adds its output into a zeroed float32 buffer.
`pre_norm_scaled`: x += m * s1 * mixer(norm(x)); x += m * s2 * ffn(norm(x)) with m one constant and s1, s2 one
weight per channel each (a layer scale).
`sandwich`: x += norm_1b(mixer(norm_1(x))); x += norm_2b(ffn(norm_2(x))): a norm before and after every sublayer;
optionally followed by a per-token side input (`TokenSide`) and an average over the depth (`DepthAverage`)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import BLOCKS, Part
from .spec import TensorDecl


@BLOCKS.register("pre_norm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None]

    def first_weights(self):
        """The weight matrix this block streams first (a hint for the part that runs before it), or None."""
        return _first_weights(self.mixer)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        rt = getattr(self.mixer, "rt", None)
        after = getattr(rt, "next_weights", None)          # what the model says comes after this block
        h = self.mixer_norm.forward(x)
        if rt is not None:
            rt.next_weights = _first_weights(self.feed_forward) if self.feed_forward is not None else after
        self.mixer.forward(h, x, ctx, cache, state, owns_cache)
        if self.feed_forward is not None:
            h = self.ffn_norm.forward(x)
            if rt is not None:
                rt.next_weights = after
            self.feed_forward.forward(h, x, ctx)
        if rt is not None:
            rt.next_weights = None


@BLOCKS.register("norm_after")
class NormAfterBlock:
    """x <- x + norm_1(mixer(x)); x <- x + norm_2(ffn(x)) (the second only with a feed-forward)."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm):
        if mixer_norm is None or (feed_forward is not None and ffn_norm is None):
            raise ValueError("norm_after: every sublayer needs the norm of its output")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm) if p is not None]

    def first_weights(self):
        return _first_weights(self.mixer)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        rt = self.mixer.rt
        rt.next_weights = None
        y = rt.buffer("sublayer_out", *x.shape, dtype=x.dtype)
        h = rt.activations(x)
        # a sublayer that can write its output (instead of adding it) saves the zeroing of the buffer
        if getattr(self.mixer, "can_overwrite", False):
            self.mixer.forward(h, y, ctx, cache, state, owns_cache, overwrite=True)
        else:
            y.zero_()
            self.mixer.forward(h, y, ctx, cache, state, owns_cache)
        self.mixer_norm.add_into(x, y, keep_cast=True)
        if self.feed_forward is not None:
            h = rt.activations(x)
            if getattr(self.feed_forward, "can_overwrite", False):
                self.feed_forward.forward(h, y, ctx, overwrite=True)
            else:
                y.zero_()
                self.feed_forward.forward(h, y, ctx)
            self.ffn_norm.add_into(x, y, keep_cast=True)


class ChannelScales(Part):
    """The per-channel weights of a block arrangement: params {"names": {key: tensor name under the prefix}, "size"}."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(self._need("size"))
        self.names = {k: prefix + v for k, v in self._need("names").items()}
        self.vec = {}

    def tensors(self):
        return [TensorDecl(n, (self.size,), "ones_normal") for n in self.names.values()]

    def load(self, get):
        self.vec = {k: self.rt.to_f32(get(n)) for k, n in self.names.items()}


@BLOCKS.register("pre_norm_scaled")
class PreNormScaledBlock:
    """x <- x + m * s1 * mixer(norm_1(x)); x <- x + m * s2 * ffn(norm_2(x)) (the second only with a feed-forward).
    params: hidden_size, residual_mult (m, default 1), mixer_scale / ffn_scale (tensor names of s1 / s2 under the
    layer's prefix; absent: no per-channel weight).  A sublayer that takes `scale=` applies m and s itself (in the
    kernel that adds its output); any other writes into a float32 buffer that one kernel scales and adds."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, params, prefix, runtime):
        if mixer_norm is None or (feed_forward is not None and ffn_norm is None):
            raise ValueError("pre_norm_scaled: every sublayer needs the norm of its input")
        self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm = mixer, feed_forward, mixer_norm, ffn_norm
        self.rt = runtime
        self.mult = float(params.get("residual_mult", 1.0))
        names = {}
        if params.get("mixer_scale"):
            names["mixer"] = params["mixer_scale"]
        if feed_forward is not None and params.get("ffn_scale"):
            names["ffn"] = params["ffn_scale"]
        self.scales = ChannelScales({"names": names, "size": params["hidden_size"]}, prefix, runtime)

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward, self.scales)
                if p is not None]

    def first_weights(self):
        return _first_weights(self.mixer)

    def _sublayer(self, part, key, h, x, *args):
        vec = self.scales.vec.get(key)
        if getattr(part, "can_scale", False):
            part.forward(h, x, *args, scale=(self.mult, vec))
            return
        y = self.rt.buffer("sublayer_out", *x.shape, dtype=torch.float32)
        if getattr(part, "can_overwrite", False):
            part.forward(h, y, *args, overwrite=True)
        else:
            y.zero_()
            part.forward(h, y, *args)
        ops.scaled_add(x, y, vec, self.mult)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        self.rt.next_weights = None
        self._sublayer(self.mixer, "mixer", self.mixer_norm.forward(x), x, ctx, cache, state, owns_cache)
        if self.feed_forward is not None:
            self._sublayer(self.feed_forward, "ffn", self.ffn_norm.forward(x), x, ctx)


class TokenSide(Part):
    """A per-token input added to the stream: every layer owns `dim` columns of a second embedding table,
        e = table[token][off : off + dim];  g = gelu_tanh(Wg x) * e;  y = Wp g;  x <- x + y / sqrt(mean(y^2) + eps) * w
    params: hidden_size, vocab_size, dim, offset (the layer's first column of the table), table_width, eps,
    names {table, gate, proj, norm} (the table's name is not under the layer's prefix)."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D, self.V = int(self._need("hidden_size")), int(self._need("vocab_size"))
        self.dim, self.offset = int(self._need("dim")), int(self._need("offset"))
        self.table_width = int(self._need("table_width"))
        self.eps = float(self._need("eps"))
        n = self._need("names")
        self.names = {"table": n["table"], "gate": prefix + n["gate"], "proj": prefix + n["proj"], "norm": prefix + n["norm"]}
        self.table = self.w_gate = self.w_proj = self.norm_w = None

    def tensors(self):
        n = self.names
        return [TensorDecl(n["table"], (self.V, self.table_width)), TensorDecl(n["gate"], (self.dim, self.D)),
                TensorDecl(n["proj"], (self.D, self.dim)), TensorDecl(n["norm"], (self.D,), "ones_normal")]

    def load(self, get):
        n = self.names
        # the layer keeps its own columns of the table only
        self.table = self.rt.to_compute(get(n["table"])[:, self.offset:self.offset + self.dim])
        self.w_gate, self.w_proj = self.rt.to_compute(get(n["gate"])), self.rt.to_compute(get(n["proj"]))
        self.norm_w = self.rt.to_f32(get(n["norm"]))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate, self.w_proj) if t is not None)

    def flops(self, start, count):
        return count * 4.0 * self.D * self.dim

    def forward(self, x, ctx):
        from .linear import matmul_nt
        T = x.shape[0]
        u = self.rt.buffer("side.u", T, self.dim, dtype=torch.float32)
        matmul_nt(self.rt, u, self.rt.activations(x), self.w_gate)
        g = self.rt.buffer("side.g", T, self.dim)
        ops.side_gate(g, u, self.table, 0, ctx.token_ids, ctx.tok_seq)
        y = self.rt.buffer("side.y", T, self.D, dtype=torch.float32)
        matmul_nt(self.rt, y, g, self.w_proj)
        ops.rmsnorm_add(x, y, self.norm_w, self.eps)


class DepthAverage(Part):
    """What leaves layer n (n = 0 for the first) is a weighted sum over the depth: with X_0 the stream that entered
    the first layer and X_(j+1) the result of layer j, x <- sum_{j <= n + 1} a[j] X_j, a the layer's own n + 2 weights.
    The X_j of a forward pass are kept in one float32 buffer [layers + 1, tokens, hidden] that lives for the pass.
    params: hidden_size, index (n), layers, name."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.index, self.layers = int(self._need("index")), int(self._need("layers"))
        self.name = prefix + self._need("name")
        self.weights = None

    def tensors(self):
        return [TensorDecl(self.name, (self.index + 2,), "ones_normal")]

    def load(self, get):
        self.weights = self.rt.to_f32(get(self.name))

    def enter(self, x):
        """The first layer makes the pass's buffer and keeps the entering stream in it; the others find it."""
        if self.index == 0:
            hist = self.rt.buffer("depth.history", self.layers + 1, x.shape[0], x.shape[1], dtype=torch.float32)
            self.rt.pass_store["depth.history"] = hist
            hist[0].copy_(x)

    def leave(self, x):
        hist = self.rt.pass_store.get("depth.history")
        if hist is None or tuple(hist.shape[1:]) != tuple(x.shape):
            raise ValueError("depth_average: the first layer of the pass has not run")
        ops.depth_average(x, hist, self.weights, self.index + 1)


@BLOCKS.register("sandwich")
class SandwichBlock:
    """x <- x + norm_1b(mixer(norm_1(x))); x <- x + norm_2b(ffn(norm_2(x))) (the second only with a feed-forward); then
    the token side input and the depth average, where the layer has them.
    params: hidden_size, mixer_out_norm / ffn_out_norm (PartSpec-like {kind, params} of the norms applied to the
    sublayers' outputs), token_side (params of `TokenSide`, or None), depth_average (params of `DepthAverage`, or None)."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, params, prefix, runtime):
        from .registry import NORMS
        if mixer_norm is None or (feed_forward is not None and ffn_norm is None):
            raise ValueError("sandwich: every sublayer needs the norm of its input")
        self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm = mixer, feed_forward, mixer_norm, ffn_norm
        self.rt = runtime

        def out_norm(key):
            spec = params[key]
            return NORMS.get(spec["kind"])(spec["params"], prefix, runtime)
        self.mixer_out_norm = out_norm("mixer_out_norm")
        self.ffn_out_norm = out_norm("ffn_out_norm") if feed_forward is not None else None
        self.side = TokenSide(params["token_side"], prefix, runtime) if params.get("token_side") else None
        self.depth = DepthAverage(params["depth_average"], prefix, runtime) if params.get("depth_average") else None

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_out_norm, self.ffn_norm, self.feed_forward,
                            self.ffn_out_norm, self.side, self.depth) if p is not None]

    def first_weights(self):
        return _first_weights(self.mixer)

    def _sublayer(self, part, out_norm, h, x, *args):
        y = self.rt.buffer("sublayer_out", *x.shape, dtype=torch.float32)
        if getattr(part, "can_overwrite", False):
            part.forward(h, y, *args, overwrite=True)
        else:
            y.zero_()
            part.forward(h, y, *args)
        out_norm.add_into(x, y)

    def forward(self, x, ctx, cache, state, owns_cache=True):
        self.rt.next_weights = None
        if self.depth is not None:
            self.depth.enter(x)
        self._sublayer(self.mixer, self.mixer_out_norm, self.mixer_norm.forward(x), x, ctx, cache, state, owns_cache)
        if self.feed_forward is not None:
            self._sublayer(self.feed_forward, self.ffn_out_norm, self.ffn_norm.forward(x), x, ctx)
        if self.side is not None:
            self.side.forward(x, ctx)
        if self.depth is not None:
            self.depth.leave(x)


def _first_weights(part):
    f = getattr(part, "first_weights", None)
    return f() if f is not None else None
