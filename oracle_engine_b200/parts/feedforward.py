"""Feed-forward `swiglu`: g = Wg h, u = Wu h, a = g/(1+exp(-g)) * u, x += Wd a  (dense, no
routing).  Reference: core/model.cpp:452-473 and :636-643.  The gate and up projections
are fused into one matrix product at load ([Wg; Wu]).
Feed-forward `relu2`: a = max(Wu h, 0)^2, x += Wd a (dense, no gate)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import chain_flags, matmul_nt
from .registry import FEED_FORWARDS, Part
from .spec import TensorDecl

_NAMES = {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"}


@FEED_FORWARDS.register("swiglu")
class SwiGLU(Part):
    graph_safe = True
    """params: hidden_size, intermediate_size, tensor_names (optional overrides)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.FF = int(self._need("intermediate_size"))
        self.names = {k: prefix + v for k, v in {**_NAMES, **self.params.get("tensor_names", {})}.items()}
        self.w_gu = self.w_down = None

    def tensors(self):
        return [TensorDecl(self.names["gate"], (self.FF, self.D)), TensorDecl(self.names["up"], (self.FF, self.D)),
                TensorDecl(self.names["down"], (self.D, self.FF))]

    def load(self, get):
        to = self.rt.to_compute
        gate, up = to(get(self.names["gate"])), to(get(self.names["up"]))
        # On the tensor-core path the activation is fused into the product's epilogue, which
        # wants gate and up rows of a feature side by side: rows g0, u0, g1, u1, ...
        self.fused = self.rt.dtype == torch.bfloat16 and self.rt.tensor_cores and self.D % 8 == 0
        if self.fused:
            self.w_gu = torch.stack([gate, up], 1).reshape(2 * self.FF, self.D).contiguous()
        else:
            self.w_gu = torch.cat([gate, up], 0)
        self.w_down = to(get(self.names["down"]))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gu, self.w_down) if t is not None)

    def flops(self, start, count):
        return count * 2.0 * 3 * self.D * self.FF

    def first_weights(self):
        return self.w_gu

    def forward(self, h, residual, ctx):
        T = h.shape[0]
        a = self.rt.empty(T, self.FF)
        if self.fused:
            from ..csrc import ops_tc
            ops_tc.gemm(a, h, self.w_gu, swiglu=True, early=chain_flags("ffn_in", T), then=self.w_down)
        else:
            gu = self.rt.empty(T, 2 * self.FF)
            matmul_nt(self.rt, gu, h, self.w_gu)
            ops.swiglu(a, gu)
        matmul_nt(self.rt, residual, a, self.w_down, accumulate=True, early=chain_flags("ffn_out", T),
                  then=self.rt.next_weights)


@FEED_FORWARDS.register("relu2")
class SquaredReLU(Part):
    graph_safe = True
    """params: hidden_size, intermediate_size, tensor_names (optional overrides of "up" and "down")."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.FF = int(self._need("intermediate_size"))
        names = {"up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight", **self.params.get("tensor_names", {})}
        self.names = {k: prefix + v for k, v in names.items()}
        self.w_up = self.w_down = None

    def tensors(self):
        return [TensorDecl(self.names["up"], (self.FF, self.D)), TensorDecl(self.names["down"], (self.D, self.FF))]

    def load(self, get):
        self.w_up = self.rt.to_compute(get(self.names["up"]))
        self.w_down = self.rt.to_compute(get(self.names["down"]))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down) if t is not None)

    def flops(self, start, count):
        return count * 2.0 * 2 * self.D * self.FF

    def first_weights(self):
        return self.w_up

    can_overwrite = True

    def forward(self, h, residual, ctx, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        a = self.rt.buffer("relu2.a", h.shape[0], self.FF)
        matmul_nt(self.rt, a, h, self.w_up)
        ops.relu2_(a)
        matmul_nt(self.rt, residual, a, self.w_down, accumulate=not overwrite)


@FEED_FORWARDS.register("poly_norm_mlp")
class PolyNormMLP(Part):
    """x += Wd P(Wu h) with P(z) = a R(z) + b R(z^2) + c R(z^3) + e: powers element by element, R(u) = u / sqrt(mean(u^2)
    + eps) over a token's intermediate values, (a, b, c, e) a weight tensor of four numbers.  The up product leaves
    float32 (the norms' sums are float32 sums of float32 values); P writes the compute dtype.
    params: hidden_size, intermediate_size, eps, tensor_names (optional overrides of "up", "down", "act")."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.FF = int(self._need("intermediate_size"))
        self.eps = float(self._need("eps"))
        names = {"up": "mlp.up", "down": "mlp.down", "act": "mlp.act", **self.params.get("tensor_names", {})}
        self.names = {k: prefix + v for k, v in names.items()}
        self.w_up = self.w_down = self.coef = None

    def tensors(self):
        return [TensorDecl(self.names["up"], (self.FF, self.D)), TensorDecl(self.names["down"], (self.D, self.FF)),
                TensorDecl(self.names["act"], (4,), "ones_normal")]

    def load(self, get):
        self.w_up = self.rt.to_compute(get(self.names["up"]))
        self.w_down = self.rt.to_compute(get(self.names["down"]))
        self.coef = self.rt.to_f32(get(self.names["act"]))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down) if t is not None)

    def flops(self, start, count):
        return count * 2.0 * 2 * self.D * self.FF

    def first_weights(self):
        return self.w_up

    def forward(self, h, residual, ctx, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T = h.shape[0]
        z = self.rt.buffer("polynorm.z", T, self.FF, dtype=torch.float32)
        matmul_nt(self.rt, z, h, self.w_up)
        a = self.rt.buffer("polynorm.a", T, self.FF)
        ops.poly_norm(a, z, self.coef, self.eps)
        matmul_nt(self.rt, residual, a, self.w_down, accumulate=not overwrite)
