"""Feed-forward `moe_swiglu`: a mixture of experts with an optional shared expert.

    z = Wr h (float32);  the `top` experts with the largest z are chosen, their weights w_e are the softmax over the
    chosen z alone;  E_e(h) = Wdown_e (silu(Wgate_e h) * (Wup_e h));
    y = sum_chosen w_e E_e(h) + sigmoid(Wsg h) * E_shared(h)                   (the second term only with a shared expert)
Variants by parameter: the weights may be each chosen expert's own sigmoid(z_e), not renormalised; the weight may
multiply the expert's input, y = sum_chosen E_e(w_e h) (its gate and up rows are linear in the input, so the kernel
scales those: silu(w_e g) * (w_e u)); the shared expert may be added without a gate; the choice may be by
sigmoid(z_e) + a learned bias per expert while the weights stay the sigmoids; the experts' unit may be clamped and
shifted, g = min(Wgate h, L), u = clamp(Wup h, -L, L), E_e(h) = Wdown_e (g * sigmoid(1.702 g) * (u + 1)).

How it is computed: the experts stand side by side.  One product with all gate and up matrices (the shared expert's
behind the routed ones), one kernel that applies silu(gate) * up and multiplies each expert's columns by the token's
weight for that expert (zero where it was not chosen, sigmoid(Wsg h) for the shared one), and one product with all
down matrices side by side, which sums the chosen experts in its float32 accumulators.  The router and the shared
gate are one small float32 product.  No token is moved and nothing depends on the host, so a step is the same
kernels whatever the routing (and can be captured in a graph); the price is the products of the experts a token
did not choose, experts / top times the arithmetic of the chosen ones, while the weights read are the same as
soon as a step's tokens choose every expert between them.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import FEED_FORWARDS, Part
from .spec import TensorDecl


@FEED_FORWARDS.register("moe_swiglu")
class MoESwiGLU(Part):
    graph_safe = True
    can_overwrite = True
    """params: hidden_size, num_experts, top, expert_size, shared_size (0 or None: no shared expert), router_weights
    ("softmax", the default: the softmax over the chosen logits alone; "sigmoid": each chosen expert's own
    sigmoid(logit), not renormalised), weight_on ("output", the default: y = sum w_e E_e(h); "input": y = sum E_e(w_e h)),
    shared_gate (default True: the shared expert's output times sigmoid(Wsg h); False: added as it is), choice_bias
    (True: a tensor of one value per expert is added to the sigmoids for the choice alone; needs router_weights
    "sigmoid"), activation ("silu", the default, or "clamped" with `limit`), tensor_names (optional overrides of
    "expert" (a format with {e}), "router", "shared", "shared_gate", "choice_bias")."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.E = int(self._need("num_experts"))
        self.top = int(self._need("top"))
        self.ff = int(self._need("expert_size"))
        self.sff = int(self.params.get("shared_size") or 0)
        self.router_weights = self.params.get("router_weights") or "softmax"
        self.weight_on = self.params.get("weight_on") or "output"
        self.shared_gate = bool(self.params.get("shared_gate", True)) and self.sff > 0
        if self.router_weights not in ("softmax", "sigmoid") or self.weight_on not in ("output", "input"):
            raise ValueError("moe_swiglu: router_weights is softmax or sigmoid, weight_on is output or input")
        self.choice_bias = bool(self.params.get("choice_bias", False))
        self.activation = self.params.get("activation") or "silu"
        self.limit = float(self.params.get("limit") or 0.0)
        if self.activation not in ("silu", "clamped") or (self.activation == "clamped" and not self.limit > 0):
            raise ValueError("moe_swiglu: activation is silu or clamped (with a positive limit)")
        if self.activation == "clamped" and self.weight_on != "output":
            raise ValueError("moe_swiglu: the clamped unit is not linear in its input; its weight goes on the output")
        if self.choice_bias and self.router_weights != "sigmoid":
            raise ValueError("moe_swiglu: a choice bias is added to sigmoids; router_weights must be sigmoid")
        if not 1 <= self.top <= self.E:
            raise ValueError(f"moe_swiglu: top {self.top} of {self.E} experts")
        if self.E > 1024:
            raise ValueError("moe_swiglu: up to 1,024 experts are supported")
        names = {"expert": "mlp.e{e}.", "router": "mlp.router", "shared": "mlp.shared.", "shared_gate": "mlp.shared.sg",
                 "choice_bias": "mlp.correction",
                 **self.params.get("tensor_names", {})}
        self.names = {k: prefix + v for k, v in names.items()}
        self.F = self.E * self.ff + self.sff
        self.w_route = self.w_gu = self.w_down = self.bias = None

    def _expert_names(self):
        out = [self.names["expert"].format(e=e) for e in range(self.E)]
        return out + ([self.names["shared"]] if self.sff else [])

    def tensors(self):
        out = []
        for i, p in enumerate(self._expert_names()):
            f = self.ff if i < self.E else self.sff
            out += [TensorDecl(p + "gate", (f, self.D)), TensorDecl(p + "up", (f, self.D)),
                    TensorDecl(p + "down", (self.D, f))]
        out.append(TensorDecl(self.names["router"], (self.E, self.D)))
        if self.shared_gate:
            out.append(TensorDecl(self.names["shared_gate"], (1, self.D)))
        if self.choice_bias:
            out.append(TensorDecl(self.names["choice_bias"], (self.E,)))
        return out

    def load(self, get):
        to = self.rt.to_compute
        ex = self._expert_names()
        self.w_gu = torch.cat([to(get(p + "gate")) for p in ex] + [to(get(p + "up")) for p in ex], 0).contiguous()
        self.w_down = torch.cat([to(get(p + "down")) for p in ex], 1).contiguous()
        route = [to(get(self.names["router"]))] + ([to(get(self.names["shared_gate"]))] if self.shared_gate else [])
        self.w_route = torch.cat(route, 0).contiguous()
        if self.choice_bias:
            self.bias = self.rt.to_f32(get(self.names["choice_bias"]))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gu, self.w_down, self.w_route) if t is not None)

    def flops(self, start, count):
        return count * 2.0 * self.D * (3 * self.F + self.w_route_rows())

    def w_route_rows(self):
        return self.E + (1 if self.shared_gate else 0)

    def first_weights(self):
        return self.w_gu

    def forward(self, h, residual, ctx, overwrite: bool = False):
        """overwrite: the output is written into `residual` (float32) instead of added."""
        T = h.shape[0]
        z = self.rt.buffer("moe.z", T, self.w_route_rows(), dtype=torch.float32)
        matmul_nt(self.rt, z, h, self.w_route)                  # float32 sums and output on both paths
        dense = self.rt.buffer("moe.dense", T, self.E + (1 if self.sff else 0), dtype=torch.float32)
        ops.moe_route(z, self.E, self.top, (True if self.shared_gate else "one") if self.sff else False, dense,
                      ctx.tok_seq, weights=self.router_weights, bias=self.bias)
        gu = self.rt.buffer("moe.gu", T, 2 * self.F)
        matmul_nt(self.rt, gu, h, self.w_gu)
        a = self.rt.buffer("moe.a", T, self.F)
        ops.moe_dense_act(a, gu, dense, self.E, self.ff, scale_input=self.weight_on == "input", act=self.activation,
                          limit=self.limit)
        matmul_nt(self.rt, residual, a, self.w_down, accumulate=not overwrite)
