"""Norms.  `rms_norm`: y = (x / sqrt(mean(x^2) + eps)) * w on the float32 residual stream,
computed in float32 and stored in the compute dtype (reference: core/ops.cpp:149-195; the
epsilon is a parameter here, always passed).  `add_into(dst, y, coef)` is the same norm applied to a
sublayer's float32 OUTPUT and added, times coef, into another float32 tensor (layers that norm what
a sublayer returns instead of what it reads).  With `groups` > 1 the row is cut into that many equal consecutive parts
and each part is divided by its own root mean square (the weight still spans the whole row).
`dynamic_tanh`: y = tanh(alpha x) * w + b with one scalar alpha and the vectors w, b: a norm that computes no
mean and no variance, so every value of a row is normed by itself."""
from __future__ import annotations

from ..csrc import ops
from .registry import NORMS, Part
from .spec import TensorDecl


@NORMS.register("rms_norm")
class RMSNorm(Part):
    graph_safe = True
    """params: size, eps, name (tensor name under the prefix), offset (added to the stored weight: 1.0 for a
    weight that is kept around zero, y = x / rms * (1 + w); default 0), groups (default 1)."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(self._need("size"))
        self.eps = float(self._need("eps"))
        self.name = prefix + self._need("name")
        self.offset = float(self.params.get("offset", 0.0) or 0.0)
        self.groups = int(self.params.get("groups") or 1)
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"rms_norm: {self.size} values do not split into {self.groups} equal groups")
        self.weight = None

    def tensors(self):
        return [TensorDecl(self.name, (self.size,), "normal" if self.offset else "ones_normal")]

    def load(self, get):
        self.weight = self.rt.to_f32(get(self.name))
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()        # float32: the sum the design asks for

    def weight_bytes(self):
        return 0 if self.weight is None else self.weight.numel() * self.weight.element_size()

    def forward(self, x):
        y = self.rt.empty(*x.shape)
        if self.groups > 1:
            ops.group_rmsnorm(y, x, self.weight, self.eps, self.groups)
        else:
            ops.rmsnorm(y, x, self.weight, self.eps)
        return y

    def add_into(self, dst, y, coef: float = 1.0, accumulate: bool = True, keep_cast: bool = False) -> None:
        """dst (+)= coef * norm(y); dst and y float32 of one shape.  keep_cast: on the bfloat16 path the kernel
        also leaves the new dst rounded to bfloat16 for the sublayer that reads it next (Runtime.activations)."""
        cast = None
        if keep_cast and self.rt.dtype != dst.dtype:
            # two buffers in turn: the copy a sublayer is reading stays while the next one is written
            self.rt._cast_turn ^= 1
            cast = self.rt.buffer(f"stream_copy{self.rt._cast_turn}", *dst.shape)
            self.rt.cast_cache = (dst.data_ptr(), cast)
        if self.groups > 1:
            ops.group_rmsnorm_add(dst, y, self.weight, self.eps, self.groups, coef, accumulate, cast)
        else:
            ops.rmsnorm_add(dst, y, self.weight, self.eps, coef, accumulate, cast)


@NORMS.register("dynamic_tanh")
class DynamicTanh(Part):
    graph_safe = True
    """params: size, name (the weight's tensor name under the prefix), bias and alpha (tensor names; default: the weight's
    name + ".b" and + ".alpha").  alpha is a scalar tensor, read once when the weights are loaded."""

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(self._need("size"))
        base = self._need("name")
        self.name = prefix + base
        self.bias_name = prefix + (self.params.get("bias") or base + ".b")
        self.alpha_name = prefix + (self.params.get("alpha") or base + ".alpha")
        self.weight = self.bias = None
        self.alpha = 1.0

    def tensors(self):
        return [TensorDecl(self.name, (self.size,), "ones_normal"), TensorDecl(self.bias_name, (self.size,)),
                TensorDecl(self.alpha_name, (), "ones_normal")]

    def load(self, get):
        self.weight, self.bias = self.rt.to_f32(get(self.name)), self.rt.to_f32(get(self.bias_name))
        self.alpha = float(get(self.alpha_name).to("cpu", dtype=__import__("torch").float32).reshape(-1)[0])

    def weight_bytes(self):
        return 0 if self.weight is None else 2 * self.weight.numel() * self.weight.element_size()

    def forward(self, x):
        y = self.rt.empty(*x.shape)
        ops.dyt_norm(y, x, self.weight, self.bias, self.alpha)
        return y
