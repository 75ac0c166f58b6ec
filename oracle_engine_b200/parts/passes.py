"""Parts that work on the residual stream between layers (STREAM_PARTS).

`pass_entry`: what a looped group of layers adds to the stream when a pass begins.  With x_e the embedding's output of
the forward pass and s [passes, hidden] a tensor of the model, before pass t (t = 0, 1, ...):
    x <- x + x_e  (t > 0 only);    x <- x + s[t]
A schedule entry names it in `before` with the argument `index` = t; the model keeps x_e for the pass."""
from __future__ import annotations

from ..csrc import ops
from .registry import STREAM_PARTS, Part
from .spec import TensorDecl


@STREAM_PARTS.register("pass_entry")
class PassEntry(Part):
    """params: hidden_size, passes, name (the tensor [passes, hidden]), add_embedding (default True: passes after the
    first add the embedding's output)."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.D = int(self._need("hidden_size"))
        self.passes = int(self._need("passes"))
        self.name = prefix + self._need("name")
        self.add_embedding = bool(self.params.get("add_embedding", True))
        self.needs_embedding_output = self.add_embedding and self.passes > 1
        self.steps = None

    def tensors(self):
        return [TensorDecl(self.name, (self.passes, self.D))]

    def load(self, get):
        self.steps = self.rt.to_f32(get(self.name))

    def forward(self, x, ctx, index: int):
        if not 0 <= index < self.passes:
            raise ValueError(f"pass_entry: pass {index} of {self.passes}")
        e = None
        if index > 0 and self.add_embedding:
            e = self.rt.pass_store.get("embedding_output")
            if e is None or tuple(e.shape) != tuple(x.shape):
                raise ValueError("pass_entry: the embedding's output of this pass was not kept")
        ops.pass_entry_add(x, e, self.steps[index])
