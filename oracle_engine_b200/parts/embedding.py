"""Token embedding and output head.

`token_embedding`: x = E[token] as float32 (core/model.cpp:352-358); an id outside the
table is an error, not clamped.  `lm_head`: logits = W x in float32, W a separate matrix
or, when tied, the embedding table (core/model.cpp:482-492); an optional constant `scale` multiplies the logits.
`pair_hash_embedding`: x = E[token] * scale + P[hash(previous token, token)], a second table indexed by a hash of
the token and the one before it; the previous token is per-sequence state."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import matmul_nt
from .registry import EMBEDDINGS, HEADS, Part
from .spec import StateNeed, TensorDecl


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.V = int(self._need("vocab_size"))
        self.D = int(self._need("hidden_size"))
        self.name = prefix + self._need("name")
        self.table = None
        self.err = None

    def tensors(self):
        return [TensorDecl(self.name, (self.V, self.D))]

    def load(self, get):
        self.table = self.rt.to_compute(get(self.name))
        self.err = torch.zeros(1, dtype=torch.int32, device=self.rt.device)

    def forward(self, ids, n_tokens, out=None):
        """The residual stream [n_tokens, hidden] float32 (written into `out` if given)."""
        x = self.rt.empty(n_tokens, self.D, dtype=torch.float32) if out is None else out
        ops.embed_gather(x, self.table, ids, self.err)
        return x


@EMBEDDINGS.register("pair_hash_embedding")
class PairHashEmbedding(Part):
    """x_t = E[tok_t] * scale + P[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets]; a sequence's first token takes row
    `buckets` (the last) of P.  The token before a step's first one is the state `prev` (one int32 per slot), so the
    sum does not depend on how a sequence is cut into steps.
    params: vocab_size, hidden_size, name, scale (default 1), pair (None, or {name, buckets, mul_prev, mul_cur})."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.V = int(self._need("vocab_size"))
        self.D = int(self._need("hidden_size"))
        self.name = prefix + self._need("name")
        self.scale = float(self.params.get("scale", 1.0))
        pair = self.params.get("pair")
        self.pair = None if not pair else {"name": prefix + pair["name"], "buckets": int(pair["buckets"]),
                                           "mul_prev": int(pair["mul_prev"]), "mul_cur": int(pair["mul_cur"])}
        if self.pair and self.pair["buckets"] < 1:
            raise ValueError("pair_hash_embedding: at least one bucket")
        self.table = self.pair_table = self.err = None

    def tensors(self):
        out = [TensorDecl(self.name, (self.V, self.D))]
        if self.pair:
            out.append(TensorDecl(self.pair["name"], (self.pair["buckets"] + 1, self.D)))
        return out

    def load(self, get):
        self.table = self.rt.to_compute(get(self.name))
        if self.pair:
            self.pair_table = self.rt.to_compute(get(self.pair["name"]))
        self.err = torch.zeros(1, dtype=torch.int32, device=self.rt.device)

    def state_need(self):
        return {"prev": StateNeed((), torch.int32)} if self.pair else {}

    def forward_step(self, ctx, state, out=None):
        """The residual stream [n_tokens, hidden] float32 of a step (written into `out` if given)."""
        x = self.rt.empty(ctx.n_tokens, self.D, dtype=torch.float32) if out is None else out
        p = self.pair or {"buckets": 0, "mul_prev": 0, "mul_cur": 0}
        prev = state.get("prev") if self.pair else None
        ops.pair_embed(x, self.table, self.pair_table, ctx, prev, p["buckets"], p["mul_prev"], p["mul_cur"], self.scale,
                       self.err)
        if self.pair:
            ops.prev_token_update(prev, ctx)
        return x


@HEADS.register("lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied, name, scale (a constant the logits are multiplied by; default 1);
    `embedding` is handed in when tied."""
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.V = int(self._need("vocab_size"))
        self.D = int(self._need("hidden_size"))
        self.tied = bool(self._need("tied"))
        self.name = prefix + self.params.get("name", "lm_head.weight")
        self.embedding = self.params.get("embedding")
        self.scale = float(self.params.get("scale", 1.0) or 1.0)
        self.weight = None

    def tensors(self):
        return [] if self.tied else [TensorDecl(self.name, (self.V, self.D))]

    def load(self, get):
        self.weight = self.embedding.table if self.tied else self.rt.to_compute(get(self.name))

    def weight_bytes(self):
        return 0 if self.weight is None else self.weight.numel() * self.weight.element_size()

    def flops(self, start, count):
        return count * 2.0 * self.V * self.D

    def forward(self, xn):
        logits = self.rt.empty(xn.shape[0], self.V, dtype=torch.float32)
        matmul_nt(self.rt, logits, xn, self.weight)
        if self.scale != 1.0:
            ops.scale_rows(logits, self.scale)
        return logits
