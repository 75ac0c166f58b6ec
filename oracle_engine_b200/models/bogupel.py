"""The Bogupel decoder as data: BogupelConfig -> ModelSpec.

Every layer is x += mixer(norm1(x)); x += ffn(norm2(x)) (`pre_norm`; the feed-forward is optional) with Dynamic Tanh
norms (`dynamic_tanh`: tanh(alpha x) * w + b).  The mixer is either an attention with biases, normed queries and keys,
a partial rotation whose frequencies may be rescaled by wavelength, normed values that are turned by their own
position (the sum is turned back by the query's), a window and a learned sink per head (`rotated_value_attention`),
or a generalized delta rule with a decay and a removal rate per key channel (`general_delta`).  The feed-forward is a
mixture of clamped gated units chosen by sigmoid scores plus a learned bias (`moe_swiglu` with `choice_bias` and the
`clamped` activation).  The embedding adds a second table indexed by a hash of the token and the one before it
(`pair_hash_embedding`).  The schedule repeats the looped group of layers (weights shared, a cache and a state of its
own per pass); the first entry of every pass runs `pass_entry` before its layer, which adds the embedding's output
(from the second pass on) and the pass's own vector.  A Dynamic Tanh final norm, a head of its own, a constant on the
logits.
Tensor names: `embed`, `bigram`, `loop.step`, `head`, `final.norm[.b|.alpha]`, `l<i>.norm1|norm2[.b|.alpha]`,
`l<i>.mix.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.bogupel import BogupelConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NO_POSITION_LIMIT = 1 << 30        # the design has no largest position; the cache's size bounds a sequence


def build_spec(cfg: BogupelConfig, max_positions: int | None = None) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    max_pos = NO_POSITION_LIMIT if max_positions is None else min(max_positions, NO_POSITION_LIMIT)
    positions, layers = {}, []

    def norm(name):
        return PartSpec("dynamic_tanh", {"size": D, "name": name})

    def position(dims, base, sc):
        """The name of the rotary tables of a rotation; equal rotations share one."""
        if not dims:
            return None
        key = f"rot:{dims}:{base!r}:" + ("-" if sc is None else
                                         f"{sc['factor']!r}:{sc['low']!r}:{sc['high']!r}:{sc['original']!r}")
        if key not in positions:
            scaling = None if sc is None else {"factor": sc["factor"], "low_freq_factor": sc["low"],
                                               "high_freq_factor": sc["high"],
                                               "original_max_position_embeddings": sc["original"]}
            positions[key] = PartSpec("rotary", {"head_dim": dims, "theta": base, "scaling": scaling,
                                                 "max_positions": max_pos})
        return key

    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        if layer["type"] == "attention":
            rot = m["rot"]
            mixer = PartSpec("rotated_value_attention", {
                "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "key_dim": m["dim"],
                "value_dim": m["vdim"], "scale": m["scale"], "eps": eps, "window": (m["mask"] or {}).get("size", 0),
                "position": None if rot is None else position(rot["dims"], rot["base"], rot["scaling"]),
                # the values turn over all their dimensions with the keys' base and no rescaling
                "value_position": None if rot is None else position(m["vdim"], rot["base"], None)})
        else:
            mixer = PartSpec("general_delta", {"hidden_size": D, "num_heads": m["heads"], "head_dim": m["dim"],
                                               "eps": eps, "rank": m.get("rank")})
        mlp = layer["mlp"]
        ffn = None if mlp is None else PartSpec("moe_swiglu", {
            "hidden_size": D, "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
            "expert_size": mlp["expert"]["ff"], "router_weights": "sigmoid", "choice_bias": True,
            "activation": "clamped", "limit": mlp["expert"]["limit"]})
        layers.append(LayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
                                ffn_norm=None if mlp is None else norm("norm2"), block="pre_norm"))
    schedule = tuple(ScheduleEntry(i, before=None if t is None else ("loop", (("index", t),))) for i, t in cfg.passes())
    looped = cfg.loop is not None and cfg.loop[1] > cfg.loop[0]
    stream_parts = {"loop": PartSpec("pass_entry", {"hidden_size": D, "passes": cfg.loop[2], "name": "loop.step"})} \
        if looped else {}
    pair = None if cfg.bigram is None else {"name": "bigram", "buckets": cfg.bigram[0], "mul_prev": cfg.bigram[1],
                                            "mul_cur": cfg.bigram[2]}
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_positions=max_pos,
        embedding=PartSpec("pair_hash_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed",
                                                   "scale": cfg.embedding_scale, "pair": pair}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": False, "name": "head",
                                  "scale": cfg.logit_scale}),
        positions=positions, layers=tuple(layers), schedule=schedule, stream_parts=stream_parts,
        # a layer without a feed-forward reads none of these, and a model without a loop no pass vectors
        ignored_tensors=(".norm2", ".norm2.b", ".norm2.alpha") + (() if looped else ("loop.step",))
        + (() if pair else ("bigram",)))


register_architecture("Bogupel", BogupelConfig, build_spec)
