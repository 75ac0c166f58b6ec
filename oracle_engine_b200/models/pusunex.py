"""The Pusunex decoder as data: PusunexConfig -> ModelSpec.

Every layer norms what a sublayer reads and what it returns (`sandwich`): x += n1b(mixer(n1(x))); x += n2b(ffn(n2(x))),
the feed-forward being optional; the model's norm is an RMS norm in groups (`rms_norm` with `groups`).  After the
feed-forward a layer adds an input made from the token itself (`TokenSide`: its own columns of a second embedding
table, gated by the stream) and what goes on to the next layer is a weighted sum of the stream after every layer so
far and of the embedding (`DepthAverage`).  Mixers: attention over a cached latent (`latent_attention`: plain, with
an output gate, optionally reading an earlier layer's latents through the schedule's `cache_from`; or with a query
latent and a turned key part shared by the heads) and gated linear attention (`gated_linear_attention`).
Feed-forwards: `poly_norm_mlp` and a mixture of experts whose weights are sigmoids applied to the experts' input
(`moe_swiglu` with its variants).  A final norm and a head of its own.
Tensor names: `embed`, `side.embed`, `head`, `final.norm`, `l<i>.norm1|norm1b|norm2|norm2b|dwa`, `l<i>.mix.*`,
`l<i>.mlp.*`, `l<i>.side.gate|proj|norm`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.pusunex import PusunexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NO_POSITION_LIMIT = 1 << 30        # the design has no largest position; the cache's size bounds a sequence


def build_spec(cfg: PusunexConfig, max_positions: int | None = None) -> ModelSpec:
    D, eps, L = cfg.width, cfg.norm_eps, len(cfg.layers)
    max_pos = NO_POSITION_LIMIT if max_positions is None else min(max_positions, NO_POSITION_LIMIT)
    positions, layers, schedule = {}, [], []

    def norm_params(name):
        return {"size": D, "eps": eps, "name": name, "groups": cfg.norm_groups}

    def position(rot):
        if not rot or not rot["dims"]:
            return None
        key = f"pairs:{rot['dims']}:{rot['base']!r}"
        positions.setdefault(key, PartSpec("rotary_pairs", {"dims": rot["dims"], "base": rot["base"]}))
        return key

    for i, layer in enumerate(cfg.layers):
        m, kind = layer["mixer"], layer["type"]
        cache_from = None
        if kind == "gla":
            mixer = PartSpec("gated_linear_attention", {
                "hidden_size": D, "num_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"], "tau": m["tau"],
                "eps": eps, "decay_rank": m.get("rank"), "tensor_names": {k: "mix." + v for k, v in {
                    "q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2",
                    "a2_bias": "a2.b"}.items()}})
        else:
            second = kind == "latent_attention_2"
            cache_from = m.get("kv_from")
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "num_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps, "rot_dim": m.get("rot_dim", 0),
                "position": position(m.get("rot")) if second else None, "q_rank": m.get("q_rank", 0),
                "gate": not second, "reads_cache": cache_from is not None,
                "tensor_names": {k: "mix." + v for k, v in {
                    "q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                    "uk": "uk", "uv": "uv", "g": "g", "o": "o"}.items()}})
        mlp = layer["mlp"]
        if mlp is None:
            ffn = None
        elif mlp["kind"] == "dense":
            ffn = PartSpec("poly_norm_mlp", {"hidden_size": D, "intermediate_size": mlp["ff"], "eps": eps})
        else:
            ffn = PartSpec("moe_swiglu", {
                "hidden_size": D, "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_size": mlp["expert"]["ff"], "shared_size": (mlp["shared"] or {}).get("ff", 0),
                "router_weights": "sigmoid", "weight_on": "input", "shared_gate": False})
        side = None
        if cfg.side_dim:
            side = {"hidden_size": D, "vocab_size": cfg.vocab, "dim": cfg.side_dim, "offset": i * cfg.side_dim,
                    "table_width": L * cfg.side_dim, "eps": eps,
                    "names": {"table": "side.embed", "gate": "side.gate", "proj": "side.proj", "norm": "side.norm"}}
        layers.append(LayerSpec(
            prefix=f"l{i}.", mixer=mixer, feed_forward=ffn, mixer_norm=PartSpec("rms_norm", norm_params("norm1")),
            ffn_norm=None if ffn is None else PartSpec("rms_norm", norm_params("norm2")), block="sandwich",
            block_params={"hidden_size": D,
                          "mixer_out_norm": {"kind": "rms_norm", "params": norm_params("norm1b")},
                          "ffn_out_norm": {"kind": "rms_norm", "params": norm_params("norm2b")},
                          "token_side": side,
                          "depth_average": {"hidden_size": D, "index": i, "layers": L, "name": "dwa"}}))
        schedule.append(ScheduleEntry(i, cache_from=cache_from))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_positions=max_pos,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed"}),
        final_norm=PartSpec("rms_norm", norm_params("final.norm")),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": False, "name": "head"}),
        positions=positions, layers=tuple(layers), schedule=tuple(schedule),
        # a layer without a feed-forward reads neither of these, whether its file holds them or not
        ignored_tensors=(".norm2", ".norm2b"))


register_architecture("Pusunex", PusunexConfig, build_spec)
