"""PusunexConfig: the sizes and constants of a Pusunex decoder, read from config.json.

config.json of this design:
    architecture    "Pusunex"
    vocab, width    sizes of the embedding table
    norm            eps (the epsilon of every root mean square), groups (the model's norm divides each of that many
                    equal consecutive parts of a vector by its own root mean square; default 1)
    token_side      optional {dim}: every layer adds an input made from `dim` columns of a second embedding table
    layers          a list; each entry has `type`, `mixer` (the sizes of that type) and `mlp` (an object or null)
      type "latent_attention"    mixer: heads, dim, vdim, kv_rank, scale; optional kv_from (the index of an earlier
                                 layer of this type whose latents it reads; it then has no down projection)
      type "latent_attention_2"  mixer: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {dims, base}
      type "gla"                 mixer: heads, dim, vdim, tau; optionally rank (else the file's tensors give it)
      mlp kind "dense"           ff
      mlp kind "moe"             expert {ff}, router {experts, top}, optional shared {ff}
Every key below the top level is checked and an unknown one is refused: it would be a mechanism this code does not
have.  Top-level keys beyond these are a file's own notes.  The design has no largest position, no stop tokens and
a head of its own.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .base import ConfigError, _Reader
from .fovirax import _obj, _only

LAYER_TYPES = ("latent_attention", "latent_attention_2", "gla")


def _latent(raw, what, second: bool, index: int, done: list) -> dict:
    raw = _obj(raw, what)
    r = _Reader(raw)
    if second:
        _only(raw, what, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"))
    else:
        _only(raw, what, ("heads", "dim", "vdim", "kv_rank", "scale", "kv_from"))
    m = {"heads": r.integer("heads"), "dim": r.integer("dim"), "vdim": r.integer("vdim"),
         "kv_rank": r.integer("kv_rank"), "scale": r.number("scale")}
    if second:
        m["rot_dim"] = r.integer("rot_dim", minimum=0)
        m["q_rank"] = r.integer("q_rank")
        rot = _obj(raw.get("rot"), what + ".rot")
        _only(rot, what + ".rot", ("dims", "base"))
        rr = _Reader(rot)
        m["rot"] = {"dims": rr.integer("dims", minimum=0), "base": rr.number("base")}
        if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
            raise ConfigError(f"config.json: `{what}.rot.dims` must be even and at most rot_dim {m['rot_dim']}")
    else:
        src = r.integer("kv_from", default=None, required=False, minimum=0)
        if src is not None:
            if src >= index or done[src]["type"] != "latent_attention" or done[src]["mixer"].get("kv_from") is not None:
                raise ConfigError(f"config.json: `{what}.kv_from` must name an earlier latent_attention layer with "
                                  f"a down projection of its own, got {src}")
            if done[src]["mixer"]["kv_rank"] != m["kv_rank"]:
                raise ConfigError(f"config.json: `{what}.kv_from`: layer {src} has kv_rank "
                                  f"{done[src]['mixer']['kv_rank']}, this layer {m['kv_rank']}")
            m["kv_from"] = src
    return m


def _gla(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("heads", "dim", "vdim", "tau", "rank"))
    r = _Reader(raw)
    m = {"heads": r.integer("heads"), "dim": r.integer("dim"), "vdim": r.integer("vdim"), "tau": r.number("tau")}
    rank = r.integer("rank", default=None, required=False)
    if rank is not None:
        m["rank"] = rank
    return m


def _mlp(raw, what):
    if raw is None:
        return None
    raw = _obj(raw, what)
    kind = raw.get("kind")
    if kind == "dense":
        _only(raw, what, ("kind", "ff"))
        return {"kind": "dense", "ff": _Reader(raw).integer("ff")}
    if kind != "moe":
        raise ConfigError(f"config.json: `{what}.kind` must be \"dense\" or \"moe\", got {kind!r}")
    _only(raw, what, ("kind", "expert", "router", "shared"))
    expert, router = _obj(raw.get("expert"), what + ".expert"), _obj(raw.get("router"), what + ".router")
    _only(expert, what + ".expert", ("ff",))
    _only(router, what + ".router", ("experts", "top"))
    out = {"kind": "moe", "expert": {"ff": _Reader(expert).integer("ff")},
           "router": {"experts": _Reader(router).integer("experts"), "top": _Reader(router).integer("top")},
           "shared": None}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"config.json: `{what}.router`: top exceeds experts")
    if raw.get("shared") is not None:
        shared = _obj(raw["shared"], what + ".shared")
        _only(shared, what + ".shared", ("ff",))
        out["shared"] = {"ff": _Reader(shared).integer("ff")}
    return out


@dataclass(frozen=True)
class PusunexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    side_dim: int              # 0: no token side input
    layers: tuple              # of {"type", "mixer", "mlp"} with checked contents

    @staticmethod
    def from_dict(raw: dict) -> "PusunexConfig":
        r = _Reader(raw)
        norm = _obj(raw.get("norm"), "norm")
        _only(norm, "norm", ("eps", "groups"))
        groups = _Reader(norm).integer("groups", default=1, required=False)
        width = r.integer("width")
        if width % groups:
            raise ConfigError(f"config.json: `norm.groups` {groups} does not divide the width {width}")
        side_dim = 0
        if raw.get("token_side") is not None:
            side = _obj(raw["token_side"], "token_side")
            _only(side, "token_side", ("dim",))
            side_dim = _Reader(side).integer("dim")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: `layers` must be a list with at least one layer")
        out = []
        for i, layer in enumerate(layers):
            what = f"layers[{i}]"
            layer = _obj(layer, what)
            _only(layer, what, ("type", "mixer", "mlp"))
            kind = layer.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: `{what}.type` must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
            if kind == "gla":
                mixer = _gla(layer.get("mixer"), what + ".mixer")
            else:
                mixer = _latent(layer.get("mixer"), what + ".mixer", kind == "latent_attention_2", i, out)
            out.append({"type": kind, "mixer": mixer, "mlp": _mlp(layer.get("mlp"), what + ".mlp")})
        name = raw.get("architecture") or (raw.get("architectures") or ["Pusunex"])[0]
        return PusunexConfig(architecture=name, vocab=r.integer("vocab"), width=width,
                             norm_eps=_Reader(norm).number("eps"), norm_groups=groups, side_dim=side_dim,
                             layers=tuple(out))

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": copy.deepcopy(list(self.layers))}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d
