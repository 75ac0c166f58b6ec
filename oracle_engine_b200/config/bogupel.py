"""BogupelConfig: the sizes and constants of a Bogupel decoder, read from config.json.

config.json of this design:
    architecture    "Bogupel"
    vocab, width    sizes of the embedding table
    embedding       scale (default 1); optional bigram {buckets, mul_prev, mul_cur}: a second table indexed by a hash of
                    the token and the one before it
    norm.eps        the epsilon of every root mean square (the layers' own norms are Dynamic Tanh and use none)
    logit_scale     a constant on the logits (default 1)
    loop            optional {start, stop, times}: layers start .. stop - 1 run `times` times as a group
    layers          a list; each entry has `type` ("attention" or "general_delta"), `mixer` and `mlp` (an object or null)
      mixer of "attention"       heads, kv_heads, dim, vdim, scale; optional mask {size}, rot {dims, base, optional
                                 scaling {factor, low, high, original}}
      mixer of "general_delta"   heads, dim; optional rank (of the decay's two-matrix projection: the weight file
                                 gives it, the key is for writing folders of random weights)
      mlp           kind "moe", expert {ff, limit}, router {experts, top}
Every key below the top level is checked and an unknown one is refused: it would be a mechanism this code does not
have.  Top-level keys beyond these are a file's own notes.  The design has no largest position, no stop tokens and
a head of its own.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .base import ConfigError, _Reader
from .fovirax import _obj, _only


def _rotation(raw, what, dim):
    """None, or {"dims", "base", "scaling": None or {"factor", "low", "high", "original"}}; dims may be 0 (the keys
    are not turned; the base still turns the values)."""
    if raw is None:
        return None
    raw = _obj(raw, what)
    _only(raw, what, ("dims", "base", "scaling"))
    r = _Reader(raw)
    out = {"dims": r.integer("dims", minimum=0), "base": r.number("base"), "scaling": None}
    if out["dims"] % 2 or out["dims"] > dim:
        raise ConfigError(f"config.json: `{what}.dims` must be even and at most the head's dim {dim}")
    if raw.get("scaling") is not None:
        sc = _obj(raw["scaling"], what + ".scaling")
        _only(sc, what + ".scaling", ("factor", "low", "high", "original"))
        rs = _Reader(sc)
        out["scaling"] = {"factor": rs.number("factor"), "low": rs.number("low"), "high": rs.number("high"),
                          "original": rs.number("original")}
        if out["scaling"]["high"] == out["scaling"]["low"]:
            raise ConfigError(f"config.json: `{what}.scaling`: high and low must differ")
    return out


def _attention(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"))
    r = _Reader(raw)
    m = {"heads": r.integer("heads"), "kv_heads": r.integer("kv_heads"), "dim": r.integer("dim"),
         "vdim": r.integer("vdim"), "scale": r.number("scale"), "mask": None}
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: `{what}`: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    if raw.get("mask") is not None:
        mask = _obj(raw["mask"], what + ".mask")
        _only(mask, what + ".mask", ("size",))
        m["mask"] = {"size": _Reader(mask).integer("size")}
    m["rot"] = _rotation(raw.get("rot"), what + ".rot", m["dim"])
    if m["rot"] is not None and m["vdim"] % 2:
        raise ConfigError(f"config.json: `{what}.vdim` must be even: the values are turned in pairs")
    return m


def _general_delta(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("heads", "dim", "rank"))
    r = _Reader(raw)
    m = {"heads": r.integer("heads"), "dim": r.integer("dim")}
    if raw.get("rank") is not None:          # the file's tensors give it; the key lets folders of random weights be written
        m["rank"] = r.integer("rank")
    return m


def _moe(raw, what) -> dict:
    raw = _obj(raw, what)
    _only(raw, what, ("kind", "expert", "router"))
    if raw.get("kind") != "moe":
        raise ConfigError(f"config.json: `{what}.kind` must be \"moe\", got {raw.get('kind')!r}")
    expert, router = _obj(raw.get("expert"), what + ".expert"), _obj(raw.get("router"), what + ".router")
    _only(expert, what + ".expert", ("ff", "limit"))
    _only(router, what + ".router", ("experts", "top"))
    out = {"kind": "moe", "expert": {"ff": _Reader(expert).integer("ff"), "limit": _Reader(expert).number("limit")},
           "router": {"experts": _Reader(router).integer("experts"), "top": _Reader(router).integer("top")}}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"config.json: `{what}.router`: top exceeds experts")
    return out


_MIXERS = {"attention": _attention, "general_delta": _general_delta}


@dataclass(frozen=True)
class BogupelConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    bigram: tuple | None       # (buckets, mul_prev, mul_cur)
    logit_scale: float
    loop: tuple | None         # (start, stop, times)
    layers: tuple              # of {"type", "mixer", "mlp"} with checked contents

    @staticmethod
    def from_dict(raw: dict) -> "BogupelConfig":
        r = _Reader(raw)
        norm = _obj(raw.get("norm"), "norm")
        _only(norm, "norm", ("eps",))
        emb = _obj(raw.get("embedding") or {}, "embedding")
        _only(emb, "embedding", ("scale", "bigram"))
        bigram = None
        if emb.get("bigram") is not None:
            bg = _obj(emb["bigram"], "embedding.bigram")
            _only(bg, "embedding.bigram", ("buckets", "mul_prev", "mul_cur"))
            rb = _Reader(bg)
            bigram = (rb.integer("buckets"), rb.integer("mul_prev", minimum=0), rb.integer("mul_cur", minimum=0))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: `layers` must be a list with at least one layer")
        out = []
        for i, layer in enumerate(layers):
            what = f"layers[{i}]"
            layer = _obj(layer, what)
            _only(layer, what, ("type", "mixer", "mlp"))
            kind = layer.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: `{what}.type` must be one of {', '.join(sorted(_MIXERS))}, got {kind!r}")
            mlp = None if layer.get("mlp") is None else _moe(layer["mlp"], what + ".mlp")
            out.append({"type": kind, "mixer": _MIXERS[kind](layer.get("mixer"), what + ".mixer"), "mlp": mlp})
        loop = None
        if raw.get("loop") is not None:
            lp = _obj(raw["loop"], "loop")
            _only(lp, "loop", ("start", "stop", "times"))
            rl = _Reader(lp)
            loop = (rl.integer("start", minimum=0), rl.integer("stop", minimum=0), rl.integer("times", minimum=1))
            if not loop[0] <= loop[1] <= len(out):
                raise ConfigError(f"config.json: `loop` must name layers inside 0 .. {len(out)}")
        name = raw.get("architecture") or (raw.get("architectures") or ["Bogupel"])[0]
        return BogupelConfig(architecture=name, vocab=r.integer("vocab"), width=r.integer("width"),
                             norm_eps=_Reader(norm).number("eps"),
                             embedding_scale=_Reader(emb).number("scale", default=1.0, required=False, positive=False),
                             bigram=bigram,
                             logit_scale=r.number("logit_scale", default=1.0, required=False, positive=False),
                             loop=loop, layers=tuple(out))

    def passes(self) -> list:
        """[(layer, pass index or None)] in the order the layers run; the pass index is given at the first layer of
        every pass of the looped group."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop
        out = [(i, None) for i in range(a)]
        for t in range(times):
            out += [(i, t if i == a else None) for i in range(a, b)]
        return out + [(i, None) for i in range(b, n)]

    def layer_order(self) -> list:
        return [i for i, _ in self.passes()]

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        emb = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": emb,
             "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d
