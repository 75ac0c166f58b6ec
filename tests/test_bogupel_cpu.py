"""The Bogupel design without a GPU: its config.json reader, its model description, random model folders and the
plain model's own mechanisms, each against a closed form."""
import copy
import json
import math

import pytest
import torch

import bogupel_models as bm
import plain_bogupel as pb


def test_config_round_trip_and_refusals():
    from oracle_engine_b200.config.base import ConfigError
    from oracle_engine_b200.config.bogupel import BogupelConfig
    for raw, _ in list(bm.ALL.values()) + [(bm.REAL, 0)]:
        cfg = BogupelConfig.from_dict(raw)
        assert BogupelConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
        assert cfg.vocab == raw["vocab"] and cfg.width == raw["width"] and cfg.norm_eps == raw["norm"]["eps"]
        assert cfg.layer_order() == [i for i, _, _ in pb.layer_order(raw)]
        assert [t for _, t in cfg.passes() if t is not None] == [t for _, t, first in pb.layer_order(raw) if first]
    noted = dict(copy.deepcopy(bm.B1), seed=3, name="a note")          # a file's own notes at the top level are not read
    assert BogupelConfig.from_dict(noted) == BogupelConfig.from_dict(bm.B1)
    nulls = copy.deepcopy(bm.B2)                                       # absent and null mean the same
    nulls["loop"] = None
    nulls["embedding"]["bigram"] = None
    nulls["layers"][3]["mixer"].update(mask=None, rot=None)
    nulls["layers"][1]["mixer"]["rot"]["scaling"] = None
    assert BogupelConfig.from_dict(nulls) == BogupelConfig.from_dict(bm.B2)
    bare = copy.deepcopy(bm.B2)                                        # defaults: no scale, no second table, no constant
    bare.pop("embedding")
    cfg = BogupelConfig.from_dict(bare)
    assert cfg.embedding_scale == 1.0 and cfg.bigram is None and cfg.logit_scale == 1.0 and cfg.loop is None

    def refused(match, change):
        bad = copy.deepcopy(bm.B1)
        change(bad)
        with pytest.raises(ConfigError, match=match):
            BogupelConfig.from_dict(bad)

    refused("type", lambda c: c["layers"][1].update(type="conv"))
    refused("softcap", lambda c: c["layers"][0]["mixer"].update(softcap=30.0))     # a mechanism this design lacks
    refused("kv_heads", lambda c: c["layers"][0]["mixer"].update(kv_heads=3))
    refused("dims", lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34))      # more than the head has
    refused("dims", lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7))
    refused("vdim", lambda c: c["layers"][0]["mixer"].update(vdim=15))             # values turn in pairs
    refused("kind", lambda c: c["layers"][1]["mlp"].update(kind="dense"))
    refused("top", lambda c: c["layers"][0]["mlp"]["router"].update(top=7))
    refused("limit", lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"))
    refused("eps", lambda c: c["norm"].pop("eps"))
    refused("loop", lambda c: c["loop"].update(stop=9))
    refused("buckets", lambda c: c["embedding"]["bigram"].pop("buckets"))
    refused("layers", lambda c: c.update(layers=[]))


def test_spec_declares_the_designs_tensors_caches_and_state(tmp_path):
    from oracle_engine_b200.config.base import load_config
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.parts.model import DecoderModel
    folder = bm.write(tmp_path / "m", bm.B1, 1)
    cfg, arch = load_config(folder)
    assert arch.name == "Bogupel"
    spec = arch.build_spec(cfg, None)
    model = DecoderModel(spec, Runtime(torch.float32, torch.device("cpu")))
    names = {d.name: tuple(d.shape) for d in model.tensors()}
    stored = pb.read_safetensors(tmp_path / "m" / "model.safetensors")
    assert set(names) == set(stored)
    assert all(tuple(stored[n].shape) == s for n, s in names.items())
    assert names["loop.step"] == (3, 96) and names["bigram"] == (212, 96) and names["l0.norm1.alpha"] == ()
    assert "l2.norm2" not in names and names["l1.mix.w2"] == (72, 5) and names["l0.mlp.correction"] == (6,)
    # the schedule: layer 0, then layers 1 and 2 three times (each run with a cache and a state of its own)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.before for e in spec.schedule if e.before] == [("loop", (("index", t),)) for t in range(3)]
    cache, state = model.cache_needs(), model.state_needs()
    assert len(cache) == len(state) == 8
    assert cache[0].kind == "window" and cache[0].window == 40 and dict(cache[0].tensors) == {"k": (2, 32), "v": (2, 16)}
    assert cache[2].kind == "full" and cache[1] is None and cache[3] is None
    assert state[1]["S"].shape == (3, 24, 24) and state[1]["S"].dtype == torch.float32 and not state[0]
    assert model.embedding_state_needs()["prev"].dtype == torch.int32
    # equal rotations share tables: the values of layer 3 (24 dimensions, base 77) have a table of their own
    assert len(spec.positions) == 6
    # the whole pass is one run of graph-safe stages
    assert model.stages() == [(True, 0, 10)]


def test_a_size_that_only_the_file_gives(tmp_path):
    """The rank of the decay's projection is read from the tensors when config.json does not give it."""
    from oracle_engine_b200.config.base import load_config
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.parts.model import DecoderModel
    folder = bm.write(tmp_path / "m", bm.LONG_MEMORY, 2)
    raw = json.loads((tmp_path / "m" / "config.json").read_text())
    del raw["layers"][0]["mixer"]["rank"]
    (tmp_path / "m" / "config.json").write_text(json.dumps(raw))
    cfg, arch = load_config(folder)
    model = DecoderModel(arch.build_spec(cfg, None), Runtime(torch.float32, torch.device("cpu")))
    names = {d.name: tuple(d.shape) for d in model.tensors()}
    assert names["l0.mix.w1"] == (-1, 48) and names["l0.mix.w2"] == (48, -1)


def test_plain_embedding_and_norm():
    w = {"embed": torch.arange(12, dtype=torch.float64).reshape(6, 2), "bigram": 100.0 * torch.arange(8, dtype=torch.float64).reshape(4, 2)}
    cfg = {"embedding": {"scale": 2.0, "bigram": {"buckets": 3, "mul_prev": 2, "mul_cur": 1}}}
    x = pb.embed(torch.tensor([5, 1, 4]), w, cfg)
    # first token: the last row; then (5 * 2 + 1) mod 3 = 2 and (1 * 2 + 4) mod 3 = 0
    assert x.tolist() == [[20.0 + 600.0, 22.0 + 700.0], [4.0 + 400.0, 6.0 + 500.0], [16.0, 18.0 + 100.0]]
    y = pb.dyt(torch.tensor([0.0, 1e9, -1e9]), 0.5, torch.tensor(3.0), torch.tensor(1.0))
    assert y.tolist() == [1.0, 4.0, -2.0]


def test_plain_frequencies_match_the_package():
    from oracle_engine_b200.parts.positions import rotary_inv_freq
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    mine = pb.frequencies(16, 10000.0, sc)
    theirs = rotary_inv_freq(16, 10000.0, {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                            "original_max_position_embeddings": 64})
    assert torch.allclose(mine, theirs, rtol=1e-12)
    plain = pb.frequencies(16, 10000.0)
    kept, divided = (mine == plain), torch.isclose(mine, plain / 8.0)
    assert kept.any() and divided.any() and (~kept & ~divided).any()          # all three bands


def test_plain_attention_sink_window_and_value_turn():
    """Equal scores: the weights are 1 / (n + e^sink) over the n keys the window leaves; with values that are the same
    unit vector at every position, turning by the key's position and back by the query's leaves the vector turned by
    the distance, so a window of one gives the vector back untouched."""
    T, d = 6, 4
    w = {"q": torch.zeros(d, 3, dtype=torch.float64), "k": torch.zeros(d, 3, dtype=torch.float64), "v": torch.zeros(d, 3, dtype=torch.float64),
         "q.b": torch.ones(d, dtype=torch.float64), "k.b": torch.ones(d, dtype=torch.float64),
         "v.b": torch.tensor([1.0, 0.0, 0.0, 0.0], dtype=torch.float64), "q.norm": torch.ones(d, dtype=torch.float64),
         "k.norm": torch.ones(d, dtype=torch.float64), "sink": torch.tensor([math.log(2.0)], dtype=torch.float64),
         "o": torch.eye(d, dtype=torch.float64)}
    h = torch.randn(T, 3, dtype=torch.float64)
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 0.5, "mask": {"size": 1}, "rot": {"dims": 0, "base": 10.0}}
    o = pb.attention(h, w, "", m, 0.0)
    # one key (itself), score s: weight e^s / (e^s + 2), value the normed vector (2, 0, 0, 0) turned by distance 0
    s = 0.5 * d
    assert torch.allclose(o, torch.tensor([2.0, 0, 0, 0], dtype=torch.float64) * math.exp(s) / (math.exp(s) + 2.0))
    m["mask"] = {"size": 3}
    o = pb.attention(h, w, "", m, 0.0)
    f = pb.frequencies(d, 10.0)
    for t in range(T):
        n = min(t + 1, 3)
        want = sum(pb.turn_halves(torch.tensor([[[2.0, 0, 0, 0]]], dtype=torch.float64), torch.tensor([j - t]), f)[0, 0]
                   for j in range(t - n + 1, t + 1)) * math.exp(s) / (n * math.exp(s) + 2.0)
        assert torch.allclose(o[t], want)


def test_plain_delta_rule_closed_forms():
    """With the removal off (a = 0) and a constant decay the state is a geometric sum; with a = 1, no decay and the
    same key twice, the second token replaces what the first one stored along that key."""
    d = 2
    big = 50.0
    base = {"r": torch.eye(d, 3, dtype=torch.float64), "k": torch.zeros(d, 3, dtype=torch.float64), "v": torch.zeros(d, 3, dtype=torch.float64),
            "g": torch.zeros(d, 3, dtype=torch.float64), "a": torch.zeros(d, 3, dtype=torch.float64), "w1": torch.zeros(1, 3, dtype=torch.float64),
            "w2": torch.zeros(d, 1, dtype=torch.float64), "norm": torch.ones(d, dtype=torch.float64), "o": torch.eye(d, dtype=torch.float64)}
    base["k"][0, 0] = 1.0          # k = (h_0, 0)
    base["v"][:, 1] = 1.0          # v = (h_1, h_1)
    m = {"heads": 1, "dim": d}
    h = torch.tensor([[1.0, 3.0, 0.0], [1.0, 5.0, 0.0]], dtype=torch.float64)
    # a = 1 (bias far above zero), decay 1 (w0 far below zero): S after token 2 holds the second value only
    w = dict(base, **{"a.b": torch.full((d,), big, dtype=torch.float64), "w0": torch.full((d,), -big, dtype=torch.float64)})
    w["r"] = torch.zeros(d, 3, dtype=torch.float64)
    w["r"][0, 0] = 1.0             # r = (h_0, 0) = k: the read-out is what is stored along the key
    y = pb.general_delta(h, w, "", m, 0.0)
    # o_1 = (3, 3), o_2 = (5, 5) up to 1e-6 in the unit key; normed per head and gated by sigmoid(0) = 1/2
    assert torch.allclose(y, torch.full((2, 2), 0.5, dtype=torch.float64), atol=1e-5)
    # a = 0, decay exp(-e^(-1/2) / 2) each step (w0 = 0): o_2 = decay * 3 + 5 along both columns
    w = dict(base, **{"a.b": torch.full((d,), -big, dtype=torch.float64), "w0": torch.zeros(d, dtype=torch.float64)})
    w["r"] = torch.zeros(d, 3, dtype=torch.float64)
    w["r"][0, 0] = 1.0
    w["norm"] = torch.ones(d, dtype=torch.float64)
    dec = math.exp(-math.exp(-0.5) * 0.5)
    H = pb.general_delta(h, dict(w, o=torch.eye(d, dtype=torch.float64)), "", m, 0.0)
    assert torch.allclose(H, torch.full((2, 2), 0.5, dtype=torch.float64))          # the norm hides the size ...
    raw = []
    orig = pb.unit_rms
    pb.unit_rms = lambda x, eps: (raw.append(x.clone()), orig(x, eps))[1]
    try:
        pb.general_delta(h, w, "", m, 0.0)
    finally:
        pb.unit_rms = orig
    assert torch.allclose(raw[0][1, 0], torch.full((2,), dec * 3.0 + 5.0, dtype=torch.float64))   # ... the read-out shows it


def test_plain_experts_with_hand_set_scores():
    """The bias decides the choice, the weights are the sigmoids without it; the unit clamps the gate from above only."""
    D = 2
    w = {"router": torch.tensor([[1.0, 0.0], [0.0, 0.0], [-1.0, 0.0]], dtype=torch.float64),
         "correction": torch.tensor([0.0, 0.0, 5.0], dtype=torch.float64)}
    for e in range(3):
        w[f"e{e}.gate"] = torch.tensor([[0.0, 1.0]], dtype=torch.float64) * (e + 1)
        w[f"e{e}.up"] = torch.tensor([[0.0, 10.0]], dtype=torch.float64)
        w[f"e{e}.down"] = torch.ones(D, 1, dtype=torch.float64)
    mlp = {"router": {"experts": 3, "top": 1}, "expert": {"limit": 2.0}}
    h = torch.tensor([[3.0, -4.0], [3.0, 1.0]], dtype=torch.float64)
    y = pb.moe(h, w, "", mlp)
    s2 = 1.0 / (1.0 + math.exp(3.0))                      # expert 2 is chosen by its bias, weighed by its small sigmoid
    g = -12.0                                             # gate 3 * -4, not clamped from below; up 10 * -4 -> -2
    assert torch.allclose(y[0], torch.full((D,), s2 * g / (1.0 + math.exp(-1.702 * g)) * (-2.0 + 1.0), dtype=torch.float64))
    g = 2.0                                               # gate 3 clamped to 2; up 10 clamped to 2
    assert torch.allclose(y[1], torch.full((D,), s2 * g / (1.0 + math.exp(-1.702 * g)) * 3.0, dtype=torch.float64))


def test_plain_loop_adds_the_embedding_and_the_pass_vectors(tmp_path):
    """With every layer's output projections zeroed the stream is the embedding plus what the passes add."""
    folder = bm.write(tmp_path / "m", bm.B1, 7)
    cfg, w = pb.load(folder)
    for n in list(w):
        if n.endswith(".mix.o") or n.endswith(".down"):
            w[n] = torch.zeros_like(w[n])
    toks = [5, 9, 200, 31]
    _, kept = pb.forward(cfg, w, toks, keep_layers=True)
    x0 = pb.embed(torch.tensor(toks), w, cfg)
    s = w["loop.step"]
    assert torch.allclose(kept[0], x0)
    assert torch.allclose(kept[2], x0 + s[0]) and torch.allclose(kept[4], 2 * x0 + s[0] + s[1])
    assert torch.allclose(kept[-1], 3 * x0 + s.sum(0))
