"""The Pusunex design without a GPU: its config.json reader, its model description, random model folders and the
plain model's own mechanisms, each against a closed form."""
import copy
import json

import pytest
import torch

import plain_pusunex as pp
import pusunex_models as pm


def test_config_round_trip_and_refusals():
    from oracle_engine_b200.config.base import ConfigError
    from oracle_engine_b200.config.pusunex import PusunexConfig
    for raw, _ in list(pm.ALL.values()) + [(pm.REAL, 0)]:
        cfg = PusunexConfig.from_dict(raw)
        assert PusunexConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
        assert cfg.vocab == raw["vocab"] and cfg.width == raw["width"] and cfg.norm_eps == raw["norm"]["eps"]
        assert cfg.norm_groups == raw["norm"]["groups"] and cfg.side_dim == (raw.get("token_side") or {"dim": 0})["dim"]
    noted = dict(copy.deepcopy(pm.P1), seed=3, name="a note")          # a file's own notes at the top level are not read
    assert PusunexConfig.from_dict(noted) == PusunexConfig.from_dict(pm.P1)
    nulls = copy.deepcopy(pm.P2)                                       # absent and null mean the same
    nulls["token_side"] = None
    nulls["layers"][2]["mixer"]["kv_from"] = None
    nulls["layers"][2]["mlp"]["shared"] = None
    assert PusunexConfig.from_dict(nulls) == PusunexConfig.from_dict(pm.P2)

    def refused(match, change):
        bad = copy.deepcopy(pm.P1)
        change(bad)
        with pytest.raises(ConfigError, match=match):
            PusunexConfig.from_dict(bad)

    refused("type", lambda c: c["layers"][1].update(type="conv"))
    refused("window", lambda c: c["layers"][0]["mixer"].update(window=64))         # a mechanism this design lacks
    refused("kv_from", lambda c: c["layers"][3]["mixer"].update(kv_from=2))        # not a plain latent attention
    refused("kv_from", lambda c: c["layers"][0]["mixer"].update(kv_from=0))        # not an earlier layer
    refused("kv_rank", lambda c: c["layers"][3]["mixer"].update(kv_rank=24))       # the latents would not fit
    refused("kind", lambda c: c["layers"][1].update(mlp={"kind": "routed", "ff": 8}))
    refused("top", lambda c: c["layers"][0]["mlp"]["router"].update(top=7))
    refused("eps", lambda c: c["norm"].pop("eps"))
    refused("groups", lambda c: c["norm"].update(groups=5))                        # 96 is no multiple of 5
    refused("dims", lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10))      # more than rot_dim
    refused("layers", lambda c: c.update(layers=[]))


def test_spec_declares_the_designs_tensors_caches_and_state(tmp_path):
    from oracle_engine_b200.config.base import load_config
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.parts.model import DecoderModel
    folder = pm.write(tmp_path / "m", pm.P1, 1)
    cfg, arch = load_config(folder)
    assert arch.name == "Pusunex"
    spec = arch.build_spec(cfg, None)
    model = DecoderModel(spec, Runtime(torch.float32, torch.device("cpu")))
    names = {d.name: tuple(d.shape) for d in model.tensors()}
    stored = pp.read_safetensors(tmp_path / "m" / "model.safetensors")
    assert set(names) == set(stored)
    assert all(tuple(stored[n].shape) == s for n, s in names.items())
    assert names["side.embed"] == (300, 4 * 8) and names["l0.side.gate"] == (8, 96) and names["l0.side.proj"] == (96, 8)
    assert names["l0.mix.dkv"] == (40, 96) and names["l2.mix.dkv"] == (24 + 8, 96) and names["l2.mix.uq"] == (2 * 24, 36)
    assert names["l0.mix.uk"] == (4 * 24, 40) and names["l0.mix.uv"] == (4 * 16, 40) and names["l0.mix.g"] == (64, 96)
    assert names["l1.mix.a1"] == (12, 96) and names["l1.mix.a2"] == (48, 12) and names["l1.mix.norm"] == (24,)
    assert names["l1.mlp.act"] == (4,) and names["l0.dwa"] == (2,) and names["l3.dwa"] == (5,)
    # the layer that reads layer 0's latents has neither a down projection nor a cache of its own; the second kind
    # of latent attention has no gate, the layer without a feed-forward no norms around one
    assert "l3.mix.dkv" not in names and "l3.mix.dkv.norm" not in names and "l2.mix.g" not in names
    assert "l2.norm2" not in names and "l2.mlp.up" not in names
    needs = model.cache_needs()
    assert needs[0].tensors == (("latent", (40,)),) and needs[2].tensors == (("latent", (24 + 8,)),)
    assert needs[1] is None and needs[3] is None
    assert spec.schedule[3].cache_from == 0 and spec.schedule[0].cache_from is None
    state = model.state_needs()
    assert state[1]["S"].shape == (3, 16, 24) and state[1]["S"].dtype == torch.float32
    assert not state[0] and not state[2] and not state[3]
    assert model.stages() == [(True, 0, len(cfg.layers) + 2)]  # every part can be captured in a CUDA graph


def test_a_size_only_the_file_gives(tmp_path):
    """Without `rank` in config.json the decay projection's rank is the shape of its tensors."""
    from oracle_engine_b200.config.base import load_config
    from oracle_engine_b200.engine.runtime import Runtime
    from oracle_engine_b200.parts.model import DecoderModel
    from oracle_engine_b200.weights.loader import check_tensors
    folder = pm.write(tmp_path / "m", pm.P1, 1)
    raw = json.loads((tmp_path / "m" / "config.json").read_text())
    del raw["layers"][1]["mixer"]["rank"]
    (tmp_path / "m" / "config.json").write_text(json.dumps(raw))
    cfg, arch = load_config(folder)
    model = DecoderModel(arch.build_spec(cfg, None), Runtime(torch.float32, torch.device("cpu")))
    decl = {d.name: tuple(d.shape) for d in model.tensors()}
    assert decl["l1.mix.a1"] == (-1, 96) and decl["l1.mix.a2"] == (3 * 16, -1)
    stored = pp.read_safetensors(tmp_path / "m" / "model.safetensors")
    check_tensors({n: (torch.bfloat16, tuple(t.shape)) for n, t in stored.items()}, model.tensors())


def test_plain_norms_and_activations():
    torch.manual_seed(0)
    x = torch.randn(5, 12, dtype=pp.F64)
    w = torch.randn(12, dtype=pp.F64)
    # one group is the ordinary root mean square; with groups every part has a mean square of (almost) one
    assert torch.allclose(pp.group_norm(x, w, 1e-6, 1), pp.rms(x, 1e-6) * w)
    parts = pp.group_norm(x, torch.ones(12, dtype=pp.F64), 0.0, 3).reshape(5, 3, 4)
    assert torch.allclose((parts ** 2).mean(-1), torch.ones(5, 3, dtype=pp.F64))
    assert not torch.allclose(pp.group_norm(x, w, 1e-6, 3), pp.group_norm(x, w, 1e-6, 1))
    # eps is inside the root: a zero vector stays zero, a tiny one is divided by sqrt(eps)
    assert torch.equal(pp.rms(torch.zeros(1, 4, dtype=pp.F64), 1e-4), torch.zeros(1, 4, dtype=pp.F64))
    assert torch.allclose(pp.rms(torch.full((1, 4), 1e-9, dtype=pp.F64), 1e-4), torch.full((1, 4), 1e-7, dtype=pp.F64))
    # PolyNorm: on a vector of +-1 every power has a root mean square of one
    z = torch.tensor([[1.0, -1.0, 1.0, -1.0]], dtype=pp.F64)
    got = pp.poly_norm(z, [2.0, 3.0, 5.0, 7.0], 0.0)
    assert torch.allclose(got, 2.0 * z + 3.0 + 5.0 * z + 7.0)
    assert abs(float(pp.gelu_tanh(torch.tensor(1.0, dtype=pp.F64))) - 0.8411919906082768) < 1e-12
    # a turn keeps lengths, turns nothing at position 0 and leaves the dimensions beyond `dims` alone
    a = torch.randn(3, 2, 8, dtype=pp.F64)
    r = pp.turn_pairs(a, torch.tensor([0, 5, 900]), 4, 100.0)
    assert torch.equal(r[0], a[0]) and torch.equal(r[..., 4:], a[..., 4:])
    assert torch.allclose(r.norm(dim=-1), a.norm(dim=-1))
    # pairs are neighbours: (1, 0, ...) at position 1 becomes (cos 1, sin 1, ...) for the first frequency (which is 1)
    e = torch.zeros(1, 4, dtype=pp.F64)
    e[0, 0] = 1.0
    t = pp.turn_pairs(e, torch.tensor([1]), 4, 100.0)
    assert torch.allclose(t[0], torch.tensor([0.5403023058681398, 0.8414709848078965, 0.0, 0.0], dtype=pp.F64))


def test_plain_latent_attention_in_closed_forms():
    torch.manual_seed(1)
    D, H, dk, dv, r, T = 6, 2, 3, 4, 5, 7
    m = {"heads": H, "dim": dk, "vdim": dv, "kv_rank": r, "scale": 0.7}
    w = {"q": torch.zeros(H * dk, D, dtype=pp.F64), "dkv": torch.randn(r, D, dtype=pp.F64),
         "dkv.norm": torch.rand(r, dtype=pp.F64) + 0.5, "uk": torch.randn(H * dk, r, dtype=pp.F64),
         "uv": torch.randn(H * dv, r, dtype=pp.F64), "o": torch.eye(H * dv, dtype=pp.F64)}
    h = torch.randn(T, D, dtype=pp.F64)
    pos = torch.arange(T)
    lat = pp.latent_of(h, w, "", m, 1e-6, pos)
    assert lat[1] is None and torch.allclose((lat[0] / w["dkv.norm"]).pow(2).mean(-1), torch.ones(T, dtype=pp.F64), atol=1e-4)
    # all scores zero: a position's output is the mean of the values it sees, its own included
    out = pp.latent_attention(h, w, "", m, 1e-6, pos, lat)
    v = lat[0] @ w["uv"].T
    for t in range(T):
        assert torch.allclose(out[t], v[:t + 1].mean(0))
    # with a gate the heads' outputs are multiplied by sigmoid(Wg h); a zero Wg halves them
    w["g"] = torch.zeros(H * dv, D, dtype=pp.F64)
    assert torch.allclose(pp.latent_attention(h, w, "", m, 1e-6, pos, lat), 0.5 * out)
    # a query that matches one key under a large scale returns that key's value, never a later one
    w.pop("g")
    w["q"] = torch.randn(H * dk, D, dtype=pp.F64)
    sharp = dict(m, scale=400.0)
    out = pp.latent_attention(h, w, "", sharp, 1e-6, pos, lat)
    q = (h @ w["q"].T).reshape(T, H, dk)
    k = (lat[0] @ w["uk"].T).reshape(T, H, dk)
    for t in range(T):
        for hh in range(H):
            best = int((k[:t + 1, hh] @ q[t, hh]).argmax())
            assert torch.allclose(out[t, hh * dv:(hh + 1) * dv], v[best, hh * dv:(hh + 1) * dv], atol=1e-6)
    # the turned part: only the difference of two positions enters a score, so shifting all positions changes nothing
    m2 = {"heads": H, "dim": dk, "rot_dim": 4, "vdim": dv, "kv_rank": r, "q_rank": 3, "scale": 0.9,
          "rot": {"dims": 4, "base": 50.0}}
    w2 = {"dq": torch.randn(3, D, dtype=pp.F64), "dq.norm": torch.ones(3, dtype=pp.F64),
          "uq": torch.randn(H * (dk + 4), 3, dtype=pp.F64), "dkv": torch.randn(r + 4, D, dtype=pp.F64),
          "dkv.norm": torch.ones(r, dtype=pp.F64), "uk": w["uk"], "uv": w["uv"], "o": w["o"]}
    a = pp.latent_attention(h, w2, "", m2, 1e-6, pos, pp.latent_of(h, w2, "", m2, 1e-6, pos))
    b = pp.latent_attention(h, w2, "", m2, 1e-6, pos + 11, pp.latent_of(h, w2, "", m2, 1e-6, pos + 11))
    assert torch.allclose(a, b)
    still = dict(m2, rot={"dims": 0, "base": 50.0})
    c = pp.latent_attention(h, w2, "", still, 1e-6, pos, pp.latent_of(h, w2, "", still, 1e-6, pos))
    assert not torch.allclose(a, c)


def test_plain_gla_in_closed_forms():
    torch.manual_seed(2)
    D, H, dk, dv, T = 5, 2, 3, 4, 9
    m = {"heads": H, "dim": dk, "vdim": dv, "tau": 2.0}
    w = {"q": torch.randn(H * dk, D, dtype=pp.F64), "k": torch.randn(H * dk, D, dtype=pp.F64),
         "v": torch.randn(H * dv, D, dtype=pp.F64), "g": torch.randn(H * dv, D, dtype=pp.F64),
         "o": torch.eye(H * dv, dtype=pp.F64), "norm": torch.ones(dv, dtype=pp.F64),
         "a1": torch.zeros(2, D, dtype=pp.F64), "a2": torch.zeros(H * dk, 2, dtype=pp.F64),
         "a2.b": torch.full((H * dk,), 0.0, dtype=pp.F64)}
    h = torch.randn(T, D, dtype=pp.F64)
    # a constant decay a = sigmoid(0)^(1/2): the state is sum_j a^(t-j) k_j v_j^T
    out, S = pp.gla(h, w, "", m, 1e-6)
    a = 0.5 ** 0.5
    q = (h @ w["q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    want_S = sum(a ** (T - 1 - j) * torch.einsum("hk,hv->hkv", k[j], v[j]) for j in range(T))
    assert torch.allclose(S, want_S)
    o = torch.stack([sum(a ** (t - j) * torch.einsum("hk,hv,hk->hv", k[j], v[j], q[t]) for j in range(t + 1))
                     for t in range(T)])
    want = (pp.rms(o, 1e-6).reshape(T, H * dv)) * pp.silu(h @ w["g"].T)
    assert torch.allclose(out, want)
    # the state carries: two halves, the second from the first's state, are the whole
    first, S1 = pp.gla(h[:4], w, "", m, 1e-6)
    second, S2 = pp.gla(h[4:], w, "", m, 1e-6, state=S1)
    assert torch.allclose(torch.cat([first, second]), out) and torch.allclose(S2, S)
    # the decay is per key channel: a channel whose bias is very negative forgets at once
    w["a2.b"][0] = -80.0
    _, S = pp.gla(h, w, "", m, 1e-6)
    assert torch.allclose(S[0, 0], k[-1, 0, 0] * v[-1, 0]) and not torch.allclose(S[0, 1], k[-1, 0, 1] * v[-1, 0])


def test_plain_experts_token_side_and_depth_average(tmp_path):
    torch.manual_seed(3)
    D, ff, E = 6, 4, 5
    w = {"router": torch.randn(E, D, dtype=pp.F64)}
    for e in list(range(E)) + ["shared"]:
        pre = f"e{e}." if e != "shared" else "shared."
        w[pre + "gate"], w[pre + "up"] = torch.randn(ff, D, dtype=pp.F64), torch.randn(ff, D, dtype=pp.F64)
        w[pre + "down"] = torch.randn(D, ff, dtype=pp.F64)
    h = torch.randn(3, D, dtype=pp.F64)
    mlp = {"router": {"experts": E, "top": 2}, "expert": {"ff": ff}, "shared": {"ff": ff}}
    s = torch.sigmoid(h @ w["router"].T)
    got = pp.moe_ffn(h, w, "", mlp)
    for t in range(3):
        order = s[t].argsort(descending=True)[:2]
        want = sum(pp.expert(s[t, e] * h[t:t + 1], w, f"e{int(e)}.")[0] for e in order) + pp.expert(h[t:t + 1], w, "shared.")[0]
        assert torch.allclose(got[t], want)
        # the weight is on the input, which is not the same as on the output, and it is not renormalised
        outside = sum(s[t, e] * pp.expert(h[t:t + 1], w, f"e{int(e)}.")[0] for e in order) + pp.expert(h[t:t + 1], w, "shared.")[0]
        assert not torch.allclose(got[t], outside)
    assert torch.allclose(pp.moe_ffn(h, w, "", dict(mlp, shared=None)) + pp.expert(h, w, "shared."), got)
    # a whole model: the depth average of the last layer alone decides what the head sees
    folder = pm.write(tmp_path / "m", pm.P1, 2)
    plain = pp.PlainPusunex(folder)
    toks = list(range(3, 40))
    lg, pre = pp.forward(plain.cfg, plain.w, toks, return_layers=True)
    assert lg.shape == (37, 300) and torch.isfinite(lg).all() and pre.shape == (4, 37, 96)
    mixed = plain.layers(toks)
    a = plain.w["l3.dwa"]
    hist = [plain.w["embed"][torch.as_tensor(toks)]] + list(pre)
    assert torch.allclose(mixed[3], sum(a[j] * hist[j] for j in range(5)))
    want = pp.group_norm(mixed[3], plain.w["final.norm"], 1e-5, 3) @ plain.w["head"].T
    assert torch.allclose(lg, want)
    # the token side reads the token itself: another token at one place changes that place's stream from layer 0 on
    other = list(toks)
    other[5] = (toks[5] + 1) % 300
    assert not torch.allclose(plain.layers(other)[0][5], mixed[0][5]) and torch.allclose(plain.layers(other)[0][4], mixed[0][4])
    # causal: a position's logits do not depend on what follows
    assert torch.allclose(plain.logits(toks[:11])[-1], lg[10])
    assert pp.generate(plain, toks[:5], 3) == pp.generate(plain, toks[:5], 4)[:3]
