"""Small Pusunex configurations for the tests, and a writer of model folders with weights that make faults show:
router weights are scaled up so that the experts' scores lie well apart, the decays' biases put the decays near
one, the depth average's weights sum to about one, norm weights vary per channel."""
from pathlib import Path

import torch


def latent(heads, dim, vdim, kv_rank, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "latent_attention", m


def latent2(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims=None):
    return "latent_attention_2", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                  "q_rank": q_rank, "scale": scale,
                                  "rot": {"dims": rot_dim if dims is None else dims, "base": base}}


def gla(heads, dim, vdim, tau, rank):
    return "gla", {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": None if shared is None else {"ff": shared}}


def layer(mixer, mlp=None):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def config(vocab, width, eps, groups, side, layers):
    c = {"architecture": "Pusunex", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
         "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    return c


# every kind of layer and of feed-forward; a layer that reads an earlier layer's latents with heads of its own; one
# without feed-forward; a router that chooses every expert; three norm groups; key, value and latent sizes all differ
P1 = config(300, 96, 1e-5, 3, 8, [
    layer(latent(4, 24, 16, 40, 0.2), moe(6, 2, 40, 24)),
    layer(gla(3, 16, 24, 8.0, 12), dense(72)),
    layer(latent2(2, 16, 8, 32, 24, 36, 0.2, 10000.0)),
    layer(latent(3, 8, 40, 40, 0.3, kv_from=0), moe(4, 4, 16))])
# one norm group, no token side, a width and sizes that are no multiples of 8 (the products of the 32-bit kind on
# both paths), one expert per token, a tau of one, a turned part of which only some dimensions turn, one head
P2 = config(257, 100, 3e-6, 1, 0, [
    layer(gla(1, 10, 30, 1.0, 5), moe(5, 1, 28, 36)),
    layer(latent2(5, 12, 6, 12, 18, 20, 0.25, 50.0, dims=4), dense(60)),
    layer(latent(2, 34, 6, 18, 0.17), moe(3, 2, 20))])
# eight norm groups, more experts than a warp has lanes, a key size above 64 and values in two column tiles in the
# linear attention, a latent wider than a warp, a layer that reads the latents of the layer just before it
P3 = config(150, 64, 1e-6, 8, 4, [
    layer(latent(2, 16, 16, 100, 0.25), moe(40, 3, 8, 16)),
    layer(latent(1, 40, 8, 100, 0.2, kv_from=0), None),
    layer(gla(2, 70, 40, 4.0, 3), dense(32)),
    layer(latent2(3, 8, 16, 8, 16, 8, 0.3, 1e6), dense(16))])
# peaked attention: large scales, so that one key decides a query's output; little else in the layers
SHARP = config(200, 64, 1e-5, 2, 0, [
    layer(latent(4, 16, 16, 32, 2.5)),
    layer(latent2(2, 16, 16, 16, 24, 32, 2.0, 10000.0), dense(32))])
# the linear attention alone decides, with decays very close to one
LONG_MEMORY = config(180, 48, 1e-5, 1, 0, [layer(gla(3, 16, 16, 16.0, 4))])
# sizes of real models at a width of 1,024: the tensor-core products and the tensor-core attention over latents
REAL = config(1000, 1024, 1e-6, 4, 32, [
    layer(latent(16, 64, 64, 128, 0.125), moe(8, 2, 256, 512)),
    layer(gla(8, 64, 128, 16.0, 32), dense(2048)),
    layer(latent2(8, 64, 32, 128, 96, 256, 0.1, 10000.0), moe(16, 4, 128)),
    layer(latent(8, 128, 128, 128, 0.09, kv_from=0), None)])

ALL = {"P1": (P1, 3), "P2": (P2, 4), "P3": (P3, 5), "SHARP": (SHARP, 6), "LONG_MEMORY": (LONG_MEMORY, 8)}


# In bfloat16 a router now and then chooses another expert than exact arithmetic does (two scores a rounding apart).
# The norm after the feed-forward gives the experts' output the stream's own size, so one such token would be half
# wrong, and every later token that attends to it a little.  The tests' mixtures add a quarter of that: the other
# choice still shows at its own position, which a comparison in bfloat16 leaves out, and no longer at the later ones.
MOE_OUT = 0.25


def write(folder, raw, seed, std=0.1, decay_bias=3.0):
    """A model folder of seeded random weights, adjusted as the top of this file says."""
    from oracle_engine_b200.config.pusunex import PusunexConfig
    from oracle_engine_b200.weights.random_init import write_model_folder
    from oracle_engine_b200.weights.safetensors_io import ModelFiles, write_safetensors
    folder = Path(folder)
    write_model_folder(folder, PusunexConfig.from_dict(raw), seed=seed, std=std)
    files = ModelFiles(folder)
    tensors, names = {}, set(files.names())
    for n in files.names():
        t = files.read(n).clone()
        f = t.float()
        if n.endswith(".router"):
            f = f * 4.0                           # scores well apart: few choices hang on a rounding
        elif n.endswith(".a2.b"):
            f = f + decay_bias                    # decays near one: a lost state shows for a long time
        elif n.endswith(".dwa"):
            f = f / f.numel()                     # a weighted mean, not a sum that grows with the depth
        elif n.endswith(".side.embed"):
            f = f * 5.0
        elif n.endswith(".norm2b") and n[:-len("norm2b")] + "mlp.router" in names:
            f = f * MOE_OUT                       # see MOE_OUT
        tensors[n] = f.to(t.dtype)
    files.close()
    write_safetensors(folder / "model.safetensors", tensors)
    return str(folder)
