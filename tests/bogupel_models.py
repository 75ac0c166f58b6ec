"""Small Bogupel configurations for the tests, and a writer of model folders with weights that make faults show:
router weights are scaled up so that the experts' scores lie well apart, the decays' offsets are pushed down so that
the recurrent state remembers for hundreds of tokens, sinks and biases are of the size of the scores, and the norms'
alphas are small enough to keep tanh away from saturation."""
from pathlib import Path

import torch


def rot(dims, base, scaling=None):
    return {"dims": dims, "base": base, "scaling": scaling}


def scaling(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


def attention(heads, kv_heads, dim, vdim, scale, window=None, rotation=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": None if window is None else {"size": window}, "rot": rotation}


def delta(heads, dim, rank=4):
    return {"heads": heads, "dim": dim, "rank": rank}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp=None):
    return {"type": "attention" if "kv_heads" in mixer else "general_delta", "mixer": mixer, "mlp": mlp}


def config(vocab, width, eps, layers, scale=1.0, bigram=None, logit_scale=None, loop=None):
    c = {"architecture": "Bogupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
         "embedding": {"scale": scale}}
    if bigram is not None:
        c["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# Wavelengths of the first rotation fall into all three bands of the rescaling; a partial rotation; key and value sizes
# that differ both ways; a loop over three passes that does not start at the first layer; a layer without feed-forward,
# one without window; a router that chooses every expert; a state of 24 x 24 (one column tile, rows padded).
B1 = config(300, 96, 1e-5, [
    layer(attention(4, 2, 32, 16, 0.25, 40, rot(16, 10000.0, scaling(4.0, 1.0, 4.0, 64))), moe(6, 2, 40, 1.5)),
    layer(delta(3, 24, 5), moe(4, 4, 16, 0.7)),
    layer(attention(2, 2, 16, 48, 0.3, None, rot(16, 500.0))),
    layer(attention(3, 1, 24, 24, 0.2, 7, rot(8, 77.0)), moe(5, 1, 28, 3.0))],
    scale=4.0, bigram=(211, 31, 17), logit_scale=0.5, loop=(1, 3, 3))
# no loop, no second table, no constant on the logits; a width and sizes that are no multiples of 8 (the products of
# the 32-bit kind on both paths); one head; windows of one page exactly and of one key; keys that are not turned while
# the values are (dims 0); an attention with neither rotation nor window; a state of 40 x 40 (two column tiles).
B2 = config(257, 100, 3e-6, [
    layer(delta(2, 40), moe(3, 2, 20, 2.0)),
    layer(attention(5, 5, 20, 12, 0.22, 64, rot(10, 1000.0)), moe(5, 1, 28, 1.0)),
    layer(attention(2, 1, 34, 6, 0.17, 1, rot(0, 50000.0))),
    layer(attention(1, 1, 18, 10, 0.3)),
    layer(delta(1, 9, 1))])
# a loop from the first layer on, over all layers, twice; more experts than a warp has lanes; a window that ends inside
# the second page; rescaled frequencies in a full rotation; head sizes of 64 (the tensor-core attention in bfloat16)
B3 = config(150, 64, 1e-6, [
    layer(attention(2, 1, 64, 64, 0.125, 70, rot(64, 50000.0, scaling(8.0, 1.0, 4.0, 128))), moe(40, 3, 8, 1.5)),
    layer(delta(2, 32))],
    scale=2.0, bigram=(64, 5, 3), logit_scale=0.25, loop=(0, 2, 2))
# peaked attention: large scales, so that one key decides a query's output; windows that end inside a page, at a
# page's edge and beyond two pages; little else in the layers
SHARP = config(200, 64, 1e-5, [
    layer(attention(4, 2, 16, 16, 2.5, 100, rot(8, 10000.0))),
    layer(attention(2, 2, 32, 32, 2.0, 64, rot(32, 1000.0))),
    layer(attention(2, 1, 16, 32, 2.0, 33, rot(16, 100.0))),
    layer(attention(2, 1, 16, 16, 2.5, None, rot(16, 10000.0)))], bigram=(97, 7, 11))
# the recurrent layer alone decides, with decays very close to one
LONG_MEMORY = config(180, 48, 1e-5, [layer(delta(3, 16))], bigram=(50, 3, 1))
# sizes of real models at a width of 1,024: the tensor-core products and the tensor-core attention
REAL = config(1000, 1024, 1e-6, [
    layer(attention(8, 2, 128, 128, 0.09, 256, rot(64, 10000.0, scaling(8.0, 1.0, 4.0, 8192))), moe(8, 2, 256, 7.0)),
    layer(delta(8, 64, 32), moe(16, 4, 128, 7.0)),
    layer(attention(16, 4, 64, 128, 0.125, None, rot(64, 500000.0))),
    layer(delta(4, 128, 64), moe(8, 2, 256, 7.0))],
    scale=8.0, bigram=(4093, 31, 17), logit_scale=0.5, loop=(1, 3, 2))

def random_config(rng):
    """A configuration drawn from `rng` (random.Random): 2 to 6 layers of either kind in any order, sizes that are and
    are not multiples of 16, every optional part present or absent, a loop anywhere or none."""
    width = rng.choice([128, 192, 256, 320, 200])
    n_layers = rng.randint(2, 6)
    layers = []
    for _ in range(n_layers):
        mlp = None if rng.random() < 0.2 else moe(rng.choice([4, 8, 12, 16]), rng.choice([1, 2, 3]), rng.choice([32, 64, 96]),
                                                  rng.choice([1.0, 1.5, 3.0]))
        if rng.random() < 0.6:
            heads = rng.choice([2, 4, 6, 8])
            kv = rng.choice([k for k in (1, 2, 4, 8) if heads % k == 0])
            dim, vdim = rng.choice([32, 48, 64, 96, 128, 40]), rng.choice([32, 48, 64, 96, 128, 24])
            dims = rng.choice([d for d in (0, 8, 16, 24, 32, dim) if d <= dim])
            sc = rng.choice([None, scaling(8.0, 1.0, 4.0, rng.choice([64, 2048])), scaling(4.0, 2.0, 8.0, 256)])
            rotation = None if rng.random() < 0.1 else rot(dims, rng.choice([10000.0, 50000.0, 500.0]), sc)
            layers.append(layer(attention(heads, kv, dim, vdim, dim ** -0.5, rng.choice([None, 17, 64, 96, 128, 200]), rotation), mlp))
        else:
            layers.append(layer(delta(rng.choice([1, 2, 4, 6]), rng.choice([16, 32, 48, 64, 96]), rng.choice([4, 16, 32])), mlp))
    loop = None
    if rng.random() < 0.7:
        a = rng.randint(0, n_layers - 1)
        loop = (a, rng.randint(a + 1, n_layers), rng.randint(1, 3))
    bigram = None if rng.random() < 0.2 else (rng.choice([509, 1021, 4093]), rng.choice([31, 7, 1]), rng.choice([17, 3, 1]))
    return config(rng.choice([256, 512, 1000]), width, rng.choice([1e-5, 1e-6]), layers, scale=rng.choice([0.25, 1.0, 4.0]),
                  bigram=bigram, logit_scale=rng.choice([None, 0.25, 2.0]), loop=loop)


ALL = {"B1": (B1, 3), "B2": (B2, 4), "B3": (B3, 5), "SHARP": (SHARP, 6), "LONG_MEMORY": (LONG_MEMORY, 8)}


def write(folder, raw, seed, std=0.1, decay_offset=-4.0, removal_offset=0.0, router_scale=6.0, moe_out=0.25):
    """A model folder of seeded random weights, adjusted as the top of this file says.  moe_out scales the experts'
    down projections: in bfloat16 a router now and then chooses another expert than exact arithmetic does (two scores
    a rounding apart); with a quarter of the output the other choice still shows at its own position, which a
    comparison in bfloat16 leaves out, and hardly at the later ones."""
    from oracle_engine_b200.config.bogupel import BogupelConfig
    from oracle_engine_b200.weights.random_init import write_model_folder
    from oracle_engine_b200.weights.safetensors_io import ModelFiles, write_safetensors
    folder = Path(folder)
    write_model_folder(folder, BogupelConfig.from_dict(raw), seed=seed, std=std)
    files = ModelFiles(folder)
    tensors = {}
    for n in files.names():
        t = files.read(n).clone()
        f = t.float()
        if n.endswith(".router"):
            f = f * router_scale                  # scores well apart: few choices hang on a rounding
        elif n.endswith(".correction"):
            f = f * (0.3 / std)                   # a bias of the size of the scores' spread: leaving it out shows
        elif n.endswith(".down"):
            f = f * moe_out
        elif n.endswith(".w0"):
            f = f + decay_offset                  # decays near one: a lost state shows for a long time
        elif n.endswith(".alpha"):
            f = f * 0.5                           # tanh well inside its bend
        elif n.endswith(".sink"):
            f = f * 10.0 + 1.0                    # a sink of the size of the scores
        elif n.endswith(".a.b"):
            f = f * 3.0 + removal_offset          # far below zero: hardly anything is removed, the state remembers
        elif n.endswith((".q.b", ".k.b", ".v.b")) or (n.endswith(".b") and "norm" in n):
            f = f * 3.0
        elif n == "loop.step" or n == "bigram":
            f = f * 5.0
        tensors[n] = f.to(t.dtype)
    files.close()
    write_safetensors(folder / "model.safetensors", tensors)
    return str(folder)
