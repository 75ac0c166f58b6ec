"""A plain, slow Bogupel: one function per mechanism, float64 on the CPU.

It shares no code with the package: it reads config.json and the safetensors file by itself
(through torch only) and follows the equations below literally.

Notation.  x_t is the residual stream at token t (width D), p its position in its sequence.
    embedding   x_t = E[tok_t] * c + B[(tok_(t-1) * m_prev + tok_t * m_cur) mod n], and B[n] for p = 0
    norm        T(x; alpha, w, b) = tanh(alpha * x) * w + b            (no mean, no variance)
    layer       x <- x + M(T_1(x));   x <- x + F(T_2(x))              (F only if the layer has one)
    loop        layers start .. stop - 1 run `times` times; before pass t: x <- x + x_embedding (t > 0), x <- x + s[t]

Mixer "attention" (H query heads, G key heads, key size d, value size dv):
    q = Wq h + bq, k = Wk h + bk, v = Wv h + bv
    q, k <- R(q) * wq, R(k) * wk per head, R(u) = u / sqrt(mean(u^2) + eps)
    q, k: the first `dims` dimensions turned by the position, i paired with i + dims/2, angle p * f_i; the f_i
          rescaled by wavelength in three bands when `scaling` is given
    v <- R(v) per head (no weight), then all dv dimensions turned by the position of the KEY, m paired with
          m + dv/2, angle j * base^(-2m/dv), never rescaled
    s_j = scale * q . k_j for t - window < j <= t;   p_j = exp(s_j) / (exp(sink_h) + sum_j exp(s_j))
    o = sum_j p_j v_j, turned back by the QUERY's position (angle -t * base^(-2m/dv));   M = Wo concat_h o

Mixer "general_delta" (H heads of size d, one matrix S [d, d] per head and sequence, zero at the start):
    r = Wr h, k = Wk h, v = Wv h;   w = exp(-e^(-1/2) * sigmoid(W2 tanh(W1 h) + w0));   a = sigmoid(Wa h + ba)
    u = k / sqrt(|k|^2 + 1e-6) per head
    S <- diag(w) S - (a * u) (u^T S) + k v^T      (both terms read the old S);    o = S^T r
    M = Wo (concat_h R(o) * wn * sigmoid(Wg h))

Feed-forward "moe":  z = Wr h, s = sigmoid(z); the `top` largest s + correction choose; weights are the chosen s;
    expert: g = min(Wgate h, L), u = clamp(Wup h, -L, L), y = g * sigmoid(1.702 g) * (u + 1), output Wdown y.

Logits = Whead T_final(x) * logit_scale.
"""
import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def read_safetensors(path):
    raw = Path(path).read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    head = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytearray(raw[8 + n + lo: 8 + n + hi])
        t = torch.frombuffer(buf, dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(F64) if t.is_floating_point() else t.clone()
    return out


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(x, alpha, w, b):
    return torch.tanh(alpha * x) * w + b


def frequencies(dims, base, scaling=None):
    """The turning rates f_i, i < dims/2, after the optional rescaling by wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            wave = 2.0 * math.pi / f
            if wave < scaling["original"] / scaling["high"]:
                pass
            elif wave > scaling["original"] / scaling["low"]:
                f = f / scaling["factor"]
            else:
                s = (scaling["original"] / wave - scaling["low"]) / (scaling["high"] - scaling["low"])
                f = (1.0 - s) * f / scaling["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def turn_halves(x, pos, freq, sign=1.0):
    """x [T, heads, n]; the first 2 * len(freq) dimensions turned, i paired with i + len(freq); pos [T]."""
    half = freq.numel()
    if half == 0:
        return x
    ang = sign * pos.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], -1)


def embed(tokens, w, cfg):
    """tokens of one sequence from position 0 -> [T, D]."""
    e = cfg["embedding"]
    x = w["embed"][tokens] * float(e.get("scale", 1.0))
    bg = e.get("bigram")
    if bg:
        n = int(bg["buckets"])
        rows = [n] + [(int(tokens[t - 1]) * int(bg["mul_prev"]) + int(tokens[t]) * int(bg["mul_cur"])) % n
                      for t in range(1, len(tokens))]
        x = x + w["bigram"][torch.tensor(rows)]
    return x


def attention(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, d)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, d)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, dv)
    q = unit_rms(q, eps) * w[pre + "q.norm"]
    k = unit_rms(k, eps) * w[pre + "k.norm"]
    rot = m.get("rot")
    if rot and rot["dims"]:
        f = frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = turn_halves(q, pos, f), turn_halves(k, pos, f)
    v = unit_rms(v, eps)
    base = rot["base"] if rot else None
    fv = frequencies(dv, base) if rot else torch.zeros(0, dtype=F64)
    v = turn_halves(v, pos, fv)
    window = (m.get("mask") or {}).get("size") or 0
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        i, j = pos[:, None], pos[None, :]
        seen = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
        s = s.masked_fill(~seen, -math.inf)
        sink = w[pre + "sink"][hh]
        top = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
        out[:, hh] = p @ v[:, g]
    out = turn_halves(out, pos, fv, sign=-1.0)
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def general_delta(h, w, pre, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ w[pre + "r"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, d)
    z = torch.tanh(h @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"]
    dec = torch.exp(-math.exp(-0.5) * torch.sigmoid(z)).view(T, H, d)
    a = torch.sigmoid(h @ w[pre + "a"].T + w[pre + "a.b"]).view(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=F64)
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        uS = torch.einsum("hi,hij->hj", u[t], S)
        S = dec[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hij,hi->hj", S, r[t])
    y = unit_rms(o, eps).reshape(T, H * d) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


def moe(h, w, pre, mlp, gaps=None):
    """gaps (a list or None) receives, per token, how far the last chosen expert's choice score lies above the best
    one that was not chosen."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    lim = float(mlp["expert"]["limit"])
    s = torch.sigmoid(h @ w[pre + "router"].T)
    chosen = torch.topk(s + w[pre + "correction"], top, dim=-1).indices
    if gaps is not None and top < E:
        ranked = torch.sort(s + w[pre + "correction"], dim=-1, descending=True).values
        gaps.append(ranked[:, top - 1] - ranked[:, top])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            g = torch.clamp(w[f"{pre}e{e}.gate"] @ h[t], max=lim)
            u = torch.clamp(w[f"{pre}e{e}.up"] @ h[t], -lim, lim)
            out[t] += s[t, e] * (w[f"{pre}e{e}.down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0)))
    return out


def layer_order(cfg):
    """[(layer, pass or None, first layer of its pass)] in the order the layers run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None, False) for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    out = [(i, None, False) for i in range(a)]
    for t in range(times):
        out += [(i, t, i == a) for i in range(a, b)]
    return out + [(i, None, False) for i in range(b, n)]


def forward(cfg, w, tokens, keep_layers=False, gaps=None):
    """Logits [T, vocab] of one sequence from its first token (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = embed(tokens, w, cfg)
    x = x0.clone()
    kept = []
    for i, t, first in layer_order(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        L, pre = cfg["layers"][i], f"l{i}."
        n1 = dyt(x, w[pre + "norm1.alpha"], w[pre + "norm1"], w[pre + "norm1.b"])
        if L["type"] == "attention":
            x = x + attention(n1, w, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "general_delta":
            x = x + general_delta(n1, w, pre + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            n2 = dyt(x, w[pre + "norm2.alpha"], w[pre + "norm2"], w[pre + "norm2.b"])
            x = x + moe(n2, w, pre + "mlp.", L["mlp"], gaps)
        kept.append(x.clone())
    xn = dyt(x, w["final.norm.alpha"], w["final.norm"], w["final.norm.b"])
    logits = xn @ w["head"].T * float(cfg.get("logit_scale", 1.0))
    return (logits, torch.stack(kept)) if keep_layers else logits


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


class PlainBogupel:
    def __init__(self, folder):
        self.cfg, self.w = load(folder)

    def logits(self, tokens):
        return forward(self.cfg, self.w, tokens)

    def layers(self, tokens):
        """The stream after every layer run (a looped layer counts each time), [runs, T, D]."""
        return forward(self.cfg, self.w, tokens, keep_layers=True)[1]

    def close_calls(self, tokens, margin):
        """The positions at which some router's choice hangs on less than `margin` of a score: arithmetic of fewer
        bits may choose otherwise there, and no comparison at reduced precision should rest on them."""
        gaps = []
        forward(self.cfg, self.w, tokens, gaps=gaps)
        if not gaps:
            return set()
        return set(torch.nonzero(torch.stack(gaps).min(0).values < margin).flatten().tolist())


def generate(plain, prompt, n_new):
    """Greedy continuation, the whole sequence recomputed for every token."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(plain.logits(toks)[-1].argmax()))
    return toks[len(prompt):]
