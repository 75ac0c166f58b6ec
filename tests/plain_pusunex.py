"""A plain, slow Pusunex: one function per mechanism, float64 on the CPU.

It shares no code with the package: it reads config.json and the safetensors file by itself (through torch only)
and follows the equations below literally.

Notation.  x_t is the residual stream at token t (width D), p its position in its sequence, tok its token id.
    R(x) = x / sqrt(mean(x^2) + eps)                                  root mean square, eps inside the root
    G(x; w): x cut into `groups` equal consecutive parts, each part P replaced by R(P), the whole times w
    layer i:  x <- x + G(M(G(x; n1)); n1b);   x <- x + G(F(G(x; n2)); n2b)        (F only if the layer has one)
              e = side_table[tok][i d : (i + 1) d];  y = Wsp (gelu(Wsg x) * e);  x <- x + R(y) * ws   (token side)
              X_(i+1) = x;   x <- sum_(j <= i + 1) a_i[j] X_j                    (depth average; X_0 the embedding)
    logits = Whead G(x; n_final)

Mixers.
  latent attention:  q_h = (Wq h)_h, or (Wuq (R(Wdq h) * wq))_h when queries go through a latent of their own;
    c = R((Wdkv h)[:r]) * wc;  kr = (Wdkv h)[r:] turned by the position (pairs (2i, 2i + 1), angle p * base^(-2i/dims));
    the last `rot_dim` dimensions of q_h are turned the same way;  k_h,j = [Wuk_h c_j, kr_j],  v_h,j = Wuv_h c_j;
    s_j = scale * q_h . k_h,j for j <= t, softmax over them, o_h = sum_j p_j v_h,j;
    out = Wo (concat_h o_h * sigmoid(Wg h))  (the gate only where the mixer has one).  A mixer with `kv_from` = j
    has no Wdkv and takes the c that layer j computed for the same tokens.
  gla:  q = (Wq h) dk^(-1/2), k = Wk h [H, dk], v = Wv h [H, dv];  alpha = sigmoid(Wa2 (Wa1 h) + b)^(1 / tau) [H, dk];
    S <- diag(alpha) S + k v^T;  o = S^T q;  out = Wo (concat_h R(o_h) * wn * silu(Wg h)).

Feed-forwards.
  dense:  Wdown P(Wup h),  P(z) = a R(z) + b R(z^2) + c R(z^3) + e with powers taken element by element.
  moe:    s = sigmoid(Wr h); the `top` largest s choose; E(u) = Wdown (silu(Wgate u) * (Wup u));
          F = sum_chosen E_e(s_e h) + E_shared(h).
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


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, w, eps, groups):
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    return rms(parts, eps).reshape(x.shape) * w


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def turn_pairs(u, positions, dims, base):
    """u [T, ..., n]: the first `dims` of the last axis turned in pairs (2i, 2i + 1) by positions * base^(-2i/dims)."""
    if not dims:
        return u
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    a = positions.to(F64).reshape(-1, *([1] * (u.dim() - 1))) * f
    cos, sin = torch.cos(a), torch.sin(a)
    even, odd = u[..., 0:dims:2], u[..., 1:dims:2]
    out = u.clone()
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def latent_of(h, w, pre, m, eps, positions):
    """The latent c [T, r] and the turned shared key part [T, rot_dim] (or None) of a latent attention."""
    r, rd = m["kv_rank"], m.get("rot_dim") or 0
    d = h @ w[pre + "dkv"].T
    c = rms(d[:, :r], eps) * w[pre + "dkv.norm"]
    kr = None
    if rd:
        rot = m["rot"]
        kr = turn_pairs(d[:, r:r + rd], positions, rot["dims"], rot["base"])
    return c, kr


def latent_attention(h, w, pre, m, eps, positions, latent):
    """One sequence, tokens 0 .. T - 1 at `positions`; `latent` = (c, kr) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, dk, dv, rd = m["heads"], m["dim"], m["vdim"], m.get("rot_dim") or 0
    if m.get("q_rank"):
        cq = rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
        q = cq @ w[pre + "uq"].T
    else:
        q = h @ w[pre + "q"].T
    q = q.reshape(T, H, dk + rd)
    c, kr = latent
    k = (c @ w[pre + "uk"].T).reshape(T, H, dk)
    v = (c @ w[pre + "uv"].T).reshape(T, H, dv)
    s = torch.einsum("thd,jhd->htj", q[..., :dk], k)
    if rd:
        rot = m["rot"]
        qr = turn_pairs(q[..., dk:], positions, rot["dims"], rot["base"])
        s = s + torch.einsum("thd,jd->htj", qr, kr)
    s = s * m["scale"]
    seen = positions.reshape(1, T, 1) >= positions.reshape(1, 1, T)
    p = torch.softmax(s.masked_fill(~seen, float("-inf")), -1)
    o = torch.einsum("htj,jhd->thd", p, v).reshape(T, H * dv)
    if pre + "g" in w:
        o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def gla(h, w, pre, m, eps, state=None):
    """One sequence; returns (output [T, D], the state [H, dk, dv] after the last token)."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[pre + "k"].T).reshape(T, H, dk)
    v = (h @ w[pre + "v"].T).reshape(T, H, dv)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms(o, eps) * w[pre + "norm"]
    y = o.reshape(T, H * dv) * silu(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T, S


def poly_norm(z, coef, eps):
    a, b, c, e = [float(v) for v in coef]
    return a * rms(z, eps) + b * rms(z ** 2, eps) + c * rms(z ** 3, eps) + e


def dense_ffn(h, w, pre, eps):
    return poly_norm(h @ w[pre + "up"].T, w[pre + "act"], eps) @ w[pre + "down"].T


def expert(u, w, pre):
    return (silu(u @ w[pre + "gate"].T) * (u @ w[pre + "up"].T)) @ w[pre + "down"].T


def router_scores(h, w, pre):
    return torch.sigmoid(h @ w[pre + "router"].T)


def moe_ffn(h, w, pre, mlp):
    s = router_scores(h, w, pre)
    top = mlp["router"]["top"]
    chosen = torch.topk(s, top, dim=-1).indices
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += expert(s[t, e] * h[t:t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + expert(h, w, pre + "shared.")
    return out


def token_side(x, tokens, w, i, dim, eps):
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e
    y = g @ w[f"l{i}.side.proj"].T
    return x + rms(y, eps) * w[f"l{i}.side.norm"]


def router_gap(h, w, pre, mlp):
    """Per token, how far the last chosen expert's router logit lies above the first one that is not chosen."""
    z = (h @ w[pre + "router"].T).sort(-1, descending=True).values
    top = mlp["router"]["top"]
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else torch.full((h.shape[0],), float("inf"), dtype=F64)


def forward(cfg, w, tokens, return_layers=False, gaps=None):
    """One sequence from its first token; logits [T, vocab] (and the stream after every layer, before averaging).
    gaps: a list that receives every mixture layer's `router_gap`."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups") or 1
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"][tokens]
    history, latents, layers = [x], {}, []
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        h = group_norm(x, w[pre + "norm1"], eps, groups)
        if layer["type"] == "gla":
            y, _ = gla(h, w, pre + "mix.", m, eps)
        else:
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, w, pre + "mix.", m, eps, positions)
                src = i
            y = latent_attention(h, w, pre + "mix.", m, eps, positions, latents[src])
        x = x + group_norm(y, w[pre + "norm1b"], eps, groups)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = group_norm(x, w[pre + "norm2"], eps, groups)
            y = dense_ffn(h, w, pre + "mlp.", eps) if mlp["kind"] == "dense" else moe_ffn(h, w, pre + "mlp.", mlp)
            if gaps is not None and mlp["kind"] == "moe":
                gaps.append(router_gap(h, w, pre + "mlp.", mlp))
            x = x + group_norm(y, w[pre + "norm2b"], eps, groups)
        if side:
            x = token_side(x, tokens, w, i, side["dim"], eps)
        history.append(x)
        layers.append(x)
        a = w[pre + "dwa"]
        x = sum(a[j] * history[j] for j in range(i + 2))
    logits = group_norm(x, w["final.norm"], eps, groups) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


def load(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


class PlainPusunex:
    """A model folder read by this file alone."""

    def __init__(self, folder):
        self.cfg, self.w = load(folder)

    def logits(self, tokens):
        return forward(self.cfg, self.w, tokens)

    def close_calls(self, tokens, margin):
        """The positions at which some router's choice hangs on less than `margin` of a logit: arithmetic of fewer
        bits may choose otherwise there, and no comparison at reduced precision should rest on them."""
        gaps = []
        forward(self.cfg, self.w, tokens, gaps=gaps)
        if not gaps:
            return set()
        return set(torch.nonzero(torch.stack(gaps).min(0).values < margin).flatten().tolist())

    def layers(self, tokens):
        """The stream that leaves every layer (after the depth average), [layers, T, D]."""
        _, pre = forward(self.cfg, self.w, tokens, return_layers=True)
        hist, out = [self.w["embed"][torch.as_tensor(tokens, dtype=torch.long)]], []
        for i in range(len(pre)):
            hist.append(pre[i])
            a = self.w[f"l{i}.dwa"]
            out.append(sum(a[j] * hist[j] for j in range(i + 2)))
        return torch.stack(out)


def generate(plain, prompt, n_new):
    """Greedy continuation, the whole sequence recomputed for every token."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(plain.logits(toks)[-1].argmax()))
    return toks[len(prompt):]
