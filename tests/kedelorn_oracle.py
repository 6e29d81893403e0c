"""Plain, slow float64 implementation of the Kedelorn design (pre-norm blocks on several residual streams, retention and
latent-attention mixers, routed feed-forward), one function per mechanism, written from the equations and sharing no code
with the product path. It takes the config.json dictionary and a {name: tensor} dict and processes a whole sequence at
once: no cache, no carried state; recurrences loop over tokens.

Notation: h [T, width] is a sublayer's input; rms(x) = x / sqrt(mean(x^2) + eps) over the last axis.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is centred on zero."""
    return rms(x, eps) * (1.0 + w)


def silu(x):
    return x * torch.sigmoid(x)


def rotary_frequencies(rot):
    """Per-pair frequencies and the factor on cos / sin, with the optional long-context interpolation."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    out = f.clone()
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, rot, start=0):
    """x [T, ..., D]: the first rot.dims channels are rotated in pairs (i, i + dims/2); the rest pass."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rotary_frequencies(rot)
    T = x.shape[0]
    p = torch.arange(start, start + T, dtype=F64)
    ang = p[:, None] * f[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [half]
    c, s = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def retention(h, w, mx, eps):
    """Decayed linear attention without normaliser: S <- decay_h S + k v^T, o = S^T q; unit-rms heads, silu gate."""
    H, D, DV = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    q = rotate((h @ w["q"].T).reshape(T, H, D), mx["rot"])
    k = rotate((h @ w["k"].T).reshape(T, H, D), mx["rot"]) * D ** -0.5
    v = (h @ w["v"].T).reshape(T, H, DV)
    o = torch.zeros(T, H, DV, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, DV, dtype=F64)
        for t in range(T):
            S = float(mx["decay"][hd]) * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms(o, eps).reshape(T, H * DV) * silu(h @ w["g"].T)
    return o @ w["o"].T


def latent_kv(h, w, mx, eps):
    """The cached part of a latent-attention layer: the normed latent and the rotated shared key part."""
    R, DR = int(mx["kv_rank"]), int(mx["rot_dim"])
    d = h @ w["dkv"].T
    c = rms(d[:, :R], eps) * w["dkv.norm"]
    kr = rotate(d[:, R:R + DR], mx["rot"])
    return c, kr


def latent_attention(h, w, mx, eps, kv, sink=True):
    """Causal softmax attention whose keys and values are up-projections of a shared latent; a per-head sink term in the
    denominator; a per-head sigmoid gate on the output."""
    H, D, DR, DV = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"])
    T = h.shape[0]
    c, kr = kv
    q = (h @ w["q"].T).reshape(T, H, D + DR)
    qn, qr = q[..., :D], rotate(q[..., D:], mx["rot"])
    kn = (c @ w["uk"].T).reshape(T, H, D)
    v = (c @ w["uv"].T).reshape(T, H, DV)
    gate = torch.sigmoid(h @ w["g"].T)                       # [T, H]
    out = torch.zeros(T, H, DV, dtype=F64)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * float(mx["scale"])
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
        m = torch.maximum(s.max(-1).values, w["sink"][hd])
        e = torch.exp(s - m[:, None])
        p = e / (e.sum(-1) + (torch.exp(w["sink"][hd] - m) if sink else 0.0))[:, None]
        out[:, hd] = p @ v[:, hd]
    return (out * gate[..., None]).reshape(T, H * DV) @ w["o"].T


def expert(h, up, down):
    return torch.relu(h @ up.T).pow(2) @ down.T


def routed_ff(h, w, mlp, correction=True):
    """Sigmoid router: the `top` largest of (score + correction) are chosen, their plain scores times `scale` weigh the
    experts; a shared expert runs for every token behind a scalar sigmoid gate."""
    r = mlp["router"]
    E, top, scale = int(r["experts"]), int(r["top"]), float(r["scale"])
    s = torch.sigmoid(h @ w["router"].T)
    pick = torch.topk(s + (w["correction"] if correction else 0.0), top, dim=-1).indices
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e in pick[t].tolist():
            out[t] += s[t, e] * scale * expert(h[t], w[f"e{e}.up"], w[f"e{e}.down"])
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * expert(h, w["shared.up"], w["shared.down"])
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: dict, tokens, sink=True, correction=True):
    """Returns (logits [T, vocab], residual stream after every layer [layers, T, width]), float64. sink / correction =
    False leave a mechanism out (tests use that to show that their weights would expose its absence)."""
    eps = float(cfg["norm"]["eps"])
    n = int(cfg.get("streams", 1))
    x0 = tensors["embed"].to(F64)[torch.tensor(list(tokens))]
    xs = [x0.clone() for _ in range(n)]
    kv_of, dumps = {}, []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q in (1, 2):
            if q == 2 and L.get("mlp") is None:
                continue
            hc = sub(tensors, f"{p}hc{q}.")
            u = sum(hc["in"][s] * xs[s] for s in range(n))
            h = offset_norm(u, tensors[f"{p}norm{q}"].to(F64), eps)
            if q == 2:
                y = routed_ff(h, sub(tensors, p + "mlp."), L["mlp"], correction)
            elif L["type"] == "retention":
                y = retention(h, sub(tensors, p + "mix."), L["mixer"], eps)
            elif L["type"] == "latent_attention":
                w = sub(tensors, p + "mix.")
                src = L["mixer"].get("kv_from")
                if src is None:
                    kv_of[i] = latent_kv(h, w, L["mixer"], eps)
                y = latent_attention(h, w, L["mixer"], eps, kv_of[i if src is None else int(src)], sink)
            else:
                raise ValueError(L["type"])
            xs = [sum(hc["mix"][s, t] * xs[s] for s in range(n)) + hc["out"][t] * y for t in range(n)]
        dumps.append(sum(xs))
    x = offset_norm(sum(xs), tensors["final.norm"].to(F64), eps)
    return x @ tensors["head"].to(F64).T, torch.stack(dumps)


def greedy(cfg: dict, tensors: dict, prompt, n_new):
    """n_new greedy tokens after the prompt (the whole sequence is recomputed for every token)."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, tensors, toks)[0][-1].argmax()))
    return toks[len(prompt):]
