"""Plain, slow float64 implementation of the hybrid sequence models (Bimopel), one function per mechanism, written from
the equations and sharing no code with the product path. It takes the config.json dictionary and a {name: tensor} dict,
processes a whole sequence at once (no cache, no state carried between calls) and loops over tokens where the model
is recurrent.

Notation: h [T, width] is a sublayer's input; rms(x) = x / sqrt(mean(x^2) + eps) over the last axis.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def sinusoid(n_tokens, width, start=0):
    """[T, width]: entry 2i = sin(p * 10000^(-2i/width)), entry 2i+1 = cos of the same angle."""
    p = torch.arange(start, start + n_tokens, dtype=F64)[:, None]
    out = torch.zeros(n_tokens, width, dtype=F64)
    for c in range(width):
        ang = p[:, 0] * 10000.0 ** (-(2 * (c // 2)) / width)
        out[:, c] = torch.cos(ang) if c % 2 else torch.sin(ang)
    return out


def causal_conv_silu(x, taps_w, bias):
    """x [T, C]; taps_w [C, K] with the last column on the current token; zeros before the start."""
    T, C = x.shape
    K = taps_w.shape[1]
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        acc = bias.clone()
        for j in range(K):
            src = t - (K - 1) + j
            if src >= 0:
                acc = acc + taps_w[:, j] * x[src]
        out[t] = silu(acc)
    return out


def ssd_scan(x, B, Cm, dt, a_log, skip, groups):
    """x [T, H, P], B / Cm [T, G, N], dt [T, H] (already softplus'ed). Per head: S <- exp(-exp(a_log) dt) S + dt B x^T,
    y = S^T C + skip x."""
    T, H, P = x.shape
    N = B.shape[-1]
    per = H // groups
    y = torch.zeros(T, H, P, dtype=F64)
    for h in range(H):
        g = h // per
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = math.exp(-math.exp(float(a_log[h])) * float(dt[t, h])) * S + float(dt[t, h]) * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ Cm[t, g] + skip[h] * x[t, h]
    return y


def ssd_mixer(h, w, pre, m, eps):
    H, P, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    T = h.shape[0]
    proj = h @ w[pre + "in"].T
    z = proj[:, :inner]
    xbc = causal_conv_silu(proj[:, inner:2 * inner + 2 * G * N], w[pre + "conv"], w[pre + "conv.b"])
    dt = torch.nn.functional.softplus(proj[:, 2 * inner + 2 * G * N:] + w[pre + "dt_bias"], threshold=1e9)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    y = ssd_scan(x, B, Cm, dt, w[pre + "A_log"], w[pre + "D"], G).reshape(T, inner)
    y = y * silu(z)                                                   # the gate comes before the norm
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def chunk_sink_attention(q, k, v, chunk, scale, sink=True):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; position i sees j <= i of its own chunk (chunks counted from position 0);
    weights exp(s_j) / (1 + sum exp(s_j)): a sink with score 0 that carries no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        lo = (i // chunk) * chunk if chunk > 0 else 0
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * scale
            e = torch.exp(s)
            p = e / ((1.0 if sink else 0.0) + e.sum())
            out[i, hh] = p @ v[lo:i + 1, g]
    return out


def attn_mixer(h, w, pre, m, eps, sink=True, chunk_shift=0):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = h @ w[pre + "q"].T + w[pre + "q.b"]
    k = h @ w[pre + "k"].T + w[pre + "k.b"]
    v = h @ w[pre + "v"].T + w[pre + "v.b"]
    q = (rms(q, eps) * w[pre + "q.norm"]).reshape(T, H, d)            # over the whole projection, before the head split
    k = (rms(k, eps) * w[pre + "k.norm"]).reshape(T, G, d)
    o = chunk_sink_attention(q, k, v.reshape(T, G, dv), m["mask"]["size"] + chunk_shift, m["scale"], sink)
    o = o * torch.sigmoid(h @ w[pre + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[pre + "o"].T


def gla_scan(q, k, v, decay):
    """q, k, decay [T, H, d], v [T, H, dv]: S <- diag(decay_t) S + k_t v_t^T, o_t = S^T q_t."""
    T, H, d = q.shape
    o = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for hh in range(H):
        S = torch.zeros(d, v.shape[-1], dtype=F64)
        for t in range(T):
            S = decay[t, hh][:, None] * S + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S.T @ q[t, hh]
    return o


def gla_mixer(h, w, pre, m, eps):
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ w[pre + "q"].T * d ** -0.5).reshape(T, H, d)
    k = (h @ w[pre + "k"].T).reshape(T, H, d)
    v = (h @ w[pre + "v"].T).reshape(T, H, dv)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / tau).reshape(T, H, d)
    o = rms(gla_scan(q, k, v, decay), eps) * w[pre + "norm"]          # per head over dv, one weight for all heads
    o = o.reshape(T, H * dv) * silu(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps, **kw):
    left = attn_mixer(h, w, pre + "left.", m["left"], eps, **kw)
    right = gla_mixer(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[pre + "left.out"] + rms(right, eps) * w[pre + "right.out"])


def feed_forward(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def forward(cfg: dict, tensors: dict, tokens, **attn_kw):
    """-> (logits [T, vocab], residual stream after every layer [L, T, width]), float64."""
    w = {k: v.to(F64) for k, v in tensors.items()}
    eps, alpha, W = cfg["norm"]["eps"], cfg["postln_alpha"], cfg["width"]
    x = w["embed"][torch.tensor(list(tokens))] * cfg["embedding"]["scale"] + sinusoid(len(tokens), W)
    after = []
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        if L["type"] == "mamba2":
            mix = ssd_mixer(x, w, pre + "mix.", L["mixer"], eps)
        else:
            mix = parallel_mixer(x, w, pre + "mix.", L["mixer"], eps, **attn_kw)
        x = rms(alpha * x + mix, eps) * w[pre + "norm1"]
        if L["mlp"] is not None:
            x = rms(alpha * x + feed_forward(x, w, pre + "mlp."), eps) * w[pre + "norm2"]
        after.append(x)
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap") or 0.0
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(after)


def greedy(cfg: dict, tensors: dict, prompt, n_new: int):
    ids = list(prompt)
    for _ in range(n_new):
        lg, _ = forward(cfg, tensors, ids)
        ids.append(int(lg[-1].argmax()))
    return ids[len(prompt):]
