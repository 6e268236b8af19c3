"""Plain, slow implementation of the Tagelorn decoder, one function per
mechanism, for whole sequences on the CPU.  It shares no code with
``prism_b200``: weights come in as a dict of tensors keyed by the model file's
tensor names, the configuration as the raw ``config.json`` dict.  Everything
runs in the dtype of the weights handed in (float32 or float64).  ``rnd``,
where a function takes it, is applied to what a 16-bit engine may keep in 16
bits (the input of a matrix product, cached keys and values, queries, the
inner activations of a feed-forward); the default leaves everything as it is.

Notation: ``x [T, D]`` is one sequence, positions are ``0 .. T-1``; ``W`` are
stored ``[out, in]`` and applied as ``x @ W.T``.
"""

from __future__ import annotations

import math

import torch

UNIT_EPS = 1e-6
DECAY_RATE = math.exp(-0.5)
WEIGHT_SUM_EPS = 1e-20
SINUSOID_BASE = 10000.0


def _same(x):
    return x


# ---- small pieces -----------------------------------------------------------------

def rms(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu2(z):
    r = torch.relu(z)
    return r * r


def sinusoid(T, width, dtype):
    """``[T, width]``: entry 2i of row p is ``sin(p b^(-2i/width))``, entry 2i+1 the cosine."""
    out = torch.zeros(T, width, dtype=dtype)
    p = torch.arange(T, dtype=dtype)
    for c in range(width):
        f = SINUSOID_BASE ** (-(c - c % 2) / width)
        out[:, c] = torch.sin(p * f) if c % 2 == 0 else torch.cos(p * f)
    return out


def embed(tokens, table, scale):
    x = table[tokens] * scale
    return x + sinusoid(len(tokens), table.shape[1], table.dtype)


def input_conv(h, taps):
    """``h + conv(h)``, ``conv(h)[t] = sum_j taps[:, j] h[t - K + 1 + j]`` with zeros before the start."""
    T, K = h.shape[0], taps.shape[1]
    y = h.clone()
    for t in range(T):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += taps[:, j] * h[s]
    return y


# ---- attention -------------------------------------------------------------------

def distance_bucket(n: int, rows: int, far: int) -> int:
    """Distances below ``rows / 2`` have a row each; the others share the upper half in steps that grow like a
    logarithm and end at ``far``."""
    half = rows // 2
    if n < half:
        return n
    if half == 0 or far <= half:
        return rows - 1
    v = math.log(n / half) / math.log(far / half) * (rows - half)
    if abs(v - round(v)) < 1e-9:
        v = round(v)
    return min(rows - 1, half + int(math.floor(v)))


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def attention(h, w, p, mx, eps, rnd=_same):
    """Grouped-query attention: biases, q and k divided by their root mean square per head, a bias by distance, a window
    that keeps the first positions, a sink in the softmax's denominator."""
    T = h.shape[0]
    H, G, d = mx["heads"], mx.get("kv_heads") or mx["heads"], mx["dim"]
    dv = mx.get("vdim") or d
    size, keep = mx["mask"]["size"], mx["mask"].get("keep_first", 0)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q, k, v = rnd(rms(q, eps)), rnd(rms(k, eps)), rnd(v)
    rel, sink = w[p + "rel"], w[p + "sink"]
    rows = rel.shape[0]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, size, keep)]
            s = torch.stack([(q[i, hh] * k[j, g]).sum() * mx["scale"] + rel[distance_bucket(i - j, rows, mx["bias_max"]), hh]
                             for j in js])
            m = torch.maximum(s.max(), sink[hh])
            e = torch.exp(s - m)
            den = e.sum() + torch.exp(sink[hh] - m)
            out[i, hh] = ((e / den)[:, None] * v[js, g]).sum(0)
    return rnd(out.reshape(T, H * dv)) @ w[p + "o"].T


# ---- generalized delta rule ------------------------------------------------------------

def general_delta(h, w, p, mx, eps, rnd=_same):
    T = h.shape[0]
    H, d = mx["heads"], mx["dim"]
    r = (h @ w[p + "r"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, d)
    decay = torch.exp(-DECAY_RATE * torch.sigmoid(torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    a = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(T, H, d)
    gate = torch.sigmoid(h @ w[p + "g"].T)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_EPS)
    S = torch.zeros(H, d, d, dtype=h.dtype)              # [head, key channel, value channel]
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            old = S[hh]
            S[hh] = decay[t, hh][:, None] * old - (a[t, hh] * u[t, hh])[:, None] * (u[t, hh] @ old)[None, :] \
                + k[t, hh][:, None] * v[t, hh][None, :]
            o[t, hh] = S[hh].T @ r[t, hh]
    o = rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return rnd(o) @ w[p + "o"].T


# ---- feed-forward ---------------------------------------------------------------------

def dense_ff(h, w, p, rnd=_same):
    return rnd(gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(h, w, p, rnd=_same):
    return rnd(relu2(h @ w[p + "up"].T)) @ w[p + "down"].T


def route(z, correction, top, groups, keep, scale):
    """For one token's router logits: the chosen experts and their weights."""
    E = z.shape[0]
    s = torch.softmax(z, -1)
    c = s + correction
    per = E // groups
    best = sorted(range(groups), key=lambda g: (-float(c[g * per:(g + 1) * per].max()), g))[:keep]
    allowed = [e for e in range(E) if e // per in best]
    chosen = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
    wsum = sum(s[e] for e in chosen) + WEIGHT_SUM_EPS
    return chosen, [s[e] / wsum * scale for e in chosen]


def moe_ff(h, w, p, mlp, rnd=_same):
    T = h.shape[0]
    rt = mlp["router"]
    z = h @ w[p + "router"].T
    out = torch.zeros(T, w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(T):
        groups = rt.get("groups") or {}
        count = groups.get("count", 1)
        chosen, weights = route(z[t], w[p + "correction"], rt["top"], count, groups.get("keep", count), rt.get("scale", 1.0))
        for e, ww in zip(chosen, weights):
            out[t] += ww * expert(h[t:t + 1], w, f"{p}e{e}.", rnd)[0]
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.", rnd)
    return out


# ---- per-layer token input --------------------------------------------------------------

def token_side(x, tokens, w, i, dim, eps, rnd=_same):
    p = f"l{i}.side."
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(rnd(x) @ w[p + "gate"].T) * e
    y = rnd(g) @ w[p + "proj"].T
    return rms(y, eps) * w[p + "norm"]


# ---- the model ------------------------------------------------------------------------

def forward(cfg, w, tokens, rnd=_same, streams=None):
    """Logits ``[T, vocab]`` for one sequence.  ``streams``: a list that receives the residual rows after every layer."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = embed(tokens, w["embed"], (cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * w[p + "norm1"]
        h = rnd(input_conv(h, w[p + "canon1"]))
        if layer["type"] == "attention":
            x = x + attention(h, w, p + "mix.", layer["mixer"], eps, rnd)
        elif layer["type"] == "general_delta":
            x = x + general_delta(h, w, p + "mix.", layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rnd(rms(x, eps) * w[p + "norm2"])
            x = x + (dense_ff(h, w, p + "mlp.", rnd) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp, rnd))
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, w, i, cfg["token_side"]["dim"], eps, rnd)
        if streams is not None:
            streams.append(x.clone())
    h = rnd(rms(x, eps) * w["final.norm"])
    logits = h @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
