"""Plain, slow implementation of the Zuvulorn decoder, one function per
mechanism, for whole sequences on the CPU.  It shares no code with
``prism_b200``: weights come in as a dict of tensors keyed by the model file's
tensor names, the configuration as the raw ``config.json`` dict.  Everything
runs in the dtype of the weights handed in (float32 or float64).  ``rnd``, where a function takes it, is applied to
what a 16-bit engine may keep in 16 bits (a sublayer's input, cached keys and values, rotated queries, what enters an
output projection or an expert's second product); the default leaves everything as it is.

Notation: ``x [T, D]`` is one sequence, positions are ``0 .. T-1``; ``W`` are
stored ``[out, in]`` and applied as ``x @ W.T``.
"""

from __future__ import annotations

import math

import torch


# ---- norms and activations --------------------------------------------------

def layer_norm(x, weight, eps):
    """``(x - mean) / sqrt(var + eps) * weight`` over the last axis, var the mean squared deviation, no bias."""
    m = x.mean(-1, keepdim=True)
    d = x - m
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight


def rms(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_conv(x, taps, bias=None):
    """``y[t, c] = sum_j taps[c, K-1-j] x[t-j, c]`` (zeros before the start), plus ``bias[c]``."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        if j < T:
            y[j:] += x[:T - j] * taps[:, K - 1 - j]
    return y if bias is None else y + bias


# ---- positions ----------------------------------------------------------------

def band_frequencies(base, dims, scaling, dtype):
    """``f_i = base^(-2i/dims)``, i < dims/2, rescaled by wavelength ``l = 2 pi / f``: kept where ``l <
    original / high``, divided by ``factor`` where ``l > original / low``, blended linearly in between."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            l = 2.0 * math.pi / f
            if l > orig / low:
                f = f / factor
            elif l >= orig / high:
                s = (orig / l - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=dtype)


def rotate_halves(x, positions, freqs):
    """Entry i of the last axis of ``x [T, heads, d]`` is paired with entry ``i + n``, n = len(freqs); the pair
    (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i.  Entries from 2n on pass."""
    n = freqs.numel()
    if n == 0:
        return x.clone()
    ang = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., :n], x[..., n:2 * n]
    out = x.clone()
    out[..., :n] = u * c - v * s
    out[..., n:2 * n] = v * c + u * s
    return out


# ---- mixers -------------------------------------------------------------------

def same(x):
    return x


def attention_keys(h, w, p, m, eps, rnd=same):
    """Keys (normed over the whole projection, rotated) ``[T, G, dim]`` and values ``[T, G, vdim]`` of a layer."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = h @ w[p + "v"].T
    rot = m.get("rot") or {}
    freqs = band_frequencies(rot.get("base", 10000.0), rot.get("dims", 0), rot.get("scaling"), h.dtype)
    pos = torch.arange(T)
    return rnd(rotate_halves(k.view(T, G, dim), pos, freqs)), rnd(v.view(T, G, vdim))


def sink_softmax(scores):
    """``exp(s_j) / (1 + sum_j exp(s_j))`` over the last axis (masked entries are -inf)."""
    mx = torch.clamp(scores.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(scores - mx)
    return e / (torch.exp(-mx) + e.sum(-1, keepdim=True))


def attention(h, w, p, m, eps, kv=None, rnd=same):
    """Grouped-query causal attention with a sink of score 0, a per-head sigmoid gate; ``kv``: another layer's
    keys and values (this layer then has no key/value tensors)."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    rot = m.get("rot") or {}
    freqs = band_frequencies(rot.get("base", 10000.0), rot.get("dims", 0), rot.get("scaling"), h.dtype)
    q = rnd(rotate_halves(q.view(T, H, dim), torch.arange(T), freqs))
    k, v = kv if kv is not None else attention_keys(h, w, p, m, eps, rnd)
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~causal, float("-inf"))
        out[:, hh] = (sink_softmax(s) @ v[:, g]) * gate[:, hh:hh + 1]
    return rnd(out.reshape(T, H * vdim)) @ w[p + "o"].T, (k, v)


def rglru(h, w, p, m, rnd=same):
    """Recurrent block with a real-gated linear recurrent unit."""
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    bs = width // blocks
    ub = u.view(T, blocks, bs)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, width)
    a = torch.exp(-8.0 * r * softplus(w[p + "lam"]))
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(width, dtype=h.dtype)
    out = torch.zeros(T, width, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + b[t]
        out[t] = S
    return rnd(out * y) @ w[p + "o"].T


def channel_delta(h, w, p, m, eps, rnd=same):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                          # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).view(T, H, dk))   # [T, H, dk]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        kv = hh // (H // G)
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = g[t, hh][:, None] * S
            uu = beta[t, hh] * (v[t, hh] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], uu)
            out[t, hh] = S.T @ q[t, kv]
    out = rms(out, eps) * w[p + "norm"] * gate
    return rnd(out.reshape(T, H * dv)) @ w[p + "o"].T


# ---- feed-forward -------------------------------------------------------------

def moe(h, w, p, mlp, rnd=same):
    """Sigmoid-scored top-k experts; the score multiplies the chosen expert's input."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    chosen = torch.topk(s, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            x = rnd(s[t, e] * h[t])
            out[t] += rnd(silu(x @ w[f"{p}e{e}.gate"].T) * (x @ w[f"{p}e{e}.up"].T)) @ w[f"{p}e{e}.down"].T
    return out


# ---- the model ----------------------------------------------------------------

def hyper_step(xs, hc, w, sublayer):
    """One sublayer under hyper-connections: ``xs [s, T, D]`` -> new streams.  A model without connection weights
    keeps one stream: ``x <- x + sublayer(x)``."""
    if hc + "in" not in w:
        return xs + sublayer(xs[0])[None]
    u = torch.einsum("s,std->td", w[hc + "in"], xs)
    y = sublayer(u)
    return torch.einsum("sr,std->rtd", w[hc + "mix"], xs) + w[hc + "out"][:, None, None] * y[None]


def forward(cfg, w, tokens, return_layers=False, rnd=same):
    """Logits ``[T, vocab]`` of one sequence; with ``return_layers`` also the sum of the streams after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    xs = x[None].repeat(cfg.get("streams") or 1, 1, 1)
    kvs, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]

        def mixer(u):
            hn = rnd(layer_norm(u, w[p + "norm1"], eps))
            if layer["type"] == "attention":
                src = m.get("kv_from")
                y, kv = attention(hn, w, p + "mix.", m, eps, None if src is None else kvs[src], rnd)
                kvs[i] = kv
                return y
            if layer["type"] == "rglru":
                return rglru(hn, w, p + "mix.", m, rnd)
            if layer["type"] == "channel_delta":
                return channel_delta(hn, w, p + "mix.", m, eps, rnd)
            raise ValueError(layer["type"])

        xs = hyper_step(xs, p + "hc1.", w, mixer)
        if layer.get("mlp") is not None:
            xs = hyper_step(xs, p + "hc2.", w, lambda u: moe(rnd(layer_norm(u, w[p + "norm2"], eps)), w, p + "mlp.", layer["mlp"], rnd))
        after.append(xs.sum(0))
    logits = rnd(layer_norm(xs.sum(0), w["final.norm"], eps)) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
