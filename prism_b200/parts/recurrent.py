"""Recurrent mixers: their memory of a sequence is a float32 matrix per head
in a state slot of the request, not a cache of keys, so a step costs the same
at any position.  Everything that enters the recurrences is float32 (the
input projections give float32 results; decays, gates and unit vectors are
formed in float32 by the kernels of ``csrc/recurrent.cu``); what leaves for
the output projection is rounded to the compute dtype once.

``gated_delta``: delta rule with a scalar decay per head and token, behind a
short causal convolution over time of q, k and v.
``wkv``: token-shift mixes of the input, a per-channel decay from a low-rank
product, and a bonus for the current token in the read-out.
``channel_delta``: the delta rule with one decay per key channel, from a
low-rank product, and a low-rank sigmoid gate on the read-out.
``general_delta``: the generalized delta rule: a decay and a removal rate per
key channel; what is removed is read along the unit key.
``rglru``: a recurrence with one number of state per channel whose gates are
block-diagonal products, behind a short convolution, beside a gelu branch.
``sum``: several mixers side by side on the same input, their results scaled
and added (one joint input product and one joint output product where the
mixers can hand theirs over).
"""

from __future__ import annotations

import os
from typing import Optional, Sequence

import torch

from ..config.model_config import ConfigError
from .base import CacheNeed, DetachedProjection, Mixer, ParamSpec, PartSpec, WeightSource, build_part, register_part
from .. import ops


@register_part("mixer", "gated_delta")
class GatedDeltaMixer(Mixer):
    """With h the input, per token (``G = num_kv_heads`` q/k heads of ``head_dim``, ``H = num_heads`` value heads of
    ``v_head_dim``; head i uses q/k head ``i // (H / G)``)::

        q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     conv: causal over time, per channel
        q <- q / sqrt(sum q^2 + unit_eps) / sqrt(head_dim);   k <- k / sqrt(sum k^2 + unit_eps)      per head
        beta = sigmoid(W_b h);   g = exp(-exp(A_log) softplus(W_a h + dt_bias))                     per head
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                              per head
        out = W_o [o / rms(o) * norm * silu(W_g h)]

    State per request: S ``[H, v_head_dim, head_dim]`` (stored column by column) and the convolution's last
    ``conv - 1`` inputs ``[conv - 1, channels]``, both float32, both starting at zero.  ``names``: the tensors'
    names in the model file (keys q, k, v, q_conv, k_conv, v_conv, b, a, A_log, dt_bias, g, norm, o)."""

    NAMES = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", q_conv="q_conv.weight", k_conv="k_conv.weight",
                 v_conv="v_conv.weight", b="b_proj.weight", a="a_proj.weight", A_log="A_log", dt_bias="dt_bias",
                 g="g_proj.weight", norm="norm.weight", o="o_proj.weight")
    graph_safe = True            # works from the device's slot array alone
    float32_projection = True
    detachable_out = detachable_in = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, conv: int,
                 eps: float, unit_eps: float = 1e-6, out_scale: float = 1.0, names: Optional[dict] = None):
        self.hidden_size, self.H, self.G = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv, self.K = int(head_dim), int(v_head_dim), int(conv)
        if min(self.H, self.G, self.dk, self.dv, self.K) < 1 or self.H % self.G:
            raise ConfigError(f"gated delta mixer: heads {self.H} must be a multiple of kv_heads {self.G}, and heads, "
                              f"sizes and the convolution's taps positive")
        if self.dk > 1024:
            raise ConfigError(f"gated delta mixer: head_dim {self.dk} exceeds the scan kernel's 1024")
        self.eps, self.unit_eps, self.out_scale = float(eps), float(unit_eps), float(out_scale)
        self.names = dict(self.NAMES, **(names or {}))
        self.C = 2 * self.G * self.dk + self.H * self.dv          # channels of the convolution: q | k | v
        self.b_off, self.a_off, self.g_off = self.C, self.C + self.H, self.C + 2 * self.H
        self.in_width = self.C + 2 * self.H + self.H * self.dv    # q | k | v | b | a | g
        self._own_in = self._own_out = True

    def cache_needs(self):
        return (CacheNeed("state", state_shape=(self.H, self.dv, self.dk)),
                CacheNeed("state", state_shape=(self.K - 1, self.C)))

    def _in_sources(self):
        W, n, G, H, dk, dv = self.hidden_size, self.names, self.G, self.H, self.dk, self.dv
        return (WeightSource(n["q"], (G * dk, W)), WeightSource(n["k"], (G * dk, W)), WeightSource(n["v"], (H * dv, W)),
                WeightSource(n["b"], (H, W)), WeightSource(n["a"], (H, W)), WeightSource(n["g"], (H * dv, W)))

    def _out_source(self):
        return WeightSource(self.names["o"], (self.hidden_size, self.H * self.dv))

    def params(self):
        n, G, H, dk, dv, K = self.names, self.G, self.H, self.dk, self.dv, self.K
        ps = [ParamSpec("in_w", self._in_sources())] if self._own_in else []
        ps += [ParamSpec("taps", (WeightSource(n["q_conv"], (G * dk, K)), WeightSource(n["k_conv"], (G * dk, K)),
                                  WeightSource(n["v_conv"], (H * dv, K)))),
               ParamSpec("A_log", (WeightSource(n["A_log"], (H,), "bias"),)),
               ParamSpec("dt_bias", (WeightSource(n["dt_bias"], (H,), "bias"),)),
               ParamSpec("norm", (WeightSource(n["norm"], (dv,), "norm"),))]
        if self._own_out:
            ps.append(ParamSpec("o_w", (self._out_source(),)))
        return ps

    def detach_out_projection(self):
        self._own_out = False
        return DetachedProjection(self.handed_over(self._out_source()), (), self.H * self.dv)

    def detach_in_projection(self):
        self._own_in = False
        return DetachedProjection(self.handed_over(*self._in_sources()), (), self.in_width, float32=True)

    def forward_inner(self, ctx, x, cache, out, proj=None):
        state, tail = cache
        T, H, G, dk, dv = x.shape[0], self.H, self.G, self.dk, self.dv
        if proj is None:
            proj = ops.linear(x, self.w["in_w"], None, out_dtype=torch.float32)
        qkv = ctx.alloc((T, self.C), torch.float32)
        bg = ctx.alloc((T, 2 * H), torch.float32)
        single = ctx.decode_only          # one token per request: the kernel that reads the tail also moves it up
        ops.conv_unit_gates(proj, self.b_off, self.a_off, self.w["taps"], tail.state, self.w["A_log"], self.w["dt_bias"],
                            ctx, G, H, dk, dv, self.unit_eps, qkv, bg, move_tail=single)
        if not single:
            ops.state_tail(proj, tail.state, ctx)
        o = ctx.alloc((T, H, dv), torch.float32)
        ops.recurrent_scan(ops.SCAN_DELTA, qkv[:, :G * dk], qkv[:, G * dk:2 * G * dk], qkv[:, 2 * G * dk:], state.state, ctx,
                           H, H // G, dk, dv, o, bg=bg)
        ops.headnorm_gate(o, proj[:, self.g_off:self.g_off + H * dv], self.w["norm"], self.eps, self.out_scale, out)

    def forward(self, ctx, x, cache):
        inner = ctx.alloc((x.shape[0], self.H * self.dv), ctx.dtype)
        self.forward_inner(ctx, x, cache, inner)
        return ops.linear_delta(inner, self.w["o_w"], None, f32=True)


@register_part("mixer", "channel_delta")
class ChannelDeltaMixer(Mixer):
    """The gated delta rule with a decay of its own for every key channel.  With h the input, per token (``G =
    num_kv_heads`` q/k heads of ``head_dim``, ``H = num_heads`` value heads of ``v_head_dim``; head i uses q/k head
    ``i // (H / G)``)::

        q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     conv: causal over time, per channel
        q <- q / sqrt(sum q^2 + unit_eps) / sqrt(head_dim);   k <- k / sqrt(sum k^2 + unit_eps)      per head
        beta = sigmoid(W_b h)                                                                        per head
        w = exp(-exp(A_log) softplus(W_a2 (W_a1 h) + dt_bias))            per head and key channel, A_log per head
        S <- diag(w) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                           per head
        out = W_o [o / rms(o) * norm * sigmoid(W_g2 (W_g1 h))]

    State per request: S ``[H, v_head_dim, head_dim]`` (stored column by column) and the convolution's last
    ``conv - 1`` inputs, both float32, both starting at zero.  The second halves of the two low-rank products run in
    float32 with their epilogues (softplus and exponential; sigmoid) in the same launch.  ``names``: keys q, k, v,
    q_conv, k_conv, v_conv, b, a1, a2, A_log, dt_bias, g1, g2, norm, o."""

    NAMES = dict(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", b="b", a1="a1", a2="a2",
                 A_log="A_log", dt_bias="dt_bias", g1="g1", g2="g2", norm="norm", o="o")
    graph_safe = True
    float32_projection = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, conv: int,
                 decay_rank: int, gate_rank: int, eps: float, unit_eps: float = 1e-6, out_scale: float = 1.0,
                 names: Optional[dict] = None):
        self.hidden_size, self.H, self.G = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv, self.K = int(head_dim), int(v_head_dim), int(conv)
        self.Ra, self.Rg = int(decay_rank), int(gate_rank)
        if min(self.H, self.G, self.dk, self.dv, self.K, self.Ra, self.Rg) < 1 or self.H % self.G:
            raise ConfigError(f"channel delta mixer: heads {self.H} must be a multiple of kv_heads {self.G}, and heads, "
                              f"sizes, ranks and the convolution's taps positive")
        if self.dk > 1024:
            raise ConfigError(f"channel delta mixer: head_dim {self.dk} exceeds the scan kernel's 1024")
        self.eps, self.unit_eps, self.out_scale = float(eps), float(unit_eps), float(out_scale)
        self.names = dict(self.NAMES, **(names or {}))
        self.C = 2 * self.G * self.dk + self.H * self.dv          # channels of the convolution: q | k | v
        self.b_off, self.a_off, self.g_off = self.C, self.C + self.H, self.C + self.H + self.Ra
        self.in_width = self.C + self.H + self.Ra + self.Rg       # q | k | v | b | a1 | g1

    def cache_needs(self):
        return (CacheNeed("state", state_shape=(self.H, self.dv, self.dk)),
                CacheNeed("state", state_shape=(self.K - 1, self.C)))

    def params(self):
        W, n, G, H, dk, dv, K = self.hidden_size, self.names, self.G, self.H, self.dk, self.dv, self.K
        return [ParamSpec("in_w", (WeightSource(n["q"], (G * dk, W)), WeightSource(n["k"], (G * dk, W)),
                                   WeightSource(n["v"], (H * dv, W)), WeightSource(n["b"], (H, W)),
                                   WeightSource(n["a1"], (self.Ra, W)), WeightSource(n["g1"], (self.Rg, W)))),
                ParamSpec("taps", (WeightSource(n["q_conv"], (G * dk, K)), WeightSource(n["k_conv"], (G * dk, K)),
                                   WeightSource(n["v_conv"], (H * dv, K)))),
                ParamSpec("a2", (WeightSource(n["a2"], (H * dk, self.Ra)),)),
                ParamSpec("g2", (WeightSource(n["g2"], (H * dv, self.Rg)),)),
                ParamSpec("A_log", (WeightSource(n["A_log"], (H,), "bias"),)),
                ParamSpec("dt_bias", (WeightSource(n["dt_bias"], (H * dk,), "bias"),)),
                ParamSpec("norm", (WeightSource(n["norm"], (dv,), "norm"),)),
                ParamSpec("o_w", (WeightSource(n["o"], (W, H * dv)),))]

    def on_bound(self):
        # the second halves run in float32 whatever the engine's dtype; transposed, so that the kernel's neighbouring
        # threads read neighbouring floats
        self.a2t = self.w["a2"].float().t().contiguous() if self.w["a2"] is not None else None
        self.g2t = self.w["g2"].float().t().contiguous() if self.w["g2"] is not None else None

    def forward(self, ctx, x, cache):
        state, tail = cache
        T, H, G, dk, dv = x.shape[0], self.H, self.G, self.dk, self.dv
        proj = ops.linear(x, self.w["in_w"], None, out_dtype=torch.float32)
        qkv = ctx.alloc((T, self.C), torch.float32)
        beta = ctx.alloc((T, H), torch.float32)
        single = ctx.decode_only          # one token per request: the kernel that reads the tail also moves it up
        ops.conv_unit_gates(proj, self.b_off, 0, self.w["taps"], tail.state, None, None, ctx, G, H, dk, dv, self.unit_eps,
                            qkv, beta, move_tail=single)
        if not single:
            ops.state_tail(proj, tail.state, ctx)
        ww = ctx.alloc((T, H * dk), torch.float32)
        ops.lowrank_decay(proj[:, self.a_off:self.a_off + self.Ra], self.a2t, self.w["dt_bias"], ww, inner_tanh=False,
                          epilogue=ops.LR_SOFTPLUS, rate_log=self.w["A_log"], per=dk)
        gate = ctx.alloc((T, H * dv), torch.float32)
        ops.lowrank_decay(proj[:, self.g_off:self.g_off + self.Rg], self.g2t, None, gate, inner_tanh=False,
                          epilogue=ops.LR_SIGMOID)
        o = ctx.alloc((T, H, dv), torch.float32)
        ops.recurrent_scan(ops.SCAN_CHANNEL, qkv[:, :G * dk], qkv[:, G * dk:2 * G * dk], qkv[:, 2 * G * dk:], state.state, ctx,
                           H, H // G, dk, dv, o, bg=beta, ww=ww)
        inner = ctx.alloc((T, H * dv), ctx.dtype)
        ops.headnorm_gate(o, gate, self.w["norm"], self.eps, self.out_scale, inner, gate_act="none")
        return ops.linear_delta(inner, self.w["o_w"], None, f32=True)


@register_part("mixer", "general_delta")
class GeneralDeltaMixer(Mixer):
    """The generalized delta rule: a decay and a removal rate of their own for every key channel.  With h the input,
    per token and head (``num_heads`` heads of ``head_dim`` key and value channels)::

        r, k, v = W_r h, W_k h, W_v h
        w = exp(-decay_rate sigmoid(W_w2 tanh(W_w1 h) + w0))            per key channel: a decay in (exp(-decay_rate), 1)
        a = sigmoid(W_a h + a_b)                                        per key channel: a removal rate
        e = k / sqrt(sum k^2 + unit_eps)                                the unit key
        S <- diag(w) S - (a * e) (e^T S) + k v^T;   o = S^T r           both corrections read the state before the token
        out = W_o [o / rms(o) * norm * sigmoid(W_g h)]

    State per request: S ``[H, head_dim, head_dim]`` (stored column by column), float32, starting at zero.  All input
    projections are one product with float32 results; the decay's second, rank-sized product runs in float32 with
    its epilogue in the same launch; unit key, removal, state, head norm and gate are float32.  The decay's rank
    is the shape of ``w1``.  ``names``: keys r, k, v, g, a, a_b, w1, w2, w0, norm, o."""

    NAMES = dict(r="r", k="k", v="v", g="g", a="a", a_b="a.b", w1="w1", w2="w2", w0="w0", norm="norm", o="o")
    graph_safe = True
    float32_projection = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int, eps: float, decay_rate: float,
                 unit_eps: float = 1e-6, out_scale: float = 1.0, names: Optional[dict] = None):
        self.hidden_size, self.H, self.d, self.rank = int(hidden_size), int(num_heads), int(head_dim), int(decay_rank)
        if min(self.H, self.d, self.rank) < 1 or self.d > 1024:
            raise ConfigError("general delta mixer: heads, head size and the decay's rank must be positive, the head size "
                              "at most 1024")
        self.eps, self.unit_eps, self.out_scale = float(eps), float(unit_eps), float(out_scale)
        self.decay_rate = float(decay_rate)
        self.names = dict(self.NAMES, **(names or {}))

    def cache_needs(self):
        return (CacheNeed("state", state_shape=(self.H, self.d, self.d)),)

    def cache_need(self):
        return self.cache_needs()[0]

    def params(self):
        W, n, A, R = self.hidden_size, self.names, self.H * self.d, self.rank
        return [ParamSpec("in_w", tuple(WeightSource(n[s], (A, W)) for s in "rkvga") + (WeightSource(n["w1"], (R, W)),)),
                ParamSpec("a_b", (WeightSource(n["a_b"], (A,), "bias"),)),
                ParamSpec("w2", (WeightSource(n["w2"], (A, R)),)),
                ParamSpec("w0", (WeightSource(n["w0"], (A,), "bias"),)),
                ParamSpec("norm", (WeightSource(n["norm"], (A,), "norm"),)),
                ParamSpec("o_w", (WeightSource(n["o"], (W, A)),))]

    def on_bound(self):
        # the decay's second product runs in float32 whatever the engine's dtype (its input is the float32 tanh);
        # transposed, so that the kernel's neighbouring threads read neighbouring floats
        self.w2t = self.w["w2"].float().t().contiguous() if self.w["w2"] is not None else None

    def forward(self, ctx, x, cache):
        state = cache[0] if isinstance(cache, tuple) else cache
        T, H, d, A = x.shape[0], self.H, self.d, self.H * self.d
        proj = ops.linear(x, self.w["in_w"], None, out_dtype=torch.float32)          # r | k | v | g | a | w1
        r, k, v, g, a = (proj[:, i * A:(i + 1) * A] for i in range(5))
        low = proj[:, 5 * A:]
        ww = ctx.alloc((T, A), torch.float32)
        ops.lowrank_decay(low, self.w2t, self.w["w0"], ww, epilogue=ops.LR_EXPSIG, rate=self.decay_rate)
        ex = ctx.alloc((T, 2 * A), torch.float32)
        ops.unit_removal(k, a, self.w["a_b"], self.unit_eps, H, d, ex)
        o = ctx.alloc((T, H, d), torch.float32)
        ops.recurrent_scan(ops.SCAN_GENERAL, r, k, v, state.state, ctx, H, 1, d, d, o, ww=ww, ex=ex)
        inner = ctx.alloc((T, A), ctx.dtype)
        ops.headnorm_gate(o, g, self.w["norm"], self.eps, self.out_scale, inner, gate_act="sigmoid")
        return ops.linear_delta(inner, self.w["o_w"], None, f32=True)


@register_part("mixer", "rglru")
class RGLRUMixer(Mixer):
    """A recurrent block around a real-gated linear recurrent unit.  With h the input and two branches of
    ``width`` channels::

        y = gelu_tanh(W_y h + b_y);    u = conv(W_x h + b_x) + b_conv          conv: causal over time, per channel
        r = sigmoid(Wr[b] u_b + br[b]);  i = sigmoid(Wi[b] u_b + bi[b])         per block b of width / blocks channels
        a = exp(-decay_scale r softplus(lam));   S <- a S + sqrt(1 - a^2) i u   per channel, S = 0 before the first token
        out = W_o (S y)

    State per request: S ``[width]`` and the convolution's last ``conv - 1`` inputs, float32, starting at zero.
    Both branches come from one product with float32 results; the gates, the coefficients and the recurrence are
    float32 (``csrc/rglru.cu``).  ``names``: keys y, y_b, x, x_b, conv, conv_b, ra, ra_b, ri, ri_b, lam, o."""

    NAMES = dict(y="y", y_b="y.b", x="x", x_b="x.b", conv="conv", conv_b="conv.b", ra="ra", ra_b="ra.b", ri="ri",
                 ri_b="ri.b", lam="lam", o="o")
    graph_safe = True

    def __init__(self, hidden_size: int, width: int, blocks: int, conv: int, decay_scale: float = 8.0,
                 names: Optional[dict] = None):
        self.hidden_size, self.C, self.blocks, self.K = int(hidden_size), int(width), int(blocks), int(conv)
        if min(self.C, self.blocks, self.K) < 1 or self.C % self.blocks:
            raise ConfigError(f"rglru mixer: width {self.C} must be a multiple of blocks {self.blocks}, and the "
                              f"convolution's taps positive")
        self.bs, self.decay_scale = self.C // self.blocks, float(decay_scale)
        self.names = dict(self.NAMES, **(names or {}))

    def cache_needs(self):
        return (CacheNeed("state", state_shape=(self.C,)), CacheNeed("state", state_shape=(self.K - 1, self.C)))

    def params(self):
        W, C, n, nb, bs = self.hidden_size, self.C, self.names, self.blocks, self.bs
        return [ParamSpec("in_w", (WeightSource(n["y"], (C, W)), WeightSource(n["x"], (C, W)))),
                ParamSpec("in_b", (WeightSource(n["y_b"], (C,), "bias"), WeightSource(n["x_b"], (C,), "bias"))),
                ParamSpec("taps", (WeightSource(n["conv"], (C, self.K)),)),
                ParamSpec("conv_b", (WeightSource(n["conv_b"], (C,), "bias"),)),
                ParamSpec("ra", (WeightSource(n["ra"], (nb, bs, bs)),)),
                ParamSpec("ri", (WeightSource(n["ri"], (nb, bs, bs)),)),
                ParamSpec("ra_b", (WeightSource(n["ra_b"], (nb, bs), "bias"),)),
                ParamSpec("ri_b", (WeightSource(n["ri_b"], (nb, bs), "bias"),)),
                ParamSpec("lam", (WeightSource(n["lam"], (C,), "bias"),)),
                ParamSpec("o_w", (WeightSource(n["o"], (W, C)),))]

    def forward(self, ctx, x, cache):
        state, tail = cache
        T, C = x.shape[0], self.C
        proj = ops.linear(x, self.w["in_w"], self.w["in_b"], out_dtype=torch.float32)      # y | x
        xb = proj[:, C:]
        u = ctx.alloc((T, C), torch.float32)
        single = ctx.decode_only
        ops.causal_conv(xb, self.w["taps"], self.w["conv_b"], tail.state, ctx, u, move_tail=single)
        if not single:
            ops.state_tail(xb, tail.state, ctx)
        ag = ctx.alloc((2, T, C), torch.float32)
        ops.block_gates(u, self.w["ra"], self.w["ri"], self.w["ra_b"], self.w["ri_b"], self.w["lam"], self.decay_scale,
                        ag[0], ag[1])
        inner = ctx.alloc((T, C), ctx.dtype)
        ops.rglru_scan(ag[0], ag[1], proj[:, :C], state.state, ctx, inner, gelu=True)
        return ops.linear_delta(inner, self.w["o_w"], None, f32=True)


@register_part("mixer", "wkv")
class WKVMixer(Mixer):
    """With x the input and x' the previous token's input (zeros before the first token), ``mix_s = x + (x' - x)
    mu_s`` for s in r, k, v, g, w; per head of ``head_dim`` channels::

        r, k, v = W_r mix_r, W_k mix_k, W_v mix_v;   gate = silu(W_g mix_g)
        w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))                         per key channel
        o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T              u: a bonus for the current token only
        out = W_o [o / rms(o) * norm * gate]

    State per request: S ``[H, head_dim, head_dim]`` and the previous token's input ``[1, hidden]``, float32,
    starting at zero.  The mixes are formed from the float32 input rows.  ``names``: keys mu_r, mu_k, mu_v, mu_g,
    mu_w, r, k, v, g, w1, w2, w0, u, norm, o."""

    NAMES = dict(mu_r="mu.r", mu_k="mu.k", mu_v="mu.v", mu_g="mu.g", mu_w="mu.w", r="r", k="k", v="v", g="g", w1="w1",
                 w2="w2", w0="w0", u="u", norm="norm", o="o")
    graph_safe = True
    reads_float32 = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int, eps: float,
                 out_scale: float = 1.0, names: Optional[dict] = None):
        self.hidden_size, self.H, self.d, self.rank = int(hidden_size), int(num_heads), int(head_dim), int(decay_rank)
        if min(self.H, self.d, self.rank) < 1 or self.d > 1024:
            raise ConfigError("wkv mixer: heads, head size and the decay's rank must be positive, the head size at most 1024")
        self.eps, self.out_scale = float(eps), float(out_scale)
        self.names = dict(self.NAMES, **(names or {}))

    def cache_needs(self):
        return (CacheNeed("state", state_shape=(self.H, self.d, self.d)),
                CacheNeed("state", state_shape=(1, self.hidden_size)))

    def params(self):
        W, n, A, R = self.hidden_size, self.names, self.H * self.d, self.rank
        return [ParamSpec("mu", tuple(WeightSource(n["mu_" + s], (W,), "bias") for s in "rkvgw")),
                # r | k | v | g | the decay's first product: one matrix, each block of rows applied to its own mix
                ParamSpec("in_w", tuple(WeightSource(n[s], (A, W)) for s in "rkvg") + (WeightSource(n["w1"], (R, W)),)),
                ParamSpec("w2", (WeightSource(n["w2"], (A, R)),)),
                ParamSpec("w0", (WeightSource(n["w0"], (A,), "bias"),)),
                ParamSpec("u", (WeightSource(n["u"], (self.H, self.d), "bias"),)),
                ParamSpec("norm", (WeightSource(n["norm"], (A,), "norm"),)),
                ParamSpec("o_w", (WeightSource(n["o"], (W, A)),))]

    def on_bound(self):
        # the decay's second product runs in float32 whatever the engine's dtype (its input is the float32 tanh);
        # transposed, so that the kernel's neighbouring threads read neighbouring floats
        self.w2t = self.w["w2"].float().t().contiguous() if self.w["w2"] is not None else None
        self.mu = self.w["mu"].view(5, self.hidden_size)

    def forward(self, ctx, x, cache):
        state, prev = cache
        T, W, H, d, A = x.shape[0], self.hidden_size, self.H, self.d, self.H * self.d
        if x.dtype != torch.float32:
            x = x.float()
        mixes = ctx.alloc((5, T, W), ctx.dtype)
        ops.shift_mix(x, prev.state, self.mu, ctx, mixes, keep_prev=ctx.decode_only)
        if not ctx.decode_only:
            ops.state_tail(x, prev.state, ctx)
        # float32 r, k, v, g and the decay's first product, each from its own mix
        r, k, v, g, low = ops.linear_grouped(mixes, self.w["in_w"], (A, A, A, A, self.rank), torch.float32)
        # tanh, the second product, the offset and both exponentials in one launch: the decay of every key channel
        ww = ctx.alloc((T, A), torch.float32)
        ops.lowrank_decay(low, self.w2t, self.w["w0"], ww)
        o = ctx.alloc((T, H, d), torch.float32)
        ops.recurrent_scan(ops.SCAN_BONUS, r, k, v, state.state, ctx, H, 1, d, d, o,
                           ww=ww, w0=self.w["w0"], u=self.w["u"], decay_ready=True)
        inner = ctx.alloc((T, A), ctx.dtype)
        ops.headnorm_gate(o, g, self.w["norm"], self.eps, self.out_scale, inner)
        return ops.linear_delta(inner, self.w["o_w"], None, f32=True)


@register_part("mixer", "sum")
class SumOfMixers(Mixer):
    """``sum_i scale_i * mixer_i(h)``: mixers side by side on the same input.  ``prefixes``: each mixer's tensors
    sit under its own prefix inside this part's.  Where every mixer hands over its output projection, the sum is
    one product over the joined inner outputs, ``[a_1 | a_2 | ..] @ [W_o1 | W_o2 | ..]^T`` with each scale folded
    into its ``a_i``, so the results are added in the product's float32 accumulator; where every mixer also hands
    over its input projection, those are one product too (float32 results if any of them wants that).  ``fuse``
    False: every mixer runs on its own and the float32 results are added.

    Between the two joint products the mixers do not depend on one another, and each is a chain of small kernels,
    so the second and later ones run on streams of their own beside the first (forked after the input product,
    joined before the output product; inside a captured graph they become parallel branches).
    ``PRISM_MIXER_STREAMS=0`` keeps them on one stream."""

    graph_safe = True
    SIDE_STREAMS = os.environ.get("PRISM_MIXER_STREAMS", "1") != "0"
    _streams = {}            # (device, i) -> stream of the i-th mixer beside the first

    def __init__(self, mixers: Sequence[PartSpec], scales: Sequence[float], fuse: bool = True):
        if len(mixers) != len(scales) or not mixers:
            raise ConfigError("a sum of mixers needs one scale for each mixer")
        self.scales = [float(s) for s in scales]
        self.mixers = [self.add_child(f"m{i}", build_part("mixer", spec)) for i, spec in enumerate(mixers)]
        self.n_needs = [len(m.cache_needs()) for m in self.mixers]
        self.outs = self.ins = None
        if fuse and all(m.detachable_out for m in self.mixers):
            for m, s in zip(self.mixers, self.scales):
                m.out_scale = s
            self.outs = [m.detach_out_projection() for m in self.mixers]
            if any(d.biases for d in self.outs):
                raise ConfigError("a fused sum of mixers takes output projections without bias")
            if all(m.detachable_in for m in self.mixers):
                self.ins = [m.detach_in_projection() for m in self.mixers]
                if any(d.biases for d in self.ins):
                    raise ConfigError("a fused sum of mixers takes input projections without bias")
        self.reads_float32 = False

    def cache_needs(self):
        return tuple(n for m in self.mixers for n in m.cache_needs())

    def params(self):
        ps = []
        if self.ins is not None:
            ps.append(ParamSpec("in_w", tuple(w for d in self.ins for w in d.weights)))
        if self.outs is not None:
            ps.append(ParamSpec("out_w", tuple(w for d in self.outs for w in d.weights), axis=1))
        return ps

    def _caches(self, cache):
        views = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        out, o = [], 0
        for n in self.n_needs:
            out.append(None if n == 0 else (views[o] if n == 1 else tuple(views[o:o + n])))
            o += n
        return out

    def forward(self, ctx, x, cache):
        caches = self._caches(cache)
        T = x.shape[0]
        if self.outs is None:
            total = None
            for m, s, c in zip(self.mixers, self.scales, caches):
                d = m.forward(ctx, x, c)
                d = (d if d.dim() == 2 else d.sum(0)).float() * s
                total = d if total is None else total.add_(d)
            return total
        inner = ctx.alloc((T, sum(d.width for d in self.outs)), ctx.dtype)
        projs = [None] * len(self.mixers)
        if self.ins is not None:
            f32 = any(d.float32 for d in self.ins)
            proj = ops.linear(x, self.w["in_w"], None, out_dtype=torch.float32 if f32 else None)
            o = 0
            for i, d in enumerate(self.ins):
                projs[i] = proj[:, o:o + d.width]
                o += d.width
        offs, o = [], 0
        for d in self.outs:
            offs.append(o)
            o += d.width
        work = list(zip(self.mixers, self.outs, caches, projs, offs))
        if self.SIDE_STREAMS and len(work) > 1:
            main = torch.cuda.current_stream(x.device)
            fork = torch.cuda.Event()
            fork.record(main)
            sides = []
            for i, (m, d, c, p, at) in enumerate(work[1:]):
                side = self._streams.get((x.device, i))
                if side is None:
                    side = self._streams[(x.device, i)] = torch.cuda.Stream(device=x.device)
                side.wait_event(fork)
                with torch.cuda.stream(side):
                    m.forward_inner(ctx, x, c, inner[:, at:at + d.width], p)
                sides.append(side)
            m, d, c, p, at = work[0]
            m.forward_inner(ctx, x, c, inner[:, at:at + d.width], p)
            for side in sides:
                main.wait_stream(side)
        else:
            for m, d, c, p, at in work:
                m.forward_inner(ctx, x, c, inner[:, at:at + d.width], p)
        return ops.linear_delta(inner, self.w["out_w"], None, f32=True)
