"""Arrangements of parts into a layer.  ``prenorm``: andre-fu/prism's decoder
layer (engine/executor.py:106-127): norm, mixer, residual add, norm,
feed-forward, residual add.  Each residual add is carried out by the norm
that follows it (the next block's first norm, or the final norm).  Options:
a short causal convolution beside a skip path on what the mixer reads, no
feed-forward, a per-layer token input after the feed-forward.
``parallel``: one norm whose output both the mixer and the feed-forward read;
their two results are added to the residual stream together.
``postnorm``: the residual stream itself is normed after every sum,
``x <- norm(alpha x + sublayer(x))``, and the sublayers read x as it is.
``hyper``: pre-norm sublayers around a residual stream kept in several
copies, with learned weights for reading it and for writing back."""

from __future__ import annotations

from typing import Optional

from .base import Block, CacheNeed, ParamSpec, PartSpec, StreamUpdate, WeightSource, build_part, register_part
from .. import ops


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))``, each sum carried out by the norm that follows it.

    ``feed_forward`` None: the layer ends after its mixer.  ``input_conv`` K: what the mixer reads is ``h + conv(h)``
    with h the normed rows and ``conv`` a causal convolution over time of K taps on each channel (tensor
    ``conv_tensor`` ``[width, K]``, no bias, zeros before the sequence's start); the last ``K - 1`` normed rows of a
    request are state of the layer, in a slot (float32), so a prompt may be cut anywhere.  h is formed and
    convolved in float32 and rounded once.  ``token_side``: a per-layer token input after the feed-forward,

        e = table[token][index * dim : (index + 1) * dim];   g = act(W_gate x) * e;   y = W_proj g
        x <- x + y / sqrt(mean(y^2) + eps) * norm

    with x the residual rows themselves (after the feed-forward's sum) and ``table`` the embedding's per-token side
    table; arguments ``dim, index, eps, activation`` and ``names`` (keys gate, proj, norm)."""

    SIDE_NAMES = dict(gate="side.gate", proj="side.proj", norm="side.norm")

    def __init__(self, mixer: PartSpec, feed_forward: Optional[PartSpec], mixer_norm: PartSpec, ff_norm: Optional[PartSpec],
                 hidden_size: Optional[int] = None, input_conv: Optional[int] = None, conv_tensor: str = "conv",
                 token_side: Optional[dict] = None):
        self.mixer_norm = self.add_child("mixer_norm", build_part("norm", mixer_norm))
        self.mixer = self.add_child("mixer", build_part("mixer", mixer))
        self.ff_norm = self.add_child("ff_norm", build_part("norm", ff_norm)) if feed_forward is not None else None
        self.feed_forward = (self.add_child("feed_forward", build_part("feed_forward", feed_forward))
                             if feed_forward is not None else None)
        if feed_forward is not None and ff_norm is None:
            raise ValueError("a prenorm block with a feed-forward needs its norm")
        self.taps = None if input_conv is None else int(input_conv)
        self.conv_tensor = conv_tensor
        self.side = None if token_side is None else dict(token_side)
        if (self.taps is not None or self.side is not None) and hidden_size is None:
            raise ValueError("an input convolution or a token input needs the block's hidden_size")
        self.hidden_size = None if hidden_size is None else int(hidden_size)
        if self.taps is not None and self.taps < 1:
            raise ValueError(f"an input convolution needs at least one tap, got {input_conv}")
        if self.side is not None:
            self.side.setdefault("activation", "gelu_tanh")
            self.side["names"] = dict(self.SIDE_NAMES, **(self.side.get("names") or {}))
            if int(self.side["dim"]) < 1 or int(self.side["index"]) < 0:
                raise ValueError("a token input needs a positive dim and the layer's index")

    def cache_needs(self):
        needs = tuple(self.mixer.cache_needs())
        if self.taps is not None and self.taps > 1:
            needs += (CacheNeed("state", state_shape=(self.taps - 1, self.hidden_size)),)
        return needs

    def cache_need(self):
        needs = self.cache_needs()
        return needs[0] if len(needs) == 1 else self.mixer.cache_need()

    def params(self):
        ps, W = [], self.hidden_size
        if self.taps is not None:
            ps.append(ParamSpec("conv_taps", (WeightSource(self.conv_tensor, (W, self.taps)),)))
        if self.side is not None:
            n, d = self.side["names"], int(self.side["dim"])
            ps += [ParamSpec("side_gate", (WeightSource(n["gate"], (d, W)),)),
                   ParamSpec("side_proj", (WeightSource(n["proj"], (W, d)),)),
                   ParamSpec("side_norm", (WeightSource(n["norm"], (W,), "norm"),))]
        return ps

    def on_bound(self):
        self.no_tail = self.taps_t = None
        if self.taps is not None and self.w.get("conv_taps") is not None:
            # the taps once more as float32 [K, width]: the kernels' neighbouring threads read neighbouring floats
            self.taps_t = self.w["conv_taps"].float().t().contiguous()
        if self.taps == 1:
            self.no_tail = ops.torch.zeros((1, 0, self.hidden_size), dtype=ops.torch.float32, device=self.device)

    def _mixer_input(self, ctx, residual, delta, cache):
        """The normed rows the mixer reads (behind the input convolution, if the layer has one) and the mixer's own
        part of the layer's cache views."""
        if self.taps is None:
            return self.mixer_norm.forward(ctx, residual, delta), cache
        if self.taps > 1:
            views = cache if isinstance(cache, tuple) else (cache,)
            tail, rest = views[-1].state, views[:-1]
            cache = None if not rest else (rest[0] if len(rest) == 1 else tuple(rest))
        else:
            tail = self.no_tail
        h32 = self.mixer_norm.forward(ctx, residual, delta, out_dtype=ops.torch.float32)
        h = ctx.alloc(tuple(h32.shape), ctx.dtype)
        single = ctx.decode_only          # one token per request: the kernel that reads the tail also moves it up
        ops.causal_conv(h32, self.w["conv_taps"], None, tail, ctx, h, move_tail=single, add_input=True, taps_t=self.taps_t)
        if not single and self.taps > 1:
            ops.state_tail(h32, tail, ctx)
        return h, cache

    def _token_side(self, ctx, residual, delta):
        """Carries out the open sum, then the token input from the summed rows; returns the new open delta."""
        table = ctx.scratch.get("token_side_table")
        if table is None:
            raise ValueError("a layer with a token input needs an embedding with a per-token side table")
        d, i = int(self.side["dim"]), int(self.side["index"])
        f32 = ctx.dtype == ops.torch.float32
        xs = residual if f32 else ctx.alloc(tuple(residual.shape), ctx.dtype)
        ops.add_rows(residual, delta, None if f32 else xs)
        z = ops.linear(xs, self.w["side_gate"], None, out_dtype=ops.torch.float32)
        g = ctx.alloc((residual.shape[0], d), ctx.dtype)
        ops.gather_gate(z, ctx.token_ids, table, i * d, g, self.side["activation"], ctx.err)
        y = ops.linear(g, self.w["side_proj"], None, out_dtype=ops.torch.float32)
        out = ctx.alloc(tuple(y.shape), ops.torch.float32)
        ops.rms_rows(y, self.w["side_norm"], float(self.side["eps"]), out)
        return out

    def forward(self, ctx, residual, delta, cache):
        h, cache = self._mixer_input(ctx, residual, delta, cache)
        d = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is not None:
            h = self.ff_norm.forward(ctx, residual, d)
            d = self.feed_forward.forward(ctx, h)
        if self.side is not None:
            d = self._token_side(ctx, residual, d)
        return residual, d


@register_part("block", "parallel")
class ParallelBlock(Block):
    """``h = norm(x); x += mixer(h) + feed_forward(h)``.

    Where both sublayers can hand over their output projections (``detach_out_projection``), the block runs
    them as one product: ``[mixer's inner output | feed-forward's hidden layer] @ [W_o | W_down]^T (+ bias)``,
    so the two results are added inside the product's float32 accumulator and reach the residual stream as
    one float32 delta.  Where both can also hand over their first projections of h, those are one product as
    well (q, k, v and the feed-forward's up projection read the same h).  Otherwise the two results travel to
    the next norm as a float32 stack ``[2, T, H]`` and are added to the float32 residual there; either way
    the sum is never rounded to 16 bits.  ``feed_forward`` None: the layer has a mixer only.  ``fuse``
    False keeps every projection with its part."""

    def __init__(self, mixer: PartSpec, norm: PartSpec, feed_forward: Optional[PartSpec] = None, fuse: bool = True):
        self.norm = self.add_child("norm", build_part("norm", norm))
        self.mixer = self.add_child("mixer", build_part("mixer", mixer))
        self.feed_forward = (self.add_child("feed_forward", build_part("feed_forward", feed_forward))
                             if feed_forward is not None else None)
        self.out_m = self.out_f = self.in_m = self.in_f = None
        ff = self.feed_forward
        if fuse and ff is not None and self.mixer.detachable_out and ff.detachable_out:
            self.out_m, self.out_f = self.mixer.detach_out_projection(), ff.detach_out_projection()
            if self.out_m.biases and self.out_f.biases:
                raise ValueError("parallel block: at most one of the two output projections may have a bias")
            if self.mixer.detachable_in and ff.detachable_in and not getattr(self.mixer, "float32_projection", False):
                self.in_m, self.in_f = self.mixer.detach_in_projection(), ff.detach_in_projection()

    def params(self):
        ps = []
        if self.in_m is not None:
            ps.append(ParamSpec("in_w", self.in_m.weights + self.in_f.weights))
            for name, d in (("in_b_mixer", self.in_m), ("in_b_ff", self.in_f)):
                if d.biases:
                    ps.append(ParamSpec(name, d.biases))
        if self.out_m is not None:
            ps.append(ParamSpec("out_w", self.out_m.weights + self.out_f.weights, axis=1))
            if self.out_m.biases or self.out_f.biases:
                ps.append(ParamSpec("out_b", self.out_m.biases or self.out_f.biases))
        return ps

    def on_bound(self):
        self.in_b = None
        if self.in_m is not None and (self.in_m.biases or self.in_f.biases):
            # one bias vector for the joint product: zeros for the rows of the part that has none
            bm, bf = self.w.get("in_b_mixer"), self.w.get("in_b_ff")
            ref = bm if bm is not None else bf
            zeros = lambda n: ops.torch.zeros(n, dtype=ref.dtype, device=ref.device)
            self.in_b = ops.torch.cat([bm if bm is not None else zeros(self.in_m.width),
                                       bf if bf is not None else zeros(self.in_f.width)])

    def forward(self, ctx, residual, delta, cache):
        h = self.norm.forward(ctx, residual, delta)
        if self.feed_forward is None:
            return residual, self.mixer.forward(ctx, h, cache)
        if self.out_m is None:
            d_mix = self.mixer.forward(ctx, h, cache)
            d_ff = self.feed_forward.forward(ctx, h)
            return residual, ops.stack_deltas(ctx, (d_mix, d_ff))
        wm = self.out_m.width
        inner = ctx.alloc((h.shape[0], wm + self.out_f.width), h.dtype)
        pm = pf = None
        if self.in_m is not None:
            proj = ops.linear(h, self.w["in_w"], self.in_b)
            pm, pf = proj[:, :self.in_m.width], proj[:, self.in_m.width:]
        self.mixer.forward_inner(ctx, h, cache, inner[:, :wm], pm)
        self.feed_forward.forward_inner(ctx, h, inner[:, wm:], pf)
        return residual, ops.linear_delta(inner, self.w["out_w"], self.w.get("out_b"), f32=True)


@register_part("block", "postnorm")
class PostNormBlock(Block):
    """``x <- mixer_norm(alpha * x + mixer(x))``, then ``x <- ff_norm(alpha * x + feed_forward(x))``: the norm
    comes after the sum and the normed rows are the residual stream, which stays float32; the sublayers read x
    itself (a mixer with ``reads_float32`` the float32 rows, the others their copy in the compute dtype, which the
    norm kernel writes beside them).  ``feed_forward`` None: the layer ends after its mixer - unless the model file
    still has the second norm's weight, in which case that norm is applied to ``alpha * x``."""

    def __init__(self, mixer: PartSpec, mixer_norm: PartSpec, alpha: float = 1.0, feed_forward: Optional[PartSpec] = None,
                 ff_norm: Optional[PartSpec] = None):
        self.alpha = float(alpha)
        self.mixer_norm = self.add_child("mixer_norm", build_part("norm", mixer_norm))
        self.mixer = self.add_child("mixer", build_part("mixer", mixer))
        self.feed_forward = (self.add_child("feed_forward", build_part("feed_forward", feed_forward))
                             if feed_forward is not None else None)
        self.ff_norm = self.add_child("ff_norm", build_part("norm", ff_norm)) if ff_norm is not None else None
        if self.feed_forward is not None and self.ff_norm is None:
            raise ValueError("a postnorm block with a feed-forward needs the norm that follows it")

    def forward(self, ctx, residual, delta, cache):
        x = residual
        if delta is not None:                # a block of another kind left its last sum to be done
            x.add_(delta if delta.dim() == 2 else delta.sum(0))
        h = ctx.scratch.get("postnorm_rows")
        if h is None or ctx.scratch.get("postnorm_rows_of") is not x:
            h = x if ctx.dtype == ops.torch.float32 else x.to(ctx.dtype)
        d = self.mixer.forward(ctx, x if self.mixer.reads_float32 else h, cache)
        h = self.mixer_norm.forward_post(ctx, x, d, self.alpha)
        if self.feed_forward is not None:
            d = self.feed_forward.forward(ctx, h)
            h = self.ff_norm.forward_post(ctx, x, d, self.alpha)
        elif self.ff_norm is not None and self.ff_norm.w.get("weight") is not None:
            h = self.ff_norm.forward_post(ctx, x, None, self.alpha)
        # the next block of this kind starts from these rows: no second rounding pass over x
        ctx.scratch["postnorm_rows"], ctx.scratch["postnorm_rows_of"] = h, x
        return x, None


@register_part("block", "hyper")
class HyperBlock(Block):
    """Hyper-connections: the residual stream is ``streams`` copies ``x_1 .. x_s`` (all equal to the embedding's
    rows at the start).  Around sublayer q (1: the mixer, 2: the feed-forward) with its weights ``in_q [s]``,
    ``mix_q [s, s]`` (indexed from, to) and ``out_q [s]``::

        u = sum_i in_q[i] x_i;    y = sublayer(norm_q(u));    x_j <- sum_i mix_q[i, j] x_i + out_q[j] y

    for all j at once from the old copies.  After the last layer the stream is the sum of the copies (the model's
    final norm reads that).  Each update is left open (a ``StreamUpdate``) and carried out by the launch that
    forms the next read-in and its norm, so the copies are read and written once per sublayer, in float32.
    ``feed_forward`` None: the layer has a mixer only.  ``learned`` False: no connection weights at all (reading
    sums the copies, writing adds the result to each; with one copy this is the plain pre-norm residual layer).
    ``names``: the tensors of a sublayer's connection, after
    ``hc1.`` / ``hc2.`` (keys in, mix, out)."""

    NAMES = dict(inp="in", mix="mix", out="out")

    def __init__(self, streams: int, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: Optional[PartSpec] = None,
                 ff_norm: Optional[PartSpec] = None, names: Optional[dict] = None, prefixes=("hc1.", "hc2."),
                 learned: bool = True):
        self.streams, self.learned = int(streams), bool(learned)
        if not 1 <= self.streams <= 8:
            raise ValueError(f"hyper-connections with {self.streams} streams: the kernel keeps 1 to 8 copies")
        self.mixer_norm = self.add_child("mixer_norm", build_part("norm", mixer_norm))
        self.mixer = self.add_child("mixer", build_part("mixer", mixer))
        self.feed_forward = (self.add_child("feed_forward", build_part("feed_forward", feed_forward))
                             if feed_forward is not None else None)
        self.ff_norm = self.add_child("ff_norm", build_part("norm", ff_norm)) if feed_forward is not None else None
        if self.feed_forward is not None and ff_norm is None:
            raise ValueError("a hyper block with a feed-forward needs its norm")
        self.names, self.prefixes = dict(self.NAMES, **(names or {})), tuple(prefixes)

    def params(self):
        s, n, ps = self.streams, self.names, []
        if not self.learned:
            return ps
        for q, pre in enumerate(self.prefixes[:2 if self.feed_forward is not None else 1], start=1):
            ps += [ParamSpec(f"in{q}", (WeightSource(pre + n["inp"], (s,), "norm"),)),
                   ParamSpec(f"mix{q}", (WeightSource(pre + n["mix"], (s, s), "eye"),)),
                   ParamSpec(f"out{q}", (WeightSource(pre + n["out"], (s,), "norm"),))]
        return ps

    def forward(self, ctx, residual, delta, cache):
        s, x = self.streams, residual
        if x.dim() == 2:                           # the first block of this kind: every copy starts as these rows
            x_out = ctx.alloc((s,) + tuple(x.shape), x.dtype)
        else:
            if x.shape[0] != s:
                raise ValueError(f"this block keeps {s} copies of the residual stream, the one before it {x.shape[0]}")
            x_out = x
        w = self.w.get
        h = self.mixer_norm.forward_streams(ctx, x, s, x_out, delta, w("in1"))
        d = StreamUpdate(self.mixer.forward(ctx, h, cache), w("mix1"), w("out1"))
        if self.feed_forward is not None:
            h = self.ff_norm.forward_streams(ctx, x_out, s, x_out, d, w("in2"))
            d = StreamUpdate(self.feed_forward.forward(ctx, h), w("mix2"), w("out2"))
        return x_out, d
