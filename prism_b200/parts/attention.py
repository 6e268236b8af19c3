"""Attention mixer.  ``gqa_attention``: andre-fu/prism's attention sub-layer
(engine/executor.py:109-122): fused q/k/v projection with bias, position
encoding of q and k, append of k and v to the paged cache, causal
grouped-query attention over the cache with scale ``hd^-1/2``, output
projection.  Head counts, head size, bias, window and the position encoding
are parameters; so are a value size of its own, a chunked mask, a softmax
sink, the score scale and whether the layer has key and value projections at
all (a layer without reads another layer's cache plane).
``latent_attention``: keys and values are up-projections of a low-rank latent
that is all the cache holds, next to one rotated key part shared by the heads."""

from __future__ import annotations

import math
import warnings
from typing import Optional

import torch

from ..config.model_config import ConfigError
from .base import CacheNeed, DetachedProjection, Mixer, ParamSpec, PartSpec, WeightSource, build_part, register_part
from .. import ops


_warned = set()
MAX_HEAD_DIM = 256        # the shape-generic attention kernel keeps one head's row in a warp's registers
MAX_DISTANCE = 1 << 20    # the farthest distance a bias table by distance is laid out for (4 MB a head in float32)


def distance_bucket(n: int, rows: int, far: int) -> int:
    """The row of a distance-bias table with ``rows`` rows for the key ``n`` positions back: distances below ``rows //
    2`` have a row each; the upper half is shared in logarithmic steps, ``half + floor(ln(n / half) / ln(far / half) *
    (rows - half))``, and ends at ``far`` (every distance from there on has the last row).  The quotient of logarithms
    is taken in float64 and a value within 1e-9 of a whole number counts as that number, so that distances at which
    the formula is exact (n = half times a power of far / half with a whole exponent) land on their row."""
    half = rows // 2
    if n < half:
        return n
    if half == 0 or far <= half or n >= far:
        return rows - 1
    v = math.log(n / half) / math.log(far / half) * (rows - half)
    if abs(v - round(v)) < 1e-9:
        v = round(v)
    return min(rows - 1, half + int(math.floor(v)))



@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    """``v_head_dim``: size of a value (default: ``head_dim``).  ``chunk``: a query sees only the keys of
    its own block of ``chunk`` positions, counted from position 0 (with ``window``: both limits hold; the
    fast kernels take one of the two).  ``sink``: a learned number per head whose exponential joins the
    softmax's denominator, unscaled and without a value.  ``own_kv`` False: no key and value projections;
    the layer's run must read another run's cache plane (``ScheduleEntry.reads_cache_of``).
    ``cache_chunk``: the block size by which the cache gives pages back - ``"mask"``: that of this layer's
    mask; None: never (a plane that layers with different masks read).  ``keep_first``: under a window, the
    first ``keep_first`` positions of the sequence stay visible to every later query (at their true positions).
    ``qk_norm_eps``: every head of q and k is RMS-normed over ``head_dim`` before it is rotated, with one weight
    vector for q and one for k that all heads share; with ``qk_norm_whole`` the norm runs over the whole projection
    instead (all heads of q, or of k, at once, with weights of that size).  ``gate``: the concatenated heads are
    multiplied by ``sigmoid(W_g h)`` before the output projection; ``gate="head"``: one gate number per head.
    ``sink_value``: a constant sink, the same for every head (0: one is added to the softmax's denominator).  ``out_scale``: a constant on the layer's result (folded into
    the gate).  A rotation with rescaled frequencies (``rotary_scaled``), the query/key norm and the gate
    work from the float32 result of the input projection; so may a layer without keys and values of its own.
    ``qk_norm_weight`` False: the query/key norm has no weights (q and k are divided by their root mean square and
    nothing else).  ``dist_bias``: a learned bias by distance on the scaled scores, ``dict(rows=B, far=D)``: a table
    ``[B, heads]`` (tensor ``rel``) whose row for the key n positions back is ``distance_bucket(n, B, D)`` - one row
    for each distance below ``B / 2``, the rest shared in steps that grow like a logarithm up to D.  ``names``: the tensors' names in the model file (keys
    q, k, v, o, q_b, k_b, v_b, o_b, sink, q_norm, k_norm, g)."""

    NAMES = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight",
                 q_b="q_proj.bias", k_b="k_proj.bias", v_b="v_proj.bias", o_b="o_proj.bias", sink="sinks",
                 q_norm="q_norm.weight", k_norm="k_norm.weight", g="g_proj.weight", rel="rel")
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool = True, o_bias: bool = False, window: Optional[int] = None,
                 position: Optional[PartSpec] = None, scale: Optional[float] = None,
                 v_head_dim: Optional[int] = None, chunk: Optional[int] = None, sink: bool = False,
                 own_kv: bool = True, cache_chunk="mask", names: Optional[dict] = None, keep_first: int = 0,
                 qk_norm_eps: Optional[float] = None, gate=False, out_scale: float = 1.0, qk_norm_whole: bool = False,
                 sink_value: Optional[float] = None, qk_norm_weight: bool = True, dist_bias: Optional[dict] = None):
        if num_heads % num_kv_heads:
            raise ConfigError(f"num_heads {num_heads} not divisible by num_kv_heads {num_kv_heads}")
        self.hidden_size, self.nh, self.nkv, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.qkv_bias, self.o_bias = bool(qkv_bias), bool(o_bias)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else self.hd ** -0.5
        self.position = self.add_child("position", build_part("position", position)) if position else None
        self.vhd = self.hd if v_head_dim is None else int(v_head_dim)
        self.chunk = None if chunk is None else int(chunk)
        if self.vhd < 1 or (self.chunk is not None and self.chunk < 1) or (self.window is not None and self.window < 1):
            raise ConfigError(f"value size {self.vhd}, chunk {self.chunk}, window {self.window}: all must be at least 1")
        if self.chunk is not None and self.window is not None:
            raise ConfigError("a layer's mask is a window or a chunk, not both")
        self.sink, self.own_kv = bool(sink), bool(own_kv)
        self.sink_value = None if sink_value is None else float(sink_value)
        if self.sink and self.sink_value is not None:
            raise ConfigError("a layer's sink is learned or a constant, not both")
        self.cache_chunk = self.chunk if cache_chunk == "mask" else (None if cache_chunk is None else int(cache_chunk))
        self.names = dict(self.NAMES, **(names or {}))
        # what the fused rotate-and-store and the equal-size attention kernels do not cover goes the general way:
        # projection, (rotation,) one store per plane, attention under a KeyMask
        self.keep_first = int(keep_first)
        if self.keep_first < 0 or (self.keep_first and self.window is None):
            raise ConfigError("keep_first: a number of first positions, kept visible behind a window")
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.gate, self.out_scale = bool(gate), float(out_scale)
        self.gate_per_head = gate == "head"
        self.qk_norm_whole = bool(qk_norm_whole) and self.qk_norm_eps is not None
        scaled = bool(position and position.kind == "rotary_scaled")
        # query/key norm, a rotation from a table of rescaled frequencies and the gate read the input projection's
        # float32 result
        self.float32_projection = self.qk_norm_eps is not None or self.gate or scaled
        if self.float32_projection and qkv_bias and self.gate:
            raise ConfigError("an output gate beside biases on q, k, v is not built: the gate's rows have no bias")
        self.qk_norm_weight = bool(qk_norm_weight)
        self.dist_bias = None
        if dist_bias is not None:
            rows, far = int(dist_bias["rows"]), int(dist_bias["far"])
            if rows < 1 or far < 1 or far > MAX_DISTANCE:
                raise ConfigError(f"a distance bias needs at least one row and a farthest distance from 1 to {MAX_DISTANCE}, "
                                  f"got rows {rows}, far {far}")
            self.dist_bias = (rows, far)
        self.general = (self.dist_bias is not None or self.vhd != self.hd or self.chunk is not None or self.sink or not self.own_kv
                        or self.sink_value is not None
                        or self.keep_first > 0 or self.float32_projection)
        self._own_in = self._own_out = True
        # the equal-size kernels keep a head's row in a warp's registers and rotate pairs; the general path takes
        # any key size (its kernels loop over it) and values of up to 1024 entries
        if not self.general and (not 2 <= self.hd <= MAX_HEAD_DIM or self.hd % 2):
            raise ConfigError(f"head_dim {head_dim}: the attention kernels take even head sizes from 2 to "
                              f"{MAX_HEAD_DIM}")
        if self.general and (self.hd < 1 or self.vhd > 1024):
            raise ConfigError(f"head_dim {head_dim}, value size {self.vhd}: keys need at least one entry and values "
                              f"at most 1024")
        self.mask = (ops.KeyMask.chunk(self.chunk) if self.chunk is not None
                     else ops.KeyMask.window(self.window, self.keep_first))

    @property
    def q_size(self):
        return self.nh * self.hd

    @property
    def kv_size(self):
        return self.nkv * self.hd

    @property
    def v_size(self):
        return self.nkv * self.vhd

    def cache_need(self):
        return CacheNeed("paged", self.nkv, self.hd, self.window,
                         v_head_dim=None if self.vhd == self.hd else self.vhd, chunk=self.cache_chunk,
                         keep_first=self.keep_first)

    def _in_sources(self):
        H, qs, kvs, vs, n = self.hidden_size, self.q_size, self.kv_size, self.v_size, self.names
        w = [WeightSource(n["q"], (qs, H))]
        b = [WeightSource(n["q_b"], (qs,), "bias")]
        if self.own_kv:
            w += [WeightSource(n["k"], (kvs, H)), WeightSource(n["v"], (vs, H))]
            b += [WeightSource(n["k_b"], (kvs,), "bias"), WeightSource(n["v_b"], (vs,), "bias")]
        if self.gate:
            w.append(WeightSource(n["g"], (self.nh if self.gate_per_head else self.nh * self.vhd, H)))
        return tuple(w), tuple(b) if self.qkv_bias else ()

    def _out_sources(self):
        n = self.names
        return ((WeightSource(n["o"], (self.hidden_size, self.nh * self.vhd)),),
                (WeightSource(n["o_b"], (self.hidden_size,), "bias"),) if self.o_bias else ())

    def params(self):
        ps = []
        if self._own_in:
            w, b = self._in_sources()
            ps.append(ParamSpec("qkv_w", w))
            if b:
                ps.append(ParamSpec("qkv_b", b))
        if self.sink:
            ps.append(ParamSpec("sink", (WeightSource(self.names["sink"], (self.nh,), "bias"),)))
        if self.dist_bias is not None:
            ps.append(ParamSpec("rel", (WeightSource(self.names["rel"], (self.dist_bias[0], self.nh), "bias"),)))
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            nq, nk = (self.q_size, self.kv_size) if self.qk_norm_whole else (self.hd, self.hd)
            ps.append(ParamSpec("q_norm", (WeightSource(self.names["q_norm"], (nq,), "norm"),)))
            if self.own_kv:
                ps.append(ParamSpec("k_norm", (WeightSource(self.names["k_norm"], (nk,), "norm"),)))
        if self._own_out:
            w, b = self._out_sources()
            ps.append(ParamSpec("o_w", w))
            if b:
                ps.append(ParamSpec("o_b", b))
        return ps

    # only the general path hands its projections to the block: the other one has fused kernels of its own
    @property
    def detachable_out(self):
        return self.general

    @property
    def detachable_in(self):
        return self.general

    def detach_out_projection(self):
        if not self.general:
            return None
        self._own_out = False
        w, b = self._out_sources()
        return DetachedProjection(self.handed_over(*w), self.handed_over(*b), self.nh * self.vhd)

    def detach_in_projection(self):
        if not self.general:
            return None
        self._own_in = False
        w, b = self._in_sources()
        return DetachedProjection(self.handed_over(*w), self.handed_over(*b), sum(s.shape[0] for s in w),
                                  float32=self.float32_projection)

    def on_bound(self):
        # Said once, when the model is built, not found out from the step time: in bfloat16 the tensor-core
        # attention kernels take head sizes in steps of 16 up to 128 with up to 16 query heads per kv head; every
        # other shape runs on the shape-generic kernel (one warp per token and head), correct but far slower.
        self.const_sink = (None if self.sink_value is None else
                           torch.full((self.nh,), self.sink_value, dtype=torch.float32, device=self.device))
        self.bias_table = None
        if self.dist_bias is not None and self.w.get("rel") is not None:
            # the table by distance that the kernels index: [heads, far + 1], distances beyond `far` share the last entry
            rows, far = self.dist_bias
            idx = torch.tensor([distance_bucket(n, rows, far) for n in range(far + 1)], dtype=torch.long, device=self.device)
            self.bias_table = self.w["rel"].float()[idx].t().contiguous()
        self.plain_norm = None
        if self.qk_norm_eps is not None and not self.qk_norm_weight:
            n = max(self.q_size, self.kv_size) if self.qk_norm_whole else self.hd
            self.plain_norm = torch.ones(n, dtype=torch.float32, device=self.device)
        if self.general:
            return
        if self.dtype == torch.bfloat16 and not ops.attention_bf16_shape_ok(self.hd, self.nh, self.nkv):
            key = (self.hd, self.nh, self.nkv)
            if key not in _warned:
                _warned.add(key)
                warnings.warn(f"attention with head_dim {self.hd}, {self.nh} heads, {self.nkv} kv heads runs on the "
                              f"shape-generic kernel in bfloat16 (the tensor-core kernels take head_dim 16, 32, ... 128 "
                              f"and up to 16 query heads per kv head): correct, but much slower", RuntimeWarning,
                              stacklevel=2)

    def forward_inner(self, ctx, x, cache, out, proj=None):
        """Projection (+ bias; ``proj``: made by the block already), rotation if the layer has one, one store
        per cache plane, attention under the layer's mask with its sink into ``out [T, nh * vhd]``."""
        T, qs, kvs = x.shape[0], self.q_size, self.kv_size
        if cache.write != self.own_kv:
            raise ValueError("a layer without key and value projections must read another run's cache plane, "
                             "and one with them owns its plane")
        if self.float32_projection:
            return self._forward_inner_f32(ctx, x, cache, out, proj)
        qkv = proj if proj is not None else ops.linear(x, self.w["qkv_w"], self.w.get("qkv_b"))
        q = qkv[:, :qs].view(T, self.nh, self.hd)
        k = qkv[:, qs:qs + kvs].view(T, self.nkv, self.hd) if self.own_kv else None
        if self.position is not None:
            rot = self.position.rotary()
            if rot is None:
                self.position.apply(ctx, q, k)
            elif rot.rotary_dim:
                ops.rotate_slice(q, q, rot.rotary_dim, rot.inv_freq, ctx.positions)
                if k is not None:
                    ops.rotate_slice(k, k, rot.rotary_dim, rot.inv_freq, ctx.positions)
        if self.own_kv:
            ops.cache_store(qkv[:, qs:qs + kvs], cache.k, cache.block_table, ctx.positions, ctx.tok_seg, cache.num_pages,
                            ctx.max_positions, ctx.err, src2=qkv[:, qs + kvs:], plane2=cache.v)
        ops.masked_attention(ctx, q, out, cache.k, cache.v, cache.block_table, cache.num_pages, self.mask, self.scale,
                             self._sink(), self.bias_table)

    def _forward_inner_f32(self, ctx, x, cache, out, proj):
        """From the float32 projection ``[q | k | v | gate]`` (``[q | gate]`` in a layer without keys and values of
        its own): one launch norms and rotates q and k and stores k and v at the tokens' slots; attention under the
        mask; the gate (and ``out_scale``) on its way into ``out``."""
        T, qs = x.shape[0], self.q_size
        kvs, vs = (self.kv_size, self.v_size) if self.own_kv else (0, 0)
        if proj is None:
            proj = ops.linear(x, self.w["qkv_w"], self.w.get("qkv_b"), out_dtype=torch.float32)
        rot = self.position.rotary() if self.position is not None else None
        if self.position is not None and rot is None:
            raise ConfigError("with query/key norm or an output gate the attention part takes a rotary position encoding")
        q = ctx.alloc((T, self.nh, self.hd), ctx.dtype)
        own = self.own_kv
        if self.plain_norm is not None:
            wq = self.plain_norm[:self.q_size if self.qk_norm_whole else self.hd]
            wk = self.plain_norm[:self.kv_size if self.qk_norm_whole else self.hd]
        else:
            wq, wk = self.w.get("q_norm"), self.w.get("k_norm")
        ops.qk_norm_rope_store(proj[:, :qs], proj[:, qs:qs + kvs] if own else None,
                               proj[:, qs + kvs:qs + kvs + vs] if own else None, wq,
                               wk if own else None, self.qk_norm_eps or 0.0,
                               rot.inv_freq if rot and rot.rotary_dim else None, rot.rotary_dim if rot else 0, q,
                               cache.k if own else None, cache.v if own else None, cache.block_table, ctx.positions,
                               ctx.tok_seg, cache.num_pages, ctx.max_positions, ctx.err, whole=self.qk_norm_whole,
                               halves=bool(rot and not rot.interleaved), nkv=self.nkv)
        attn = ctx.alloc((T, self.nh * self.vhd), ctx.dtype) if self.gate else out
        ops.masked_attention(ctx, q, attn, cache.k, cache.v, cache.block_table, cache.num_pages, self.mask, self.scale,
                             self._sink(), self.bias_table)
        if self.gate:
            ops.gated_product(attn, proj[:, qs + kvs + vs:], out, "sigmoid", self.out_scale)
        elif self.out_scale != 1.0:
            out.mul_(self.out_scale)

    def _sink(self):
        return self.w.get("sink") if self.sink else self.const_sink

    def forward(self, ctx, x, cache):
        if self.general:
            attn = ctx.alloc((x.shape[0], self.nh * self.vhd), ctx.dtype)
            self.forward_inner(ctx, x, cache, attn)
            return ops.linear_delta(attn, self.w["o_w"], self.w.get("o_b"))
        T, qs, kvs = x.shape[0], self.q_size, self.kv_size
        rot = self.position.rotary() if self.position is not None else None
        if rot is None and self.position is not None:
            # a position encoding that is not rotary: project, let it encode q and k, then store
            qkv = ops.linear(x, self.w["qkv_w"], self.w.get("qkv_b"))
            q = qkv[:, :qs].view(T, self.nh, self.hd)
            k = qkv[:, qs:qs + kvs].view(T, self.nkv, self.hd)
            v = qkv[:, qs + kvs:].view(T, self.nkv, self.hd)
            self.position.apply(ctx, q, k)
            ops.rope_kv_write(q, k, v, ctx.positions, ctx.tok_seg, None, 0,
                              cache.k if cache.write else None, cache.v if cache.write else None,
                              cache.block_table, cache.num_pages, ctx.max_positions, ctx.err)
        else:
            attn = ctx.alloc((T, qs), x.dtype)
            ops.qkv_attention(ctx, x, self.w["qkv_w"], self.w.get("qkv_b"), self.nh, self.nkv, self.hd, rot, cache,
                              self.window, self.scale, attn)
            return ops.linear_delta(attn, self.w["o_w"], self.w.get("o_b"))
        attn = ctx.alloc((T, qs), x.dtype)
        ops.attention(ctx, q, attn, cache, self.window, self.scale)
        return ops.linear_delta(attn, self.w["o_w"], self.w.get("o_b"))


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Attention whose keys and values are up-projections of a cached latent.

    With h the layer's input, per token::

        c_q = rmsnorm(W_dq h)            q = W_uq c_q        per head [head_dim plain | rot_dim rotated]
        [c' | k_r] = W_dkv h             c = rmsnorm(c')     k_r: rot_dim entries, rotated, one for all heads
        k_h = W_uk,h c                   v_h = W_uv,h c
        score_h(i, j) = (q_plain,h(i) . k_h(j) + q_rot,h(i) . k_r(j)) * scale

    The cache holds ``[c | k_r]`` per token (``kv_rank + rot_dim`` numbers, one "head").  Nothing is
    up-projected again at a later step: the key up-projection moves to the query side (``q_plain,h W_uk,h``
    is scored against c itself) and the value up-projection behind the attention (the weighted sum of the
    latents is projected once per query), so each step is attention with ``num_heads`` query heads over one
    key/value head whose values are the first ``kv_rank`` entries of its key rows.

    ``window``: sliding window (None: all keys).  ``rope_dims`` (default ``rot_dim``): how many entries of the
    rotated part really turn.  ``names``: the tensors' names in the model file.
    """

    NAMES = dict(dq="q_a_proj.weight", dq_norm="q_a_layernorm.weight", uq="q_b_proj.weight",
                 dkv="kv_a_proj_with_mqa.weight", dkv_norm="kv_a_layernorm.weight", uk="k_b_proj.weight",
                 uv="v_b_proj.weight", o="o_proj.weight")

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int,
                 kv_rank: int, eps: float, rope_base: float = 10000.0, rope_dims: Optional[int] = None,
                 window: Optional[int] = None, scale: Optional[float] = None, names: Optional[dict] = None):
        self.hidden_size, self.nh, self.hd = int(hidden_size), int(num_heads), int(head_dim)
        self.rd, self.vhd, self.q_rank, self.kv_rank = int(rot_dim), int(v_head_dim), int(q_rank), int(kv_rank)
        self.eps, self.rope_base = float(eps), float(rope_base)
        self.rope_dims = self.rd if rope_dims is None else int(rope_dims)
        if self.rope_dims % 2 or not 0 <= self.rope_dims <= self.rd:
            raise ConfigError(f"{self.rope_dims} rotated entries: must be even and at most rot_dim {self.rd}")
        if min(self.nh, self.hd, self.vhd, self.q_rank, self.kv_rank) < 1 or self.rd < 0:
            raise ConfigError("latent attention: heads, sizes and ranks must be positive")
        self.window = None if window is None else int(window)
        if self.window is not None and self.window < 1:
            raise ConfigError(f"window {self.window} must be at least 1")
        self.scale = float(scale) if scale is not None else (self.hd + self.rd) ** -0.5
        self.names = dict(self.NAMES, **(names or {}))
        self.mask = ops.KeyMask.window(self.window)
        self._own_out = True

    def cache_need(self):
        return CacheNeed("paged", 1, self.kv_rank + self.rd, self.window, v_head_dim=0)

    def params(self):
        H, nh, n = self.hidden_size, self.nh, self.names
        return [
            ParamSpec("down_w", (WeightSource(n["dq"], (self.q_rank, H)),
                                 WeightSource(n["dkv"], (self.kv_rank + self.rd, H)))),
            ParamSpec("dq_norm", (WeightSource(n["dq_norm"], (self.q_rank,), "norm"),)),
            ParamSpec("dkv_norm", (WeightSource(n["dkv_norm"], (self.kv_rank,), "norm"),)),
            ParamSpec("uq_w", (WeightSource(n["uq"], (nh * (self.hd + self.rd), self.q_rank)),)),
            ParamSpec("uk_w", (WeightSource(n["uk"], (nh * self.hd, self.kv_rank)),)),
            ParamSpec("uv_w", (WeightSource(n["uv"], (nh * self.vhd, self.kv_rank)),)),
        ] + ([ParamSpec("o_w", (self._o_source(),))] if self._own_out else [])

    detachable_out = True        # the down projections feed norms and stay float32: they are not handed over

    def _o_source(self):
        return WeightSource(self.names["o"], (self.hidden_size, self.nh * self.vhd))

    def detach_out_projection(self):
        self._own_out = False
        return DetachedProjection(self.handed_over(self._o_source()), (), self.nh * self.vhd)

    def on_bound(self):
        half = self.rope_dims // 2
        i = torch.arange(half, dtype=torch.float64)
        self.inv_freq = (self.rope_base ** (-2.0 * i / max(self.rope_dims, 1))).to(torch.float32).to(self.device)
        # W_uk per head, turned so that a head's plain query part is projected into the latent space
        self.uk_t = self.w["uk_w"].view(self.nh, self.hd, self.kv_rank).transpose(1, 2).contiguous()     # [nh, R, hd]
        self.uv = self.w["uv_w"].view(self.nh, self.vhd, self.kv_rank)                                  # [nh, vhd, R]

    def forward(self, ctx, x, cache):
        attn = ctx.alloc((x.shape[0], self.nh * self.vhd), x.dtype)
        self.forward_inner(ctx, x, cache, attn)
        return ops.linear_delta(attn, self.w["o_w"])

    def forward_inner(self, ctx, x, cache, out, proj=None):
        T, nh, hd, rd, R = x.shape[0], self.nh, self.hd, self.rd, self.kv_rank
        # both down projections in one product; float32, because each feeds a norm
        down = ops.linear(x, self.w["down_w"], None, out_dtype=torch.float32)
        cq = ctx.alloc((T, self.q_rank), x.dtype)
        # one launch: the query latent normed, the key/value latent normed, the shared key part rotated, the row stored
        ops.latent_kv_store(down[:, self.q_rank:], self.w["dkv_norm"], self.eps, R, self.rope_dims, self.inv_freq,
                            cache.k, cache.block_table, ctx.positions, ctx.tok_seg, cache.num_pages, ctx.max_positions,
                            ctx.err, xq=down[:, :self.q_rank], q_weight=self.w["dq_norm"], q_out=cq)
        q = ops.linear(cq, self.w["uq_w"]).view(T, nh, hd + rd)
        qf = ctx.alloc((T, nh, R + rd), x.dtype)                   # per head [plain part in latent space | rotated part]
        ops.matmul_heads(q[:, :, :hd], self.uk_t, qf[:, :, :R])
        if rd:
            ops.rotate_slice(q[:, :, hd:], qf[:, :, R:], self.rope_dims, self.inv_freq, ctx.positions)
        lat = ctx.alloc((T, nh * R), x.dtype)
        ops.masked_attention(ctx, qf, lat, cache.k, cache.k[..., :R], cache.block_table, cache.num_pages, self.mask,
                             self.scale, None)
        ops.matmul_heads(lat.view(T, nh, R), self.uv, out.view(T, nh, self.vhd))
