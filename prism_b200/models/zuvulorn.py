"""Zuvulorn: a small decoder whose ``config.json`` lists its layers one by one.
Its typed configuration, its layer plan and its entry in the architecture
registry; everything this engine knows about the design by name is here.

The design, as this file builds it from the parts:

* embedding rows as they are;
* every layer is a *hyper* block: the residual stream is kept in ``streams``
  copies, each sublayer reads a learned weighted sum of them through a layer
  norm (weight, no bias) and writes back through a learned mix of the copies
  plus its result times a weight per copy (``l<i>.hc1.*`` for the mixer,
  ``l<i>.hc2.*`` for the feed-forward);
* mixer ``attention``: grouped-query attention without biases; q and k are
  RMS-normed over the whole projection (all heads at once) before the first
  ``rot.dims`` entries of each head are rotated in halves, with frequencies
  rescaled in three bands; an explicit score scale; plain causal mask; one
  added to the softmax's denominator (a sink of score 0); a sigmoid gate per
  head on the heads' outputs; with ``kv_from: j`` the layer has no key and
  value tensors and attends over layer j's cache plane with its own queries;
* mixer ``channel_delta``: the delta rule with one decay per key channel from
  a low-rank product and a low-rank sigmoid gate (``parts/recurrent.py``);
* mixer ``rglru``: a gelu branch times a real-gated linear recurrence behind
  a short convolution (``parts/recurrent.py``);
* feed-forward ``moe``: sigmoid router, the ``top`` largest scores, the score
  multiplies the chosen expert's input (``parts/feedforward.py``);
* the final layer norm (``final.norm``) reads the sum of the copies; an
  untied linear head (``head``).

The ranks of the channel-delta mixer's low-rank products are the shapes of
``a1`` and ``g1`` in the model file (``decay_rank`` and ``gate_rank`` in the
mixer's configuration where there is no file).  The design puts no limit on
positions; block tables need a width, so ``max_positions`` (an engine knob,
default 131072) may be given in the file.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..config.model_config import ConfigError
from ..model_registry import register_architecture
from ..parts.base import PartSpec
from .decoder import ModelSpec, ScheduleEntry

ARCHITECTURE = "Zuvulorn"
DEFAULT_MAX_POSITIONS = 131072
UNIT_EPS = 1e-6            # the design fixes it: q and k of the delta rule are x / sqrt(sum x^2 + 1e-6)
RGLRU_DECAY = 8.0          # the design fixes it: log a = -8 r softplus(lam)
SINK_SCORE = 0.0           # the design fixes it: the softmax's denominator has one more term, exp(0)


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = int(_need(d, key, where))
    if v < 1:
        raise ConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _heads(mx, where):
    heads = _pos_int(mx, "heads", where)
    kvh = int(mx.get("kv_heads") or heads)
    if kvh < 1 or heads % kvh:
        raise ConfigError(f"config.json: {where}: heads ({heads}) not divisible by kv_heads ({kvh})")
    return heads, kvh


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[Tuple[float, float, float, float]]     # factor, low, high, original
    kv_from: Optional[int]            # layer whose keys and values this layer uses (None: its own)


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int


@dataclass(frozen=True)
class RGLRUConfig:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class ZuvulornLayer:
    type: str                         # "attention" | "channel_delta" | "rglru"
    mixer: object
    mlp: Optional[ExpertsConfig]      # None: the layer has no feed-forward


def _rank(mx, key, tensor, shapes, where):
    rank = mx.get(key)
    if shapes is not None:
        shape = shapes.get(tensor)
        if shape is None or len(shape) != 2:
            raise ConfigError(f"the model file has no matrix '{tensor}', whose rows are a low-rank product's rank")
        rank = shape[0]
    if rank is None:
        raise ConfigError(f"config.json: {where} has no '{key}' (without a model file nothing else gives it)")
    return int(rank)


def _attention(mx, where, i, layers) -> SinkAttentionConfig:
    heads, kvh = _heads(mx, where)
    dim = _pos_int(mx, "dim", where)
    vdim = int(mx.get("vdim") or dim)
    rot = mx.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    if dims % 2 or not 0 <= dims <= dim:
        raise ConfigError(f"config.json: {where}.rot.dims = {dims}: must be even and at most dim ({dim})")
    sc = rot.get("scaling")
    scaling = None
    if sc:
        scaling = tuple(float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "low", "high", "original"))
    src = mx.get("kv_from")
    if src is not None:
        src = int(src)
        if not 0 <= src < i or layers[src].type != "attention" or layers[src].mixer.kv_from is not None:
            raise ConfigError(f"config.json: {where}.kv_from = {src}: must name an earlier attention layer with key and "
                              f"value projections of its own")
        o = layers[src].mixer
        if (o.kv_heads, o.dim, o.vdim) != (kvh, dim, vdim):
            raise ConfigError(f"config.json: {where}: kv_heads, dim and vdim must equal those of layer {src}, whose keys "
                              f"and values it uses")
    return SinkAttentionConfig(heads, kvh, dim, vdim, float(_need(mx, "scale", where)), dims, float(rot.get("base", 10000.0)),
                               scaling, src)


@dataclass(frozen=True)
class ZuvulornConfig:
    vocab: int
    width: int
    eps: float
    streams: Optional[int]            # None: one residual stream and no connection weights (plain pre-norm layers)
    layers: Tuple[ZuvulornLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict, tensor_shapes: Optional[dict] = None) -> "ZuvulornConfig":
        vocab, width = _pos_int(raw, "vocab", "the model"), _pos_int(raw, "width", "the model")
        eps = float(_need(_need(raw, "norm", "the model"), "eps", "norm"))
        streams = None if raw.get("streams") is None else int(raw["streams"])
        if streams is not None and not 1 <= streams <= 8:
            raise ConfigError(f"config.json: streams = {streams}: this engine keeps 1 to 8 copies of the residual stream")
        layers_raw = _need(raw, "layers", "the model")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            kind, mx = _need(lr, "type", where), _need(lr, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                mixer = _attention(mx, mw, i, layers)
            elif kind == "channel_delta":
                heads, kvh = _heads(mx, mw)
                mixer = ChannelDeltaConfig(heads, kvh, _pos_int(mx, "dim", mw), _pos_int(mx, "vdim", mw), _pos_int(mx, "conv", mw),
                                           _rank(mx, "decay_rank", f"l{i}.mix.a1", tensor_shapes, mw),
                                           _rank(mx, "gate_rank", f"l{i}.mix.g1", tensor_shapes, mw))
            elif kind == "rglru":
                mixer = RGLRUConfig(_pos_int(mx, "width", mw), _pos_int(mx, "blocks", mw), _pos_int(mx, "conv", mw))
                if mixer.width % mixer.blocks:
                    raise ConfigError(f"config.json: {mw}: width ({mixer.width}) not divisible by blocks ({mixer.blocks})")
            else:
                raise ConfigError(f"config.json: {where}.type = {kind!r}: this design has 'attention', 'channel_delta' "
                                  f"and 'rglru' mixers")
            mlp = lr.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind = {mlp.get('kind')!r}: only 'moe' is computed")
                router = _need(mlp, "router", where + ".mlp")
                ff = ExpertsConfig(_pos_int(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert"),
                                   _pos_int(router, "experts", where + ".mlp.router"), _pos_int(router, "top", where + ".mlp.router"))
                if ff.top > ff.experts:
                    raise ConfigError(f"config.json: {where}.mlp.router: top ({ff.top}) exceeds experts ({ff.experts})")
            layers.append(ZuvulornLayer(kind, mixer, ff))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab, width, eps, streams, tuple(layers), int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS), eos)


def zuvulorn_spec(cfg: ZuvulornConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda tensor, prefix: PartSpec("layernorm", dict(width=W, eps=cfg.eps, tensor=tensor), prefix=prefix)
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        reads = None
        if layer.type == "attention":
            reads = m.kv_from
            mixer = PartSpec("gqa_attention", dict(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
                qkv_bias=False, o_bias=False, scale=m.scale, own_kv=m.kv_from is None, cache_chunk=None,
                qk_norm_eps=cfg.eps, qk_norm_whole=True, gate="head", sink_value=SINK_SCORE,
                position=PartSpec("rotary_scaled", dict(
                    rotary_dim=m.rot_dims, theta=m.rot_base, interleaved=False,
                    scaling=None if m.rot_scaling is None else dict(zip(("factor", "low", "high", "original"), m.rot_scaling)))),
                names=dict(q="q", k="k", v="v", o="o", g="g", q_norm="q.norm", k_norm="k.norm")), prefix=p + "mix.")
        elif layer.type == "channel_delta":
            mixer = PartSpec("channel_delta", dict(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim, conv=m.conv,
                decay_rank=m.decay_rank, gate_rank=m.gate_rank, eps=cfg.eps, unit_eps=UNIT_EPS), prefix=p + "mix.")
        else:
            mixer = PartSpec("rglru", dict(hidden_size=W, width=m.width, blocks=m.blocks, conv=m.conv,
                                           decay_scale=RGLRU_DECAY), prefix=p + "mix.")
        schedule.append(ScheduleEntry(i, reads_cache_of=reads))
        ff = None if layer.mlp is None else PartSpec(
            "moe", dict(hidden_size=W, intermediate_size=layer.mlp.ff, experts=layer.mlp.experts, top=layer.mlp.top),
            prefix=p + "mlp.")
        layers.append(PartSpec("hyper", dict(streams=cfg.streams or 1, learned=cfg.streams is not None, mixer=mixer, mixer_norm=norm("norm1", p), feed_forward=ff,
                                             ff_norm=None if ff is None else norm("norm2", p)), prefix=p))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab, hidden_size=W, tensor="embed")),
        layers=layers, schedule=schedule, final_norm=norm("norm", "final."),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=W, tensor="head")),
        eos_token_id=cfg.eos_token_id)


register_architecture(ARCHITECTURE, ZuvulornConfig.from_dict, zuvulorn_spec, sizes_from_tensors=True)
