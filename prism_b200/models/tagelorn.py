"""Tagelorn: a small decoder whose ``config.json`` lists its layers one by one.
Its typed configuration, its layer plan and its entry in the architecture
registry; everything this engine knows about the design by name is here.

The design, as this file builds it from the parts:

* embedding rows times ``embedding.scale``, plus a sinusoidal position vector
  (entry 2i the sine, entry 2i + 1 the cosine of ``p 10000^(-2i/width)``);
* every layer is a pre-norm block (RMS norms ``norm1`` / ``norm2``) whose mixer
  reads ``h + conv(h)``, a causal convolution over time of ``canon.taps`` taps
  per channel (``l<i>.canon1``) beside a skip path (a file without ``canon``
  has no such convolution); the feed-forward may be
  absent; after it comes a per-layer token input: a slice of the row of
  ``side.embed`` that belongs to the token, gated by ``gelu_tanh(side.gate x)``,
  projected back (``side.proj``), RMS-normed with ``side.norm`` and added;
* mixer ``attention``: grouped-query attention with biases on q, k and v; q and
  k divided by their root mean square per head (no weights); no rotation; an
  explicit score scale; a learned bias by distance (``rel``, rows by logarithmic
  buckets up to ``bias_max``); a sliding window that keeps the first positions;
  a learned sink per head in the softmax's denominator; values of their own size;
* mixer ``general_delta``: the generalized delta rule (``parts/recurrent.py``)
  with a decay from a low-rank product and a removal rate per key channel;
* feed-forward ``dense``: ``down(gelu_tanh(gate h) * up h)``; ``moe``: softmax
  router with a correction for the choice, groups of experts of which the best
  are kept, weights renormalised and scaled, experts ``down(relu(up h)^2)``, and
  a shared expert of the same form for every token;
* the final RMS norm (``final.norm``), the embedding table as the head, and a
  soft cap on the logits.

Two sizes are in no key: the rows of an attention layer's distance-bias table
are the shape of ``l<i>.mix.rel`` and the rank of a general-delta layer's decay
is the shape of ``l<i>.mix.w1`` (``bias_rows`` / ``decay_rank`` in the mixer's
configuration where there is no file).  The design puts no limit on positions;
block tables need a width, so ``max_positions`` (an engine knob, default 131072)
may be given in the file.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from ..config.model_config import ConfigError
from ..model_registry import register_architecture
from ..parts.base import PartSpec
from .decoder import ModelSpec

ARCHITECTURE = "Tagelorn"
DEFAULT_MAX_POSITIONS = 131072
SINUSOID_BASE = 10000.0          # the design fixes these
UNIT_EPS = 1e-6                  # the unit key: k / sqrt(sum k^2 + 1e-6)
DECAY_RATE = math.exp(-0.5)      # the decay: exp(-exp(-1/2) sigmoid(..))
WEIGHT_SUM_EPS = 1e-20           # an expert's weight: score / (sum of the chosen + 1e-20)


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = int(_need(d, key, where))
    if v < 1:
        raise ConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _from_shape(mx, key, tensor, shapes, where, what):
    value = mx.get(key)
    if shapes is not None:
        shape = shapes.get(tensor)
        if shape is None or len(shape) != 2:
            raise ConfigError(f"the model file has no matrix '{tensor}', whose rows are {what}")
        value = shape[0]
    if value is None:
        raise ConfigError(f"config.json: {where} has no '{key}' (without a model file nothing else gives it)")
    return int(value)


@dataclass(frozen=True)
class BiasedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]         # None: no window
    keep_first: int
    bias_rows: Optional[int]      # None: no bias by distance
    bias_max: Optional[int]


@dataclass(frozen=True)
class GeneralDeltaConfig:
    heads: int
    dim: int
    decay_rank: int


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class RoutedConfig:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int
    scale: float
    shared_ff: Optional[int]


@dataclass(frozen=True)
class TagelornLayer:
    type: str                     # "attention" | "general_delta"
    mixer: object
    mlp: object                   # DenseConfig, RoutedConfig or None


def _mlp(mlp, where):
    if mlp is None:
        return None
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return DenseConfig(_pos_int(mlp, "ff", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind = {kind!r}: this design has 'dense' and 'moe' feed-forwards")
    router = _need(mlp, "router", where)
    rw = where + ".router"
    experts, top = _pos_int(router, "experts", rw), _pos_int(router, "top", rw)
    groups = router.get("groups") or {}
    count = int(groups.get("count") or 1)
    keep = int(groups.get("keep") or count)
    if count < 1 or experts % count or not 1 <= keep <= count:
        raise ConfigError(f"config.json: {rw}.groups: {experts} experts do not form {count} equal groups of which {keep} are kept")
    if top > keep * (experts // count):
        raise ConfigError(f"config.json: {rw}: top ({top}) exceeds the experts of the {keep} kept groups")
    shared = mlp.get("shared")
    return RoutedConfig(_pos_int(_need(mlp, "expert", where), "ff", where + ".expert"), experts, top, count, keep,
                        float(router.get("scale", 1.0)), None if not shared else _pos_int(shared, "ff", where + ".shared"))


@dataclass(frozen=True)
class TagelornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    taps: Optional[int]           # None: the layers have no input convolution
    side_dim: Optional[int]           # None: no per-layer token input
    logit_softcap: Optional[float]
    layers: Tuple[TagelornLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict, tensor_shapes: Optional[dict] = None) -> "TagelornConfig":
        vocab, width = _pos_int(raw, "vocab", "the model"), _pos_int(raw, "width", "the model")
        eps = float(_need(_need(raw, "norm", "the model"), "eps", "norm"))
        scale = float((raw.get("embedding") or {}).get("scale", 1.0))
        taps = None if not raw.get("canon") else _pos_int(raw["canon"], "taps", "canon")     # no key: no input convolution
        side = raw.get("token_side")
        side_dim = None if not side else _pos_int(side, "dim", "token_side")
        cap = raw.get("logit_softcap")
        if cap is not None and float(cap) <= 0:
            raise ConfigError(f"config.json: logit_softcap must be positive, got {cap}")
        layers_raw = _need(raw, "layers", "the model")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            kind, mx = _need(lr, "type", where), _need(lr, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                heads = _pos_int(mx, "heads", mw)
                kvh = int(mx.get("kv_heads") or heads)
                if kvh < 1 or heads % kvh:
                    raise ConfigError(f"config.json: {mw}: heads ({heads}) not divisible by kv_heads ({kvh})")
                dim = _pos_int(mx, "dim", mw)
                mask = mx.get("mask")                     # no mask: every earlier key is visible
                window = None if not mask else _pos_int(mask, "size", mw + ".mask")
                keep_first = 0 if not mask else int(mask.get("keep_first") or 0)
                if keep_first < 0:
                    raise ConfigError(f"config.json: {mw}.mask.keep_first must not be negative")
                bias_max = None if mx.get("bias_max") is None else _pos_int(mx, "bias_max", mw)      # no key: no bias by distance
                rows = None if bias_max is None else _from_shape(mx, "bias_rows", f"l{i}.mix.rel", tensor_shapes, mw,
                                                                 "the distance-bias table's")
                mixer = BiasedAttentionConfig(heads, kvh, dim, int(mx.get("vdim") or dim), float(_need(mx, "scale", mw)), window,
                                              keep_first, rows, bias_max)
            elif kind == "general_delta":
                mixer = GeneralDeltaConfig(_pos_int(mx, "heads", mw), _pos_int(mx, "dim", mw),
                                           _from_shape(mx, "decay_rank", f"l{i}.mix.w1", tensor_shapes, mw, "the decay's rank"))
            else:
                raise ConfigError(f"config.json: {where}.type = {kind!r}: this design has 'attention' and 'general_delta' mixers")
            layers.append(TagelornLayer(kind, mixer, _mlp(lr.get("mlp"), where + ".mlp")))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab, width, eps, scale, taps, side_dim, None if cap is None else float(cap), tuple(layers),
                   int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS), eos)


def tagelorn_spec(cfg: TagelornConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda tensor, prefix: PartSpec("rmsnorm", dict(width=W, eps=cfg.eps, tensor=tensor), prefix=prefix)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("gqa_attention", dict(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
                qkv_bias=True, o_bias=False, scale=m.scale, window=m.window, keep_first=m.keep_first, sink=True,
                qk_norm_eps=cfg.eps, qk_norm_weight=False,
                dist_bias=None if m.bias_max is None else dict(rows=m.bias_rows, far=m.bias_max),
                names=dict(q="q", k="k", v="v", o="o", q_b="q.b", k_b="k.b", v_b="v.b", sink="sink", rel="rel")),
                prefix=p + "mix.")
        else:
            mixer = PartSpec("general_delta", dict(hidden_size=W, num_heads=m.heads, head_dim=m.dim, decay_rank=m.decay_rank,
                                                   eps=cfg.eps, decay_rate=DECAY_RATE, unit_eps=UNIT_EPS), prefix=p + "mix.")
        ff = None
        if isinstance(layer.mlp, DenseConfig):
            ff = PartSpec("swiglu", dict(hidden_size=W, intermediate_size=layer.mlp.ff, names=("gate", "up", "down"),
                                         activation="gelu_tanh"), prefix=p + "mlp.")
        elif isinstance(layer.mlp, RoutedConfig):
            r = layer.mlp
            shared = None if r.shared_ff is None else PartSpec(
                "mlp", dict(hidden_size=W, intermediate_size=r.shared_ff, activation="relu2", names=("up", "down")),
                prefix=p + "mlp.shared.")
            ff = PartSpec("moe", dict(
                hidden_size=W, intermediate_size=r.ff, experts=r.experts, top=r.top, softmax=True, renorm=True,
                scale_input=False, activation="relu2", gated=False, correction="correction", groups=r.groups, keep=r.keep,
                weight_scale=r.scale, sum_eps=WEIGHT_SUM_EPS, shared=shared), prefix=p + "mlp.")
        side = None if cfg.side_dim is None else dict(dim=cfg.side_dim, index=i, eps=cfg.eps, activation="gelu_tanh")
        layers.append(PartSpec("prenorm", dict(
            mixer=mixer, feed_forward=ff, mixer_norm=norm("norm1", p), ff_norm=None if ff is None else norm("norm2", p),
            hidden_size=W, input_conv=cfg.taps, conv_tensor="canon1", token_side=side), prefix=p))
    n_layers = len(cfg.layers)
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token", dict(
            vocab_size=cfg.vocab, hidden_size=W, scale=cfg.embedding_scale, tensor="embed", sinusoid_base=SINUSOID_BASE,
            side_tensor=None if cfg.side_dim is None else "side.embed",
            side_width=0 if cfg.side_dim is None else cfg.side_dim * n_layers)),
        layers=layers, final_norm=norm("norm", "final."),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=W, tied_to="embedding.weight", tensor="head",
                                     softcap=cfg.logit_softcap)),
        eos_token_id=cfg.eos_token_id)


register_architecture(ARCHITECTURE, TagelornConfig.from_dict, tagelorn_spec, sizes_from_tensors=True)
