"""Shared pieces of the Zuvulorn tests: small configurations that differ from one another in every size and
option, model folders with weights drawn here (larger than the framework's random-weights recipe, so that
attention is far from uniform, decays are neither 0 nor 1, the copies of the residual stream differ and a wrong
key, a lost state or a missing sink shows), and the comparison with the plain implementation."""

from __future__ import annotations

import json
import math
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

from plain import zuvulorn_plain as ZP  # noqa: E402


def attn(heads, kv_heads, dim, vdim=None, scale=None, rot_dims=None, base=10000.0, scaling=None, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, scale=scale if scale is not None else dim ** -0.5)
    if vdim is not None:
        m["vdim"] = vdim
    if rot_dims is None:
        rot_dims = dim // 2 * 2
    if rot_dims:
        m["rot"] = dict(base=base, dims=rot_dims)
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, decay_rank=decay_rank, gate_rank=gate_rank)


def rglru(width, blocks, conv):
    return dict(width=width, blocks=blocks, conv=conv)


def experts(ff, n, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=n, top=top))


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def model(vocab, width, layers, streams=2, eps=1e-6):
    raw = dict(architecture="Zuvulorn", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if streams is not None:
        raw["streams"] = streams
    return raw


# A: three copies of the stream; three query heads per kv head, values larger than keys, part of a head rotated
# with rescaled frequencies in all three bands, a layer on another's keys, two value heads per q/k head in the
# delta rule, ranks that differ, five blocks, two of six experts, a layer without feed-forward
CONFIG_A = model(211, 72, streams=3, eps=1e-5, layers=[
    layer("attention", attn(6, 2, 16, 24, scale=0.3, rot_dims=8, base=50.0, scaling=(4.0, 1.0, 3.0, 64)), experts(24, 6, 2)),
    layer("channel_delta", delta(4, 2, 12, 20, 3, 5, 7), experts(40, 3, 1)),
    layer("attention", attn(6, 2, 16, 24, scale=0.2, rot_dims=8, base=50.0, scaling=(4.0, 1.0, 3.0, 64), kv_from=0), None),
    layer("rglru", rglru(40, 5, 4), experts(16, 4, 3)),
])
# B: sizes the tensor-core kernels take, pages of 64, one kv head, whole heads rotated without rescaling, the
# recurrent layers first, the layer on another's keys last with other layers between
CONFIG_B = model(300, 128, streams=2, layers=[
    layer("rglru", rglru(192, 3, 2), experts(64, 8, 3)),
    layer("attention", attn(4, 1, 64, 32, scale=0.11, rot_dims=64, base=30000.0), experts(96, 4, 2)),
    layer("channel_delta", delta(2, 2, 64, 32, 4, 16, 8), experts(64, 8, 1)),
    layer("attention", attn(4, 1, 64, 32, scale=0.15, rot_dims=64, base=30000.0, kv_from=1), experts(32, 2, 2)),
])
# C: everything 1 that can be: one copy of the stream (with connection weights), one head, one block, one tap (no
# tail), rank 1, one expert, no rotation in one layer
CONFIG_C = model(64, 32, streams=1, layers=[
    layer("attention", attn(1, 1, 8, rot_dims=0), experts(16, 1, 1)),
    layer("rglru", rglru(8, 1, 1), experts(8, 2, 2)),
    layer("channel_delta", delta(1, 1, 1, 1, 1, 1, 1), None),
    layer("attention", attn(1, 1, 8, rot_dims=2, kv_from=0), experts(8, 2, 1)),
])
# D: no copies at all (the file has no connection weights: plain pre-norm layers); sizes that are multiples of
# nothing; every expert chosen; as many kv heads as heads
CONFIG_D = model(77, 52, streams=None, layers=[
    layer("attention", attn(3, 3, 10, 14, rot_dims=6, base=100.0), experts(18, 5, 5)),
    layer("rglru", rglru(33, 3, 3), experts(9, 7, 2)),
    layer("channel_delta", delta(3, 1, 7, 5, 2, 3, 2), experts(11, 3, 2)),
])
# E: recurrent layers only: the model has no paged cache group at all; four copies
CONFIG_E = model(90, 48, streams=4, layers=[layer("rglru", rglru(64, 4, 4), experts(32, 4, 1)),
                                            layer("channel_delta", delta(6, 3, 8, 8, 3, 4, 4), None),
                                            layer("rglru", rglru(24, 2, 2), None)])
# F: a few hundred wide, sizes the tensor-core kernels take throughout but none a power of two times another: heads of
# 128 with values of 64 and half a head rotated, four of twelve experts, inner widths of 72 and 136 (no multiple of a
# k-block), values wider than keys in the delta rule, four copies, the layer on another's keys without feed-forward
CONFIG_F = model(500, 320, streams=4, eps=1e-5, layers=[
    layer("rglru", rglru(384, 3, 2), experts(72, 12, 4)),
    layer("channel_delta", delta(4, 2, 64, 128, 4, 24, 40), experts(136, 5, 2)),
    layer("attention", attn(8, 2, 128, 64, scale=0.05, rot_dims=64, base=8000.0, scaling=(8.0, 1.0, 4.0, 128)), experts(72, 12, 4)),
    layer("attention", attn(8, 2, 128, 64, scale=0.07, rot_dims=64, base=8000.0, scaling=(8.0, 1.0, 4.0, 128), kv_from=2), None),
    layer("attention", attn(4, 4, 32, 32, scale=0.2, rot_dims=32, base=1000.0), experts(40, 3, 3)),
])
CONFIGS = {"F": (CONFIG_F, 16, 64), "A": (CONFIG_A, 11, 8), "B": (CONFIG_B, 12, 64), "C": (CONFIG_C, 13, 16), "D": (CONFIG_D, 14, 8),
           "E": (CONFIG_E, 15, 16)}      # config, seed, page size


def every_expert(raw: dict) -> dict:
    """The same model with every expert chosen for every token (weights: their scores, as before).  In bfloat16 two
    experts' scores lie within rounding of each other for a token now and then, the choice falls the other way, and
    through the recurrent states every later row of the request moves: no rounding bound holds then.  The bfloat16
    runs of whole models use these variants, in which rounding has no choice to make; the choice itself is
    covered in float32 and, in bfloat16, by the test of the experts' kernels on given scores."""
    out = json.loads(json.dumps(raw))
    for l in out["layers"]:
        if l.get("mlp") is not None:
            l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
    return out


for _name in list(CONFIGS):
    CONFIGS[_name + "x"] = (every_expert(CONFIGS[_name][0]),) + CONFIGS[_name][1:]


def draw_weights(raw: dict, seed: int) -> dict:
    """bf16 tensors keyed by the model file's names.  Matrices ``normal(0, 1 / sqrt(in))`` times a gain, so that
    activations stay of order one through the layers, attention scores spread over several units (some rows far
    below the sink's zero, some far above), decays lie well inside (0, 1), the gates are neither shut nor open,
    the router's scores are spread, and the copies of the stream are read and written with unequal weights."""
    g = torch.Generator().manual_seed(seed)
    W, s = raw["width"], raw.get("streams")

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, std, mean=0.0):
        return torch.randn(n, generator=g) * std + mean

    t = {"embed": torch.randn(raw["vocab"], W, generator=g) * 0.7, "final.norm": vec(W, 0.1, 1.0), "head": mat(raw["vocab"], W)}
    for i, lr in enumerate(raw["layers"]):
        p, m, q = f"l{i}.", lr["mixer"], f"l{i}.mix."
        t[p + "norm1"] = vec(W, 0.1, 1.0)
        subs = [1] + ([2] if lr.get("mlp") is not None else [])
        if s is not None:
            for j in subs:
                t[f"{p}hc{j}.in"] = vec(s, 0.3, 0.8)
                t[f"{p}hc{j}.out"] = vec(s, 0.3, 0.7)
                t[f"{p}hc{j}.mix"] = torch.eye(s) * 0.8 + torch.randn(s, s, generator=g) * 0.25
        if lr["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            dv = m.get("vdim", d)
            t[q + "q"], t[q + "q.norm"] = mat(H * d, W, 2.0), vec(H * d, 0.4, 2.5)
            if m.get("kv_from") is None:
                t[q + "k"], t[q + "v"], t[q + "k.norm"] = mat(G * d, W, 2.0), mat(G * dv, W, 1.5), vec(G * d, 0.4, 2.5)
            t[q + "g"], t[q + "o"] = mat(H, W, 2.0), mat(W, H * dv, 0.8)
        elif lr["type"] == "channel_delta":
            H, G, d, dv, K, Ra, Rg = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], m["decay_rank"], m["gate_rank"]
            t[q + "q"], t[q + "k"], t[q + "v"] = mat(G * d, W, 2.0), mat(G * d, W, 2.0), mat(H * dv, W, 1.5)
            for n_, c in (("q", G * d), ("k", G * d), ("v", H * dv)):
                t[q + n_ + ".conv"] = torch.randn(c, K, generator=g) * 0.6
            t[q + "b"], t[q + "a1"], t[q + "a2"] = mat(H, W, 2.0), mat(Ra, W, 1.5), mat(H * d, Ra, 1.5)
            t[q + "A_log"], t[q + "dt_bias"] = vec(H, 0.5, -0.5), vec(H * d, 0.7)
            t[q + "g1"], t[q + "g2"] = mat(Rg, W, 1.5), mat(H * dv, Rg, 2.0)
            t[q + "norm"], t[q + "o"] = vec(dv, 0.1, 1.0), mat(W, H * dv, 0.8)
        else:
            C, nb, K = m["width"], m["blocks"], m["conv"]
            bs = C // nb
            t[q + "y"], t[q + "y.b"], t[q + "x"], t[q + "x.b"] = mat(C, W, 1.5), vec(C, 0.3), mat(C, W, 1.5), vec(C, 0.3)
            t[q + "conv"], t[q + "conv.b"] = torch.randn(C, K, generator=g) * 0.6, vec(C, 0.2)
            t[q + "ra"], t[q + "ri"] = (torch.randn(nb, bs, bs, generator=g) * (1.5 / math.sqrt(bs)),
                                        torch.randn(nb, bs, bs, generator=g) * (1.5 / math.sqrt(bs)))
            t[q + "ra.b"], t[q + "ri.b"] = vec(C, 0.5).view(nb, bs), vec(C, 0.5).view(nb, bs)
            t[q + "lam"], t[q + "o"] = vec(C, 1.0, -2.5), mat(W, C, 0.8)
        if lr.get("mlp") is not None:
            F, E = lr["mlp"]["expert"]["ff"], lr["mlp"]["router"]["experts"]
            t[p + "norm2"], t[p + "mlp.router"] = vec(W, 0.1, 1.0), mat(E, W, 3.0)
            for e in range(E):
                t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = mat(F, W, 1.5), mat(F, W, 1.2), mat(W, F, 0.8)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def file_config(raw: dict) -> dict:
    """The configuration as an exporter writes it: the ranks of the low-rank products are in no key of config.json."""
    out = json.loads(json.dumps(raw))
    for l in out["layers"]:
        l["mixer"].pop("decay_rank", None)
        l["mixer"].pop("gate_rank", None)
    return out


_folders = {}


def write_folder(raw: dict, weights: dict, d: str = None) -> str:
    from safetensors.torch import save_file
    d = d or tempfile.mkdtemp(prefix="prism_zuvulorn_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(file_config(raw), f)
    save_file(weights, os.path.join(d, "model.safetensors"))
    return d


def model_folder(name: str) -> str:
    if name not in _folders:
        raw, seed, _ = CONFIGS[name]
        _folders[name] = write_folder(raw, draw_weights(raw, seed))
    return _folders[name]


_plain = {}


def plain_weights(name: str, dtype=torch.float64):
    if (name, dtype) not in _plain:
        raw, seed, _ = CONFIGS[name]
        _plain[(name, dtype)] = {k: v.to(dtype) for k, v in draw_weights(raw, seed).items()}
    return _plain[(name, dtype)]


_logits = {}


def plain_logits(name: str, seq) -> torch.Tensor:
    """The plain model in float64 on the whole sequence."""
    key = (name, tuple(seq))
    if key not in _logits:
        _logits[key] = ZP.forward(CONFIGS[name][0], plain_weights(name), list(seq))
    return _logits[key]


_rounding = {}


def to_bf16_and_back(x):
    return x.to(torch.bfloat16).to(x.dtype)


def plain_rounding(name: str, seq, dtype: str = "float32") -> list:
    """Per position: how far rounding alone moves the plain model from itself in float64 (``row_error``).  For
    float32 it is the plain model run in float32; for bfloat16 the plain model in float64 with what a 16-bit engine
    may keep in 16 bits rounded to bfloat16.  Where a head's read-out is divided by a root mean square close to
    zero, or a decay lies close to one, this is many times the usual; what arithmetic alone does to a row is not
    held against the engine."""
    key = (name, tuple(seq), dtype)
    if key not in _rounding:
        ref = plain_logits(name, seq)
        if dtype == "float32":
            low = ZP.forward(CONFIGS[name][0], plain_weights(name, torch.float32), list(seq))
        else:
            low = ZP.forward(CONFIGS[name][0], plain_weights(name), list(seq), rnd=to_bf16_and_back)
        scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
        _rounding[key] = [row_error(low[p], ref[p], scale) for p in range(len(seq))]
    return _rounding[key]


def row_error(got: torch.Tensor, ref: torch.Tensor, scale: float) -> float:
    """Root mean square over the vocabulary of the difference with its mean taken off, over ``scale``."""
    d = got.double() - ref.double()
    d = d - d.mean()
    return float(torch.sqrt((d * d).mean())) / scale


def errors(ref: torch.Tensor, rows: dict, rid, rounding=None) -> list:
    """``(error, request, position)`` of every row that ``rows`` has; ``rounding``: per position, an error that
    arithmetic alone causes there - three times as much is taken off the row's."""
    scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    out = []
    for pos in range(ref.shape[0]):
        if (rid, pos) in rows:
            e = row_error(rows[(rid, pos)], ref[pos], scale)
            if rounding is not None:
                e = max(0.0, e - 3.0 * rounding[pos])
            out.append((e if e == e else math.inf, rid, pos))
    return out


def judge(errs: list, limit: float, ill: float = 0.0):
    """No row over ``limit`` - but for a share ``ill`` of them, which may lie up to eight times over it.  (In
    bfloat16 only: where a head's read-out is divided by a root mean square close to zero, or two experts' scores
    lie within rounding of each other, rounding decides, and that row - not the ones around it - moves.  A wrong
    key or a lost state moves most rows that follow it, and moves them in float32 too, where no row may differ.)"""
    errs = sorted(errs, reverse=True)
    over = [x for x in errs if not x[0] <= limit]
    assert len(over) <= ill * len(errs) and (not over or over[0][0] <= 8 * limit), \
        f"{len(over)} of {len(errs)} rows over {limit:.1e}; worst {over[0][0]:.3e} at {over[0][1:]}"
    return errs[0] if errs else None


def compare(name: str, seqs: dict, got: dict, limit: float, ill: float = 0.0, dtype: str = "float32"):
    """Every row the trace produced against the plain model on the whole sequence."""
    errs = []
    for rid, seq in seqs.items():
        errs += errors(plain_logits(name, seq), got, rid, plain_rounding(name, seq, dtype))
    return judge(errs, limit, ill)
