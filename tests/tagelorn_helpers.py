"""Shared pieces of the Tagelorn tests: small configurations that differ from one another in every size and
option, model folders with weights drawn here (larger than the framework's random-weights recipe, so that
attention is far from uniform, the distance bias and the sink matter, decays and removal rates lie well inside
(0, 1), the router's scores are spread, and a wrong key, a window that is one token off, a lost state or a missing
sink shows), and the comparison with the plain implementation."""

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

from plain import tagelorn_plain as TP  # noqa: E402
from zuvulorn_helpers import errors, judge, row_error, to_bf16_and_back  # noqa: E402,F401  (generic: rows against a reference)


def attn(heads, kv_heads, dim, vdim=None, scale=0.5, size=16, keep_first=0, bias_rows=8, bias_max=40):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, scale=scale, mask=dict(size=size, keep_first=keep_first),
             bias_rows=bias_rows, bias_max=bias_max)
    if vdim is not None:
        m["vdim"] = vdim
    return m


def delta(heads, dim, decay_rank):
    return dict(heads=heads, dim=dim, decay_rank=decay_rank)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, count=1, keep=None, scale=1.0, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale,
                                                         groups=dict(count=count, keep=count if keep is None else keep)))
    if shared is not None:
        m["shared"] = dict(ff=shared)
    return m


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def model(vocab, width, layers, taps=3, side=None, softcap=None, scale=1.0, eps=1e-5):
    raw = dict(architecture="Tagelorn", vocab=vocab, width=width, norm=dict(eps=eps), canon=dict(taps=taps),
               embedding=dict(scale=scale), layers=layers)
    if side is not None:
        raw["token_side"] = dict(dim=side)
    if softcap is not None:
        raw["logit_softcap"] = softcap
    return raw


# A: sizes that are multiples of nothing; three query heads per kv head, values larger than keys, a window of 9 with two
# kept positions, an odd table of distances that ends inside the window of the next layer; three groups of which two
# are kept; a layer without feed-forward; two taps
CONFIG_A = model(211, 72, taps=2, side=5, softcap=9.0, scale=2.0, layers=[
    layer("attention", attn(6, 2, 12, 20, scale=0.6, size=9, keep_first=2, bias_rows=10, bias_max=30), dense(50)),
    layer("general_delta", delta(3, 7, 5), moe(24, 6, 3, count=3, keep=2, scale=1.7, shared=18)),
    layer("attention", attn(4, 4, 10, 6, scale=0.4, size=40, keep_first=0, bias_rows=6, bias_max=11), None),
    layer("general_delta", delta(2, 20, 3), dense(33)),
])
# B: sizes the tensor-core kernels take, pages of 64, one kv head, a window beyond a page with kept positions, recurrent
# layer first, no token input and no soft cap, four taps
CONFIG_B = model(300, 128, taps=4, layers=[
    layer("general_delta", delta(2, 64, 16), moe(64, 8, 2, count=4, keep=2, scale=2.5, shared=96)),
    layer("attention", attn(4, 1, 64, 32, scale=0.15, size=70, keep_first=5, bias_rows=32, bias_max=200), moe(32, 4, 2)),
    layer("general_delta", delta(4, 32, 8), dense(256)),
    layer("attention", attn(8, 2, 32, 64, scale=0.2, size=33, keep_first=70, bias_rows=16, bias_max=64), dense(96)),
])
# C: everything 1 that can be: one head, one key channel, one tap (no tail), rank 1, one expert, one group, one row of
# distances, a window of one, one kept position, a token input of one channel
CONFIG_C = model(64, 32, taps=1, side=1, softcap=30.0, layers=[
    layer("attention", attn(1, 1, 8, size=1, keep_first=1, bias_rows=1, bias_max=1), moe(16, 1, 1)),
    layer("general_delta", delta(1, 1, 1), moe(8, 2, 2, count=2, keep=2)),
    layer("attention", attn(2, 1, 4, 1, size=5, keep_first=0, bias_rows=2, bias_max=3), None),
])
# D: recurrent layers only: the model has no paged cache group at all; five taps
CONFIG_D = model(90, 48, taps=5, side=8, scale=0.5, layers=[
    layer("general_delta", delta(6, 8, 4), moe(32, 4, 1, count=2, keep=1)),
    layer("general_delta", delta(3, 16, 6), None),
    layer("general_delta", delta(1, 40, 2), dense(24)),
])
# E: a few hundred wide, sizes the tensor-core kernels take throughout but none a power of two times another; heads of 128;
# inner widths that are no multiple of a k-block; every distance beyond the table; attention layers side by side
CONFIG_E = model(500, 384, taps=3, side=16, softcap=20.0, scale=1.5, layers=[
    layer("attention", attn(4, 2, 128, 64, scale=0.09, size=100, keep_first=3, bias_rows=20, bias_max=50), moe(72, 12, 3, count=6, keep=4, scale=2.0, shared=136)),
    layer("attention", attn(6, 2, 64, 32, scale=0.11, size=48, keep_first=9, bias_rows=24, bias_max=180), dense(200)),
    layer("general_delta", delta(2, 128, 24), moe(40, 3, 3)),
])
CONFIGS = {"A": (CONFIG_A, 11, 8), "B": (CONFIG_B, 12, 64), "C": (CONFIG_C, 13, 16), "D": (CONFIG_D, 14, 16), "E": (CONFIG_E, 15, 64)}
LENGTHS = {"A": (61, 9, 2, 34, 1, 27), "B": (150, 31, 77, 64, 3), "C": (40, 1, 17, 5), "D": (45, 3, 22, 1, 30), "E": (130, 40, 66, 7)}


def every_expert(raw: dict) -> dict:
    """The same model with every expert chosen for every token (weights: the scores over their sum, as before).  In
    bfloat16 two experts' choice scores lie within rounding of each other for a token now and then, the choice falls
    the other way, and through the recurrent states every later row of the request moves: no rounding bound holds
    then.  The bfloat16 runs of whole models use these variants, in which rounding has no choice to make; the choice
    itself is covered in float32 and, in bfloat16, by the test of the routing kernel on given logits."""
    out = json.loads(json.dumps(raw))
    for l in out["layers"]:
        if l.get("mlp") is not None and l["mlp"]["kind"] == "moe":
            r = l["mlp"]["router"]
            r["top"] = r["experts"]
            r["groups"]["keep"] = r["groups"]["count"]
    return out


for _name in list(CONFIGS):
    CONFIGS[_name + "x"] = (every_expert(CONFIGS[_name][0]),) + CONFIGS[_name][1:]


def draw_weights(raw: dict, seed: int) -> dict:
    """bf16 tensors keyed by the model file's names."""
    g = torch.Generator().manual_seed(seed)
    W, K = raw["width"], raw["canon"]["taps"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / math.sqrt(i))

    def vec(n, std, mean=0.0):
        return torch.randn(n, generator=g) * std + mean

    t = {"embed": torch.randn(raw["vocab"], W, generator=g) * 0.7, "final.norm": vec(W, 0.1, 1.0)}
    side = (raw.get("token_side") or {}).get("dim")
    if side:
        t["side.embed"] = torch.randn(raw["vocab"], side * len(raw["layers"]), generator=g)
    for i, lr in enumerate(raw["layers"]):
        p, m, q = f"l{i}.", lr["mixer"], f"l{i}.mix."
        t[p + "norm1"], t[p + "canon1"] = vec(W, 0.1, 1.0), torch.randn(W, K, generator=g) * 0.4
        if lr["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            dv = m.get("vdim", d)
            t[q + "q"], t[q + "k"], t[q + "v"] = mat(H * d, W, 2.0), mat(G * d, W, 2.0), mat(G * dv, W, 1.5)
            t[q + "q.b"], t[q + "k.b"], t[q + "v.b"] = vec(H * d, 0.3), vec(G * d, 0.3), vec(G * dv, 0.3)
            t[q + "rel"], t[q + "sink"] = torch.randn(m["bias_rows"], H, generator=g), vec(H, 1.0)
            t[q + "o"] = mat(W, H * dv, 0.8)
        else:
            H, d, R = m["heads"], m["dim"], m["decay_rank"]
            A = H * d
            t[q + "r"], t[q + "k"], t[q + "v"], t[q + "g"] = mat(A, W, 1.5), mat(A, W, 1.5), mat(A, W, 1.5), mat(A, W, 2.0)
            t[q + "a"], t[q + "a.b"] = mat(A, W, 2.0), vec(A, 0.5)
            t[q + "w1"], t[q + "w2"], t[q + "w0"] = mat(R, W, 1.5), mat(A, R, 2.0), vec(A, 1.0)
            t[q + "norm"], t[q + "o"] = vec(A, 0.1, 1.0), mat(W, A, 0.8)
        mlp = lr.get("mlp")
        if mlp is not None:
            t[p + "norm2"] = vec(W, 0.1, 1.0)
            if mlp["kind"] == "dense":
                F = mlp["ff"]
                t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(F, W, 1.5), mat(F, W, 1.2), mat(W, F, 0.8)
            else:
                F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
                t[p + "mlp.router"], t[p + "mlp.correction"] = mat(E, W, 3.0), vec(E, 0.5 / E)
                for e in range(E):
                    t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = mat(F, W, 1.5), mat(W, F, 0.8)
                if mlp.get("shared"):
                    S = mlp["shared"]["ff"]
                    t[p + "mlp.shared.up"], t[p + "mlp.shared.down"] = mat(S, W, 1.5), mat(W, S, 0.8)
        if side:
            t[p + "side.gate"], t[p + "side.proj"], t[p + "side.norm"] = mat(side, W, 1.5), mat(W, side, 1.0), vec(W, 0.05, 0.4)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def file_config(raw: dict) -> dict:
    """The configuration as an exporter writes it: the distance table's rows and the decay's rank are in no key."""
    out = json.loads(json.dumps(raw))
    for l in out["layers"]:
        l["mixer"].pop("decay_rank", None)
        l["mixer"].pop("bias_rows", None)
    return out


_folders = {}


def write_folder(raw: dict, weights: dict, d: str = None) -> str:
    from safetensors.torch import save_file
    d = d or tempfile.mkdtemp(prefix="prism_tagelorn_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(file_config(raw), f)
    save_file(weights, os.path.join(d, "model.safetensors"))
    return d


def model_folder(name: str) -> str:
    if name not in _folders:
        raw, seed, _ = CONFIGS[name]
        _folders[name] = write_folder(raw, draw_weights(raw, seed))
    return _folders[name]


_plain, _logits, _rounding = {}, {}, {}


def plain_weights(name: str, dtype=torch.float64):
    if (name, dtype) not in _plain:
        raw, seed, _ = CONFIGS[name]
        _plain[(name, dtype)] = {k: v.to(dtype) for k, v in draw_weights(raw, seed).items()}
    return _plain[(name, dtype)]


def plain_logits(name: str, seq) -> torch.Tensor:
    """The plain model in float64 on the whole sequence."""
    key = (name, tuple(seq))
    if key not in _logits:
        _logits[key] = TP.forward(CONFIGS[name][0], plain_weights(name), list(seq))
    return _logits[key]


def plain_rounding(name: str, seq, dtype: str = "float32") -> list:
    """Per position: how far rounding alone moves the plain model from itself in float64.  For float32 it is the
    plain model run in float32; for bfloat16 the plain model in float64 with what a 16-bit engine may keep in 16 bits
    rounded to bfloat16."""
    key = (name, tuple(seq), dtype)
    if key not in _rounding:
        ref = plain_logits(name, seq)
        if dtype == "float32":
            low = TP.forward(CONFIGS[name][0], plain_weights(name, torch.float32), list(seq))
        else:
            low = TP.forward(CONFIGS[name][0], plain_weights(name), list(seq), rnd=to_bf16_and_back)
        scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
        _rounding[key] = [row_error(low[p], ref[p], scale) for p in range(len(seq))]
    return _rounding[key]


def compare(name: str, seqs: dict, got: dict, limit: float, ill: float = 0.0, dtype: str = "float32"):
    """Every row the trace produced against the plain model on the whole sequence."""
    errs = []
    for rid, seq in seqs.items():
        errs += errors(plain_logits(name, seq), got, rid, plain_rounding(name, seq, dtype))
    return judge(errs, limit, ill)
