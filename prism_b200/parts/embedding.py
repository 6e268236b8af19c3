"""Embedding and output-head parts (andre-fu/prism engine/executor.py:74-75,130)."""

from __future__ import annotations

from typing import Optional

from .base import Embedding, Head, ParamSpec, PartSpec, WeightSource, build_part, register_part
from .. import ops


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    """Row gather, times ``scale`` (in float32; 1: no scaling); the output is the
    float32 residual stream.  ``tensor``: the table's name in the model file.  ``norm``: a norm part applied to
    the gathered rows (in float32, in place).  ``sinusoid_base`` b: a sinusoidal position vector is added to every
    row, entry 2i ``sin(p b^(-2i/width))`` and entry 2i + 1 the cosine of the same angle (frequencies made once on the
    host in float64 and kept in float32; angles and both functions float32).  ``side_tensor`` / ``side_width``: a
    second table ``[vocab, side_width]`` with a row per token that layers read slices of (a per-layer token input);
    the embedding owns it and leaves it in ``ctx.scratch["token_side_table"]`` for the step."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, tensor: str = "embed_tokens.weight",
                 norm: Optional[PartSpec] = None, sinusoid_base: Optional[float] = None, side_tensor: Optional[str] = None,
                 side_width: int = 0):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.scale = float(scale)
        self.tensor = tensor
        self.norm = self.add_child("norm", build_part("norm", norm)) if norm is not None else None
        self.sinusoid_base = None if sinusoid_base is None else float(sinusoid_base)
        if self.sinusoid_base is not None and self.sinusoid_base <= 0:
            raise ValueError(f"the sinusoid's base must be positive, got {sinusoid_base}")
        self.side_tensor, self.side_width = side_tensor, int(side_width)
        if (side_tensor is None) != (self.side_width == 0):
            raise ValueError("a per-token side table needs a tensor name and a width")

    def params(self):
        ps = [ParamSpec("weight", (WeightSource(self.tensor, (self.vocab_size, self.hidden_size)),))]
        if self.side_tensor is not None:
            ps.append(ParamSpec("side", (WeightSource(self.side_tensor, (self.vocab_size, self.side_width)),)))
        return ps

    def on_bound(self):
        self.sin_freq = None
        if self.sinusoid_base is not None:
            W = self.hidden_size
            i = ops.torch.arange((W + 1) // 2, dtype=ops.torch.float64)
            self.sin_freq = (self.sinusoid_base ** (-2.0 * i / W)).to(ops.torch.float32).to(self.device)

    def forward(self, ctx):
        out = ctx.alloc((ctx.T, self.hidden_size), ops.torch.float32)
        ops.embed(ctx.token_ids, self.w["weight"], out, ctx.err, self.scale, ctx.positions, self.sin_freq)
        if self.side_tensor is not None:
            ctx.scratch["token_side_table"] = self.w["side"]
        if self.norm is not None:
            # in place on the float32 rows; the same launch leaves their copy in the compute dtype for the first
            # block's matrix products (a block that norms after the sum looks for it under this key)
            h = self.norm.forward_post(ctx, out, None, 1.0)
            ctx.scratch["postnorm_rows"], ctx.scratch["postnorm_rows_of"] = h, out
        return out


@register_part("head", "linear")
class LinearHead(Head):
    """``logits = h @ W^T`` in float32, no bias or scale; ``softcap`` c: ``logits <- c tanh(logits / c)``.  ``tied_to``
    names the parameter whose storage is shared when the model file has no
    head tensor (engine/weight_manager.py:84-86; the reference copies into a
    second buffer, engine/weight_pool.py:157-160: here it is one buffer)."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: str = None, tensor: str = "weight",
                 softcap: Optional[float] = None):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.tied_to = tied_to
        self.tensor = tensor
        self.softcap = None if softcap is None else float(softcap)
        if self.softcap is not None and self.softcap <= 0:
            raise ValueError(f"a soft cap must be positive, got {softcap}")

    def params(self):
        return [ParamSpec("weight", (WeightSource(self.tensor, (self.vocab_size, self.hidden_size)),),
                          optional=self.tied_to is not None, absent="none", alias_of=self.tied_to)]

    def forward(self, ctx, normed_rows):
        logits = ops.linear(normed_rows, self.w["weight"], None, out_dtype=ops.torch.float32)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits
