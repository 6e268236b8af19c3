"""Norm parts.  ``rmsnorm``: andre-fu/prism's ``fused_rms_norm``
(engine/fused_kernels.py:30-65) with the residual add that precedes it
(engine/executor.py:122-124) fused in, eps and width as parameters.
``layernorm``: mean and variance, a weight and no bias; it also serves a
residual stream kept in several copies (hyper-connections), where the sum
that precedes it is the streams' update and its input their weighted sum."""

from __future__ import annotations

from .base import Norm, ParamSpec, StreamUpdate, WeightSource, register_part
from .. import ops


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """``x * rsqrt(mean(x^2) + eps) * weight``: the weight multiplies (no
    ``1 + w``), no bias, no mean subtraction (fused_kernels.py:41-49)."""

    def __init__(self, width: int, eps: float, tensor: str = "weight", optional: bool = False):
        self.width = int(width)
        self.eps = float(eps)
        self.tensor = tensor          # the weight's name in the model file, after the part's prefix
        self.optional = bool(optional)    # the model file may leave the weight out: the block then skips this norm

    def params(self):
        return [ParamSpec("weight", (WeightSource(self.tensor, (self.width,), "norm"),), optional=self.optional)]

    def forward(self, ctx, residual, delta, rows=None, out_dtype=None):
        """``out_dtype``: the normed rows' dtype where it is not the compute dtype (float32 for a reader that goes on
        in 32-bit)."""
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = ctx.alloc((n, self.width), out_dtype or ctx.dtype)
        ops.add_rmsnorm(residual, delta, self.w["weight"], self.eps, out, rows)
        return out

    def forward_post(self, ctx, x, delta, alpha: float = 1.0):
        """Norm after the sum: ``x <- rmsnorm(alpha * x + delta) * weight`` in place on the float32 rows; returns
        the new rows in the compute dtype (``x`` itself in a float32 engine)."""
        copy = None if ctx.dtype == ops.torch.float32 else ctx.alloc(tuple(x.shape), ctx.dtype)
        ops.scale_add_rmsnorm(x, alpha, delta, self.w["weight"], self.eps, copy)
        return x if copy is None else copy


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight``: the weight multiplies, no bias.  ``rms`` True drops
    the mean (the RMS norm, for a stream kept in several copies)."""

    def __init__(self, width: int, eps: float, tensor: str = "weight", rms: bool = False):
        self.width, self.eps, self.tensor, self.rms = int(width), float(eps), tensor, bool(rms)

    def params(self):
        return [ParamSpec("weight", (WeightSource(self.tensor, (self.width,), "norm"),))]

    def forward_streams(self, ctx, x, streams: int, x_out, update, in_w, rows=None):
        """The residual stream in ``streams`` copies ``x [streams, T, W]`` (or ``[T, W]``: all copies equal): carry out
        ``update`` (a ``StreamUpdate``, a plain delta that every copy receives, or None), write the copies to
        ``x_out`` (None with ``rows``), and return the norm of ``sum_j in_w[j] x_j`` (``in_w`` None: the plain sum) in
        the compute dtype, for all tokens or for ``rows``."""
        n = x.shape[-2] if rows is None else rows.shape[0]
        h = ctx.alloc((n, self.width), ctx.dtype)
        if isinstance(update, StreamUpdate):
            delta, mix, out_w = update.delta, update.mix, update.out
        else:
            delta, mix, out_w = update, None, None
        ops.hyper_norm(x, streams, x_out, delta, mix, out_w, in_w, self.w["weight"], self.eps, h, rows, self.rms)
        return h

    def forward(self, ctx, residual, delta, rows=None):
        if residual.dim() == 3:          # the copies of a stream that hyper-connections keep: their sum is normed
            return self.forward_streams(ctx, residual, residual.shape[0], None if rows is not None else residual, delta,
                                        None, rows)
        if isinstance(delta, StreamUpdate):
            raise ValueError("a stream update needs the residual stream in its copies")
        return self.forward_streams(ctx, residual, 1, None if rows is not None else residual.view((1,) + tuple(residual.shape)),
                                    delta, None, rows)
