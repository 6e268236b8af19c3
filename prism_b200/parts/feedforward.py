"""Feed-forward parts.  ``swiglu``: andre-fu/prism's dense MLP
(engine/executor.py:125-127): fused gate/up projection, ``silu(gate) * up``,
down projection; no biases (engine/weight_pool.py:194-199).  ``mlp``: up
projection, an elementwise activation, down projection.  ``moe``: a router
sends every token through a few of many small gated layers."""

from __future__ import annotations

from typing import Optional

from .base import DetachedProjection, FeedForward, ParamSpec, PartSpec, WeightSource, build_part, register_part
from .. import ops


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """``names``: the gate, up and down tensors' names in the model file.  ``activation``: what the gate goes
    through, ``silu`` or ``gelu_tanh``."""

    def __init__(self, hidden_size: int, intermediate_size: int,
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight"), activation: str = "silu"):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.names = tuple(names)
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"a gated feed-forward's activation is silu or gelu_tanh, got {activation!r}")
        self.activation = activation

    def params(self):
        H, I = self.hidden_size, self.intermediate_size
        return [
            ParamSpec("gate_up_w", (WeightSource(self.names[0], (I, H)),
                                    WeightSource(self.names[1], (I, H)))),
            ParamSpec("down_w", (WeightSource(self.names[2], (H, I)),)),
        ]

    def forward(self, ctx, x):
        return ops.feed_forward_glu(ctx, x, self.w["gate_up_w"], self.w["down_w"], self.activation)


@register_part("feed_forward", "mlp")
class ActMLP(FeedForward):
    """``down(act(up(x)))`` without gate.  ``activation``: one of ``ops.ACTIVATIONS`` (``relu2``: the square of
    relu; ``gelu_tanh``; ``silu``; ``relu``).  ``names``: the up and down tensors' names in the model file."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2",
                 names=("up_proj.weight", "down_proj.weight")):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r}: one of {sorted(ops.ACTIVATIONS)}")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.activation = activation
        self.names = tuple(names)
        self._own_up = self._own_down = True

    detachable_out = detachable_in = True

    def _sources(self):
        H, I = self.hidden_size, self.intermediate_size
        return WeightSource(self.names[0], (I, H)), WeightSource(self.names[1], (H, I))

    def params(self):
        up, down = self._sources()
        return ([ParamSpec("up_w", (up,))] if self._own_up else []) + ([ParamSpec("down_w", (down,))] if self._own_down else [])

    def detach_out_projection(self):
        self._own_down = False
        return DetachedProjection(self.handed_over(self._sources()[1]), (), self.intermediate_size)

    def detach_in_projection(self):
        self._own_up = False
        return DetachedProjection(self.handed_over(self._sources()[0]), (), self.intermediate_size)

    def forward_inner(self, ctx, x, out, proj=None):
        ops.feed_forward_hidden(ctx, x, self.w.get("up_w"), self.activation, out, hidden=proj)

    def forward(self, ctx, x):
        return ops.feed_forward_act(ctx, x, self.w["up_w"], self.w["down_w"], self.activation)

    def forward_to(self, ctx, x, out):
        """The layer's result into ``out [T, hidden]`` (float32, contiguous): a plane of a stack that the next norm adds up."""
        act = ctx.alloc((x.shape[0], self.intermediate_size), x.dtype)
        ops.feed_forward_hidden(ctx, x, self.w["up_w"], self.activation, act)
        ops.linear(act, self.w["down_w"], None, out=out)


@register_part("feed_forward", "moe")
class MixtureOfExperts(FeedForward):
    """``experts`` gated layers ``down_e(act(gate_e(a)) * up_e(a))`` without biases, of which each token uses ``top``:
    router logits ``z = W_router h`` in float32, scores ``sigmoid(z)`` (``softmax`` True: their softmax), the ``top``
    largest chosen; a choice's weight is its score (``renorm``: divided by the sum of the chosen) and multiplies the
    expert's input, ``out = sum_e expert_e(w_e h)`` (``scale_input`` False: its output).  The result is a float32
    stack with one plane per choice, which the next norm adds to the residual stream.  ``names``: the router's
    tensor, the prefix pattern of an expert (``{e}``: its index), and its gate, up and down tensors.

    ``gated`` False: experts without a gate, ``down_e(act(up_e(a)))``.  ``correction``: the name of a tensor ``[experts]``
    that is added to the scores for the choice only (the weights use the scores without it).  ``groups`` / ``keep``:
    the experts form ``groups`` equal groups of neighbours, a group's score is its largest choice score, and only
    experts of the best ``keep`` groups can be chosen.  ``weight_scale``: a constant on the weights; ``sum_eps``: added
    to the sum that ``renorm`` divides by.  ``shared``: a feed-forward part with ``forward_to`` (``mlp``) that every token
    goes through and whose result is added (its tensors under this part's prefix)."""

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, softmax: bool = False,
                 renorm: bool = False, scale_input: bool = True, activation: str = "silu",
                 names=("router", "e{e}.", "gate", "up", "down"), gated: bool = True, correction: Optional[str] = None,
                 groups: int = 1, keep: Optional[int] = None, weight_scale: float = 1.0, sum_eps: float = 0.0,
                 shared: Optional[PartSpec] = None):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.experts, self.top = int(experts), int(top)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"a token uses {self.top} of {self.experts} experts: between 1 and all of them")
        if activation not in ops.MOE_ACTS:
            raise ValueError(f"activation {activation!r}: one of {sorted(ops.MOE_ACTS)}")
        self.softmax, self.renorm, self.scale_input, self.activation = bool(softmax), bool(renorm), bool(scale_input), activation
        self.names = tuple(names)
        self.gated, self.correction = bool(gated), correction
        self.groups, self.keep = int(groups), int(groups if keep is None else keep)
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.experts} experts in {self.groups} groups of which {self.keep} are kept: the groups must "
                             f"be equal and at least one kept")
        if self.keep * (self.experts // self.groups) < self.top:
            raise ValueError(f"{self.keep} groups of {self.experts // self.groups} experts hold fewer than the {self.top} "
                             f"experts a token uses")
        self.weight_scale, self.sum_eps = float(weight_scale), float(sum_eps)
        self.shared = self.add_child("shared", build_part("feed_forward", shared)) if shared is not None else None

    def params(self):
        H, I, (router, pat, gate, up, down) = self.hidden_size, self.intermediate_size, self.names
        gu, dn = [], []
        for e in range(self.experts):
            p = pat.format(e=e)
            gu += ([WeightSource(p + gate, (I, H))] if self.gated else []) + [WeightSource(p + up, (I, H))]
            dn.append(WeightSource(p + down, (H, I)))
        ps = [ParamSpec("router_w", (WeightSource(router, (self.experts, H)),)),
              ParamSpec("gate_up_w", tuple(gu)), ParamSpec("down_w", tuple(dn))]
        if self.correction is not None:
            ps.append(ParamSpec("correction", (WeightSource(self.correction, (self.experts,), "bias"),)))
        return ps

    def on_bound(self):
        self.choice = ops.MoeChoice(self.w.get("correction"), self.groups, self.keep, self.weight_scale, self.sum_eps)

    def forward(self, ctx, x):
        H, I, E = self.hidden_size, self.intermediate_size, self.experts
        logits = ops.linear(x, self.w["router_w"], None, out_dtype=ops.torch.float32)
        y = ops.moe_feed_forward(ctx, x, logits, self.w["gate_up_w"].view(E, (2 if self.gated else 1) * I, H),
                                 self.w["down_w"].view(E, H, I), self.top, self.softmax, self.renorm, self.scale_input,
                                 self.activation, self.gated, self.choice, extra_planes=0 if self.shared is None else 1)
        if self.shared is not None:
            self.shared.forward_to(ctx, x, y[self.top])          # the shared expert's result is the stack's last plane
        return y
