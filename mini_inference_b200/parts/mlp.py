"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)) (engine/core/model_runner.py:124-131).
gate and up are stored as one [2*inter, hidden] matrix so that one product serves both, as
the reference does with FUSED_PROJ (engine/core/fused_linear.py:173-177,196)."""
from __future__ import annotations

import torch

from .base import Part, WeightSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(Part):
    offers_open = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.get("hidden_size"))
        self.inter = int(spec.get("intermediate_size"))
        self.gate_up = self.down = None

    def weight_specs(self):
        return [WeightSpec("gate_proj", (self.inter, self.hidden)),
                WeightSpec("up_proj", (self.inter, self.hidden)),
                WeightSpec("down_proj", (self.hidden, self.inter))]

    def load(self, tensors, dtype, device):
        self.gate_up = torch.cat([tensors.pop("gate_proj"), tensors.pop("up_proj")], dim=0).contiguous()
        self.down = tensors.pop("down_proj")

    @property
    def open_weight(self):
        return self.down

    @property
    def first_weight(self):
        return self.gate_up

    @property
    def gated_weight(self):
        return self.gate_up

    def first_product_probe(self, ops, rows):
        x = torch.randn(rows, self.hidden, device=self.gate_up.device, dtype=self.gate_up.dtype)
        return lambda w: ops.gated_linear(x, w)

    def forward(self, h, ctx):
        rows, w = self.forward_open(h, ctx)
        return ctx.ops.linear(rows, w)

    def forward_open(self, h, ctx):
        """Everything but the last product: (silu(gate) * up, down weight)."""
        return ctx.ops.gated_linear(h, self.gate_up), self.down


@register_feed_forward("polynorm_mlp")
class PolyNormMLP(Part):
    """down(act(up(h))) with the polynomial-norm activation
        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,   N(y) = y / sqrt(mean(y^2) + eps) over a token's row,
    powers taken element by element; a, b, c, e are the four learned numbers of the tensor `act`.
    The three statistics are float32 sums over the row, made in one pass by one kernel."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.get("hidden_size"))
        self.inter = int(spec.get("intermediate_size"))
        self.eps = float(spec.get("eps"))
        self.up = self.down = self.coef = None

    def weight_specs(self):
        return [WeightSpec("up", (self.inter, self.hidden)), WeightSpec("down", (self.hidden, self.inter)),
                WeightSpec("act", (4,), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.up, self.down = tensors.pop("up"), tensors.pop("down")
        self.coef = tensors.pop("act").float().contiguous()

    @property
    def first_weight(self):
        return self.up

    def forward(self, h, ctx):
        ops = ctx.ops
        return ops.linear(ops.polynorm(ops.linear(h, self.up), self.coef, self.eps), self.down)


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    """A mixture of small gated feed-forwards of which each token uses `top`, plus an optional expert that every token uses.

    Router (float32): s = softmax(W_r h) over all experts; the CHOICE is made on s + correction, confined to the `keep`
    groups (of `count` equal groups of neighbouring experts) whose best choice score is largest; the chosen experts'
    weights are their plain s, not renormalised.  Expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
    y = g * sigmoid(gate_slope * g) * (u + 1), output W_down y.  The token's output is the weighted sum over its experts
    (added in the order of choice, in float32) plus the shared expert's output."""

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.E, self.top, self.F = int(g("hidden_size")), int(g("num_experts")), int(g("top")), int(g("expert_size"))
        self.groups = tuple(g("groups")) if g("groups") else None
        self.limit, self.slope = float(g("limit")), float(g("gate_slope", 1.702))
        self.shared_size = g("shared_size")
        self.shared_limit = float(g("shared_limit")) if self.shared_size else None
        self.router = self.correction = self.w_in = self.w_out = self.shared_in = self.shared_out = None

    def weight_specs(self):
        hid, F = self.hidden, self.F
        specs = [WeightSpec("router", (self.E, hid)), WeightSpec("correction", (self.E,), kind="vector", init="zeros")]
        for e in range(self.E):
            specs += [WeightSpec(f"e{e}.gate", (F, hid)), WeightSpec(f"e{e}.up", (F, hid)), WeightSpec(f"e{e}.down", (hid, F))]
        if self.shared_size:
            S = int(self.shared_size)
            specs += [WeightSpec("shared.gate", (S, hid)), WeightSpec("shared.up", (S, hid)), WeightSpec("shared.down", (hid, S))]
        return specs

    def load(self, tensors, dtype, device):
        self.router = tensors.pop("router").contiguous()                   # stored values as they are; products and sums are float32
        self.correction = tensors.pop("correction").float().contiguous()
        # per expert [gate rows | up rows] and the down matrix, stacked: one grouped product each
        self.w_in = torch.stack([torch.cat([tensors.pop(f"e{e}.gate"), tensors.pop(f"e{e}.up")], dim=0) for e in range(self.E)]).contiguous()
        self.w_out = torch.stack([tensors.pop(f"e{e}.down") for e in range(self.E)]).contiguous()
        if self.shared_size:
            self.shared_in = torch.cat([tensors.pop("shared.gate"), tensors.pop("shared.up")], dim=0).contiguous()
            self.shared_out = tensors.pop("shared.down")

    @property
    def first_weight(self):
        return self.shared_in if self.shared_size else None

    def step_flops(self, rows, pairs):
        return 2 * rows * self.top * 3 * self.F * self.hidden      # the chosen experts' three products (the stacked tensors are not matrices)

    def forward(self, h, ctx):
        ops = ctx.ops
        chosen, weights = ops.route_topk(h, self.router, self.correction, self.top, self.groups)
        shared = None
        if self.shared_size:
            shared = ops.linear(ops.clamped_glu(ops.linear(h, self.shared_in), self.shared_limit, self.slope), self.shared_out)
        return ops.expert_ffn(h, chosen, weights, self.w_in, self.w_out, self.limit, self.slope, shared)
