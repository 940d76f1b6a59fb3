"""RMSNorm: y = w * cast(x32 * rsqrt(mean(x32^2) + eps)), statistics in float32.  The
reference calls the loaded model's norm modules (engine/core/model_runner.py:120-121,133);
here the residual addition that precedes a norm is fused into the same kernel."""
from __future__ import annotations

import torch

from .base import Part, WeightSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    accepts_deferred = True      # delta goes to the kernel namespace untouched
    takes_next_weight = True     # and so does the hint about the weight that is read next

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec.get("size"))
        self.eps = float(spec.get("eps"))
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.size,), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"]

    def forward(self, x, delta, ctx, rows=None, next_weight=None):
        if next_weight is not None and ctx.hints_ok:
            return ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, rows, next_weight=next_weight)
        return ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, rows)


@register_norm("scalar_rmsnorm")
class ScalarRMSNorm(Part):
    """y = g * x / sqrt(mean(x^2) + eps) with ONE learned number g for all coordinates.  The stream x is float32
    whatever the run's dtype: the kernel adds the pending delta (and a pass vector, if one is due) to it in
    float32, stores it back in float32 and hands out the normed rows in the run's dtype."""
    keeps_float32_stream = True

    def __init__(self, spec):
        super().__init__(spec)
        self.eps = float(spec.get("eps"))
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"].float().reshape(1).contiguous()

    def embed(self, ids, table, ctx, float32=True):
        return ctx.ops.embed_scaled_norm(ids, table, self.weight, self.eps, torch.float32 if float32 else ctx.dtype)

    def forward(self, x, delta, ctx, rows=None, pre_add=None):
        return ctx.ops.add_scaled_rmsnorm(x, delta, self.weight, self.eps, rows, pre_add, ctx.dtype)
