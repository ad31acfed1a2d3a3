"""RMSNorm: y = (x * inv) * w, inv = 1 / sqrt(mean(x^2) + eps), no offset on the weight
(src/kernels.cpp:264-271), and layer norm with a weight and no bias: y = (x - mean) / sqrt(var +
eps) * w with var the mean of the squared deviations.  The statistics are always computed in
32-bit.  ``suffix`` is what follows the prefix in the tensor's name (".weight" in Hugging Face
checkpoints, nothing where the tensor carries the norm's own name).  A norm may hold its weight
around zero (``offset`` 1: the factor is 1 + w) and carry a constant ``gain`` (a model's output
scale applied with its last norm); both are folded into the 32-bit weight once, when it is loaded:
the kernels multiply by ``(offset + w) * gain``."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import KEEP32, ParamSpec
from .base import Norm, StepContext, register_norm


class RMSNorm(Norm):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, width: int, eps: float, suffix: str = ".weight", offset: float = 0.0, gain: float = 1.0):
        self.width = width
        self.eps = float(eps)
        self.suffix = suffix
        self.offset, self.gain = float(offset), float(gain)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [ParamSpec(prefix + self.suffix, (self.width,), KEEP32, init="zeros" if self.offset else "ones")]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        w = state[prefix + self.suffix]
        if self.offset:
            w = w + self.offset
        if self.gain != 1.0:
            w = w * self.gain
        self.weight = w

    def param_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx: StepContext, x, out, rows=None) -> None:
        ctx.ops.rmsnorm(x, self.weight, self.eps, out, rows)

    def forward_residual(self, ctx: StepContext, d, x) -> None:
        """x += norm(d): the norm of a sublayer's output ``d`` (float32) on its way into the stream."""
        ctx.ops.rmsnorm_residual(d, self.weight, self.eps, x)

    def forward_residual_then(self, ctx: StepContext, d, x, nxt: "RMSNorm", out) -> None:
        """``forward_residual(d, x)`` followed by ``nxt.forward(x, out)``, in one kernel where ``nxt`` is a
        norm of this kind."""
        if type(nxt) is not RMSNorm or nxt.width != self.width:
            self.forward_residual(ctx, d, x)
            nxt.forward(ctx, x, out)
            return
        ctx.ops.rmsnorm_residual(d, self.weight, self.eps, x, next_weight=nxt.weight, next_eps=nxt.eps, next_out=out)


class LayerNorm(RMSNorm):
    """Mean and variance over the row; a weight, no bias.  ``out`` may be float32 (also ``x``
    itself: the norm then works in place on the stream) or the activation type."""

    def forward(self, ctx, x, out, rows=None) -> None:
        ctx.ops.layernorm(x, self.weight, self.eps, out, rows)

    def forward_pair(self, ctx, x, out, other: "LayerNorm", other_out) -> None:
        """This norm and ``other`` of the same rows in one pass: they share mean and variance."""
        if other.eps != self.eps or other.width != self.width:
            self.forward(ctx, x, out)
            other.forward(ctx, x, other_out)
            return
        ctx.ops.layernorm(x, self.weight, self.eps, out, None, other.weight, other_out)

    def forward_residual(self, ctx: StepContext, d, x) -> None:
        """x += norm(d) with the row statistics of the sublayer's output ``d`` (float32); a constant factor on
        what is added is this norm's ``gain``."""
        ctx.ops.layernorm_residual(d, self.weight, self.eps, x)

    def forward_residual_then(self, ctx: StepContext, d, x, nxt: "LayerNorm", out) -> None:
        if type(nxt) is not LayerNorm or nxt.width != self.width:
            self.forward_residual(ctx, d, x)
            nxt.forward(ctx, x, out)
            return
        ctx.ops.layernorm_residual(d, self.weight, self.eps, x, next_weight=nxt.weight, next_eps=nxt.eps, next_out=out)


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
