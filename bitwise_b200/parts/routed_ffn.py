"""A routed feed-forward: many small experts, a few per row, and a shared expert for all rows.

Router: ``z = W_r h`` in 32-bit, scores ``s = sigmoid(z)``.  The choice uses ``s + correction``
(a stored vector), the weights use ``s`` alone, times ``weight_scale``, not renormalised.  The
experts form ``groups`` equal groups of neighbours; a group counts as the sum of its two largest
corrected scores and only the experts of the ``keep_groups`` best groups can be chosen; of those
the ``top`` with the largest corrected scores are.  An expert is ``W_down (act(W_gate h, W_up
h))`` with ``act(g, u) = g' sigmoid(alpha g') (u' + 1)``, ``g' = min(g, limit)``, ``u' = clamp(u,
-limit, limit)``.  The output is the weighted sum of the chosen experts' outputs, in the order
of choice, plus the shared expert's.

On the device: the router's product, ``route`` (one warp per row), ``group_rows`` (the (row,
choice) pairs listed expert by expert), one grouped product for gate and up of all experts, the
activation, one grouped product for down, and ``combine``, which adds the weighted outputs into
the stream.  Nothing is read back to the host: a step's launches depend on its sizes only.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import KEEP32, MATRIX, ParamSpec
from .base import FeedForward, StepContext, register_feed_forward


class ClampedGLU(FeedForward):
    """gate / up / down with the clamped activation: the shared expert, the form of every
    routed one, and a dense feed-forward of its own."""
    graph_safe = True  # kernels only

    def __init__(self, width: int, inner: int, limit: float, alpha: float):
        self.width, self.inner, self.limit, self.alpha = width, inner, float(limit), float(alpha)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [ParamSpec(f"{prefix}.gate", (self.inner, self.width), MATRIX),
                ParamSpec(f"{prefix}.up", (self.inner, self.width), MATRIX),
                ParamSpec(f"{prefix}.down", (self.width, self.inner), MATRIX)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        self.w_gate_up = torch.cat([state[f"{prefix}.gate"], state[f"{prefix}.up"]], 0).contiguous()
        self.w_down = state[f"{prefix}.down"]

    def param_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor, accumulate: bool = True) -> None:
        """``accumulate`` False: the output is written to ``x`` (float32) instead of added to it."""
        ops, n = ctx.ops, ctx.n
        gate_up = ctx.workspace.rows("glu_gate_up", n, 2 * self.inner, ctx.act_dtype)
        ops.linear(xn, self.w_gate_up, gate_up)
        h = ctx.workspace.rows("glu_h", n, self.inner, ctx.act_dtype)
        ops.glu_clamped(gate_up, h, self.limit, self.alpha)
        ops.linear(h, self.w_down, x, residual=x if accumulate else None)


class RoutedFFN(FeedForward):
    graph_safe = True  # kernels only; nothing of the routing is read on the host

    def __init__(self, width: int, experts: int, top: int, inner: int, limit: float, alpha: float,
                 weight_scale: float = 1.0, groups: int = 1, keep_groups: int = 1, correction: bool = True,
                 shared: Optional[ClampedGLU] = None, scoring: str = "sigmoid", activation: str = "clamped"):
        """``scoring``: "sigmoid" (the weights are the chosen experts' sigmoid scores) or "softmax_top" (the
        largest logits are chosen and the weights are the softmax over the chosen logits only).
        ``activation``: "clamped" (``limit``, ``alpha``) or "silu" (``silu(gate) * up``)."""
        if scoring not in ("sigmoid", "softmax_top") or activation not in ("clamped", "silu"):
            raise ValueError(f"unknown scoring {scoring!r} or activation {activation!r}")
        self.scoring, self.activation = scoring, activation
        if experts <= 0 or groups <= 0 or experts % groups:
            raise ValueError(f"{experts} experts do not form {groups} equal groups")
        if not (0 < keep_groups <= groups) or not (0 < top <= keep_groups * (experts // groups)):
            raise ValueError(f"{top} choices among {keep_groups} groups of {experts // groups} experts")
        self.width, self.experts, self.top, self.inner = width, experts, top, inner
        self.limit, self.alpha, self.weight_scale = float(limit), float(alpha), float(weight_scale)
        self.groups, self.keep_groups, self.has_correction, self.shared = groups, keep_groups, correction, shared
        self.w_router = self.correction = self.w_gate_up = self.w_down = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        specs = []
        for e in range(self.experts):
            specs += [ParamSpec(f"{prefix}.e{e}.gate", (self.inner, self.width), MATRIX),
                      ParamSpec(f"{prefix}.e{e}.up", (self.inner, self.width), MATRIX),
                      ParamSpec(f"{prefix}.e{e}.down", (self.width, self.inner), MATRIX)]
        specs.append(ParamSpec(f"{prefix}.router", (self.experts, self.width), MATRIX))
        if self.has_correction:
            specs.append(ParamSpec(f"{prefix}.correction", (self.experts,), KEEP32))
        if self.shared is not None:
            specs += self.shared.param_specs(f"{prefix}.shared")
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        # all experts in two tensors: [experts, 2 * inner, width] (gate rows, then up rows) and
        # [experts, width, inner]
        self.w_gate_up = torch.stack([torch.cat([state[f"{prefix}.e{e}.gate"], state[f"{prefix}.e{e}.up"]], 0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([state[f"{prefix}.e{e}.down"] for e in range(self.experts)]).contiguous()
        self.w_router = state[f"{prefix}.router"]
        self.correction = state[f"{prefix}.correction"] if self.has_correction else None
        if self.shared is not None:
            self.shared.load_params(state, f"{prefix}.shared")

    def param_bytes(self) -> int:
        own = sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down, self.w_router, self.correction)
                  if t is not None)
        return own + (self.shared.param_bytes() if self.shared is not None else 0)

    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor) -> None:
        self.forward_sum(ctx, xn, None, x)

    def forward_scaled(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor, scale: torch.Tensor) -> None:
        """``x += scale * feed_forward(xn)`` column by column (``scale`` float32 [width])."""
        if self.shared is not None:
            raise NotImplementedError("a scaled sum with a shared expert")
        self.forward_sum(ctx, xn, None, x, scale=scale)

    def forward_sum(self, ctx: StepContext, xn: torch.Tensor, d: Optional[torch.Tensor], x: torch.Tensor,
                    scale: Optional[torch.Tensor] = None) -> None:
        """``x += d + feed_forward(xn)``; ``d`` (float32 rows, or None) is used as scratch."""
        ops, ws, n, top = ctx.ops, ctx.workspace, ctx.n, self.top
        act = ctx.act_dtype
        pairs = n * top
        # routing
        z = ws.rows("route_logits", n, self.experts, torch.float32)
        ops.linear(xn, self.w_router, z)
        chosen = ws.rows("route_chosen", n, top, torch.int32)
        weights = ws.rows("route_weights", n, top, torch.float32)
        ops.route(z, self.correction, self.groups, self.keep_groups, top, self.weight_scale, chosen, weights,
                  softmax_top=self.scoring == "softmax_top")
        lists = ws.rows("route_lists", 3, self.experts + 1, torch.int32)
        order = ws.rows("route_order", n, top, torch.int32)
        place = ws.rows("route_place", n, top, torch.int32)
        ops.group_rows(chosen, self.experts, lists[0], lists[1:3], order, place)
        grouped = (lists[0], lists[1:3], order)
        # the chosen experts, all in one product each for gate/up and down
        gate_up = ws.rows("routed_gate_up", n, top * 2 * self.inner, act).view(pairs, 2 * self.inner)
        sorted_x = None
        if getattr(ops, "grouped_takes_tiles", None) and ops.grouped_takes_tiles(pairs, self.experts, 2 * self.inner, self.width):
            sorted_x = ws.rows("routed_x", n, top * self.width, act).view(pairs, self.width)
        ops.grouped_linear(xn, self.w_gate_up, gate_up, pairs, lists=grouped, order_div=top, sorted_x=sorted_x)
        h = ws.rows("routed_h", n, top * self.inner, act).view(pairs, self.inner)
        if self.activation == "silu":
            ops.swiglu(gate_up, h)
        else:
            ops.glu_clamped(gate_up, h, self.limit, self.alpha)
        y = ws.rows("routed_y", n, top * self.width, torch.float32).view(pairs, self.width)
        ops.grouped_linear(h, self.w_down, y, pairs, lists=grouped, gather=False)
        # the shared expert adds into d (or, without d, into the stream), then everything into the stream
        if self.shared is not None:
            self.shared.forward(ctx, xn, d if d is not None else x)
        ops.combine(x, d, y, place, weights, top, scale=scale)


register_feed_forward("routed", RoutedFFN)
