"""A per-layer token input: every layer adds a gated, normed projection of a small per-token vector.

One table ``[vocab, layers * dim]`` for the whole model (:class:`TokenSideTable`); layer i reads columns
``[i * dim, (i + 1) * dim)`` of its row's token, ``e``.  With the stream ``x`` after the layer's sublayers:
``g = gelu_tanh(W_gate x) * e``, ``y = W_proj g``, and the layer adds ``mult * y / rms(y) * w`` to the stream
(a root-mean-square norm with a plain weight).  The two products may run in the activation type; the gate's
activation, the norm and the sum are 32-bit.  The sum itself is formed by the block, which may join it with
what it does next on the stream (``ops.normed_add_mix``).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import KEEP32, MATRIX, ParamSpec
from .base import Part, StepContext


class TokenSideTable(Part):
    """The table that all layers' token inputs share; declared and loaded once per model."""
    graph_safe = True

    def __init__(self, vocab: int, layers: int, dim: int, tensor: str = "side.embed"):
        self.vocab, self.layers, self.dim, self.tensor = vocab, layers, dim, tensor
        self.table: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str = "") -> List[ParamSpec]:
        return [ParamSpec(self.tensor, (self.vocab, self.layers * self.dim), MATRIX)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str = "") -> None:
        self.table = state[self.tensor]

    def param_bytes(self) -> int:
        return self.table.numel() * self.table.element_size()


class TokenSide(Part):
    graph_safe = True  # kernels only

    NAMES = {"gate": "gate", "proj": "proj", "norm": "norm"}

    def __init__(self, width: int, table: TokenSideTable, layer: int, eps: float, names: Optional[Dict[str, str]] = None):
        if not (0 <= layer < table.layers):
            raise ValueError(f"layer {layer} of a table for {table.layers} layers")
        self.width, self.dim, self.table, self.layer, self.eps = width, table.dim, table, layer, float(eps)
        self.names = dict(self.NAMES, **(names or {}))
        self.w_gate = self.w_proj = self.norm_weight = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        n = self.names
        return [ParamSpec(f"{prefix}.{n['gate']}", (self.dim, self.width), MATRIX),
                ParamSpec(f"{prefix}.{n['proj']}", (self.width, self.dim), MATRIX),
                ParamSpec(f"{prefix}.{n['norm']}", (self.width,), KEEP32, init="ones")]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        n = self.names
        self.w_gate, self.w_proj = state[f"{prefix}.{n['gate']}"], state[f"{prefix}.{n['proj']}"]
        self.norm_weight = state[f"{prefix}.{n['norm']}"]

    def param_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate, self.w_proj, self.norm_weight))

    def forward(self, ctx: StepContext, x_act: torch.Tensor) -> torch.Tensor:
        """``x_act``: the stream's rows in the activation type.  Returns y (float32 [n, width]) before its norm."""
        ops, ws, n = ctx.ops, ctx.workspace, ctx.n
        t = ws.rows("side_gate", n, self.dim, torch.float32)
        ops.linear(x_act, self.w_gate, t)
        g = ws.rows("side_gated", n, self.dim, ctx.act_dtype)
        ops.token_gate(t, self.table.table, self.layer * self.dim, ctx.tokens, g)
        y = ws.rows("side_out", n, self.width, torch.float32)
        ops.linear(g, self.w_proj, y)
        return y
