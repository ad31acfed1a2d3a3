"""The output gate of a mixer: what the heads produced is multiplied, entry by entry, with the
sigmoid of a projection of the mixer's own input, before the output projection.

``mode`` "entry": one gate number per entry of the concatenated heads (the tensor is ``[heads *
vdim, width]``); "head": one per head (``[heads, width]``), shared by the head's entries.  The
projection runs in the activation type with a 32-bit result; the sigmoid and the product are
32-bit.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import MATRIX, ParamSpec
from .base import StepContext

GATE_MODES = ("entry", "head")


class OutputGate:
    def __init__(self, width: int, heads: int, vdim: int, mode: str, name: str = "g"):
        if mode not in GATE_MODES:
            raise ValueError(f"an output gate is per 'entry' or per 'head', not {mode!r}")
        self.width, self.heads, self.vdim, self.mode, self.name = width, heads, vdim, mode, name
        self.cols = heads * vdim if mode == "entry" else heads
        self.group = 1 if mode == "entry" else vdim
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [ParamSpec(f"{prefix}.{self.name}", (self.cols, self.width), MATRIX)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        self.weight = state[f"{prefix}.{self.name}"]

    def param_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def apply(self, ctx: StepContext, xn: torch.Tensor, heads_out: torch.Tensor, logits: Optional[torch.Tensor] = None) -> None:
        """``heads_out`` [n, heads * vdim] is gated in place.  ``logits``: the gate's projection of ``xn`` where
        the caller formed it already (as columns of a wider product)."""
        if logits is None:
            logits = ctx.workspace.rows("gate_logits", ctx.n, self.cols, torch.float32)
            ctx.ops.linear(xn, self.weight, logits)
        ctx.ops.sigmoid_gate(heads_out, logits, self.group)
