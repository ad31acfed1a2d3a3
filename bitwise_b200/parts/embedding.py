"""Token embedding and output head.

Embedding: a row copy, widened to the 32-bit stream (src/model.cpp:233-239,274); no
scaling of embeddings.  Head: gather the rows whose logits are wanted, final norm on those
rows only, one product with lm_head, or with the embedding table when the model ties them
(src/model.cpp:170-171,308-321); logits are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import MATRIX, ParamSpec
from .base import Norm, Part, SlotStateNeed, StepContext


class TokenEmbedding(Part):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, vocab: int, width: int, name: str = "embed_tokens", tensor: Optional[str] = None,
                 norm: Optional[Norm] = None, norm_tensor: Optional[str] = None, scale: float = 1.0,
                 pair_table: Optional[str] = None, pair_buckets: int = 0, pair_mul_prev: int = 0, pair_mul_cur: int = 0):
        """``tensor``: the table's full name where it is not ``<prefix>.<name>.weight``.  ``norm``:
        a norm applied to the embedded rows in place on the stream, its weight named ``norm_tensor``.
        ``scale``: a constant that the embedded rows are multiplied by (in 32-bit).  ``pair_table``:
        the name of a second table ``[pair_buckets + 1, width]`` whose row ``(previous token *
        pair_mul_prev + token * pair_mul_cur) mod pair_buckets`` is added (unscaled), the last row
        for a sequence's first token; the previous token is kept per request in a state slot."""
        self.vocab, self.width, self.name = vocab, width, name
        self.scale = float(scale)
        self.tensor, self.norm, self.norm_tensor = tensor, norm, norm_tensor
        self.table: Optional[torch.Tensor] = None
        self.pair_name = pair_table
        self.pair_buckets, self.pair_mul_prev, self.pair_mul_cur = int(pair_buckets), int(pair_mul_prev), int(pair_mul_cur)
        if pair_table is not None and self.pair_buckets <= 0:
            raise ValueError("a second table needs a positive number of buckets")
        self.pair: Optional[torch.Tensor] = None

    def state_need(self):
        """With a second table: the request's last token, one int32 per slot."""
        return SlotStateNeed((1,), torch.int32) if self.pair_name is not None else None

    def query_tile_rows(self, ops=None):
        from .scored_attention import SEQUENCE_TILE
        return [SEQUENCE_TILE] if self.pair_name is not None else []

    def tensor_name(self, prefix: str) -> str:
        return self.tensor if self.tensor is not None else f"{prefix}.{self.name}.weight"

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        specs = [ParamSpec(self.tensor_name(prefix), (self.vocab, self.width), MATRIX)]
        if self.pair_name is not None:
            specs.append(ParamSpec(self.pair_name, (self.pair_buckets + 1, self.width), MATRIX))
        if self.norm is not None:
            specs += self.norm.param_specs(self.norm_tensor)
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        self.table = state[self.tensor_name(prefix)]
        if self.pair_name is not None:
            self.pair = state[self.pair_name]
        if self.norm is not None:
            self.norm.load_params(state, self.norm_tensor)

    def param_bytes(self) -> int:
        pair = self.pair.numel() * self.pair.element_size() if self.pair is not None else 0
        return self.table.numel() * self.table.element_size() + pair + (self.norm.param_bytes() if self.norm else 0)

    def forward(self, ctx: StepContext, x: torch.Tensor, state=None) -> None:
        """``state``: the ``SlotStateView`` of ``state_need`` (the requests' last tokens)."""
        if self.pair is not None:
            from .scored_attention import SEQUENCE_TILE
            ctx.ops.embed_pair(self.table, self.pair, ctx, state.state, x, self.scale, self.pair_buckets,
                               self.pair_mul_prev, self.pair_mul_cur)
            ctx.ops.last_token_update(ctx, state.state, ctx.query_tiles(SEQUENCE_TILE))
        elif self.scale != 1.0:
            ctx.ops.embed_rows(self.table, ctx.tokens, x, scale=self.scale)
        else:
            ctx.ops.embed_rows(self.table, ctx.tokens, x)
        if self.norm is not None:
            self.norm.forward(ctx, x, x)


class OutputHead(Part):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, vocab: int, width: int, norm: Norm, tied_to: Optional[TokenEmbedding] = None,
                 norm_name: str = "model.norm", head_name: str = "lm_head", suffix: str = ".weight",
                 softcap: Optional[float] = None):
        """A constant scale of the logits belongs to ``norm`` as its ``gain`` (the product is linear).
        ``softcap``: the logits become ``softcap * tanh(logits / softcap)``."""
        if softcap is not None and not softcap > 0:
            raise ValueError(f"the logits' cap must be positive, got {softcap!r}")
        self.softcap = float(softcap) if softcap is not None else None
        self.vocab, self.width = vocab, width
        self.suffix = suffix
        self.norm, self.tied_to = norm, tied_to
        self.norm_name, self.head_name = norm_name, head_name
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self, prefix: str = "") -> List[ParamSpec]:
        specs = self.norm.param_specs(self.norm_name)
        if self.tied_to is None:
            specs.append(ParamSpec(f"{self.head_name}{self.suffix}", (self.vocab, self.width), MATRIX))
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str = "") -> None:
        self.norm.load_params(state, self.norm_name)
        self.weight = self.tied_to.table if self.tied_to is not None else state[f"{self.head_name}{self.suffix}"]

    def param_bytes(self) -> int:
        own = 0 if self.tied_to is not None else self.weight.numel() * self.weight.element_size()
        return own + self.norm.param_bytes()

    def forward(self, ctx: StepContext, x: torch.Tensor) -> Optional[torch.Tensor]:
        c = ctx.num_logit_rows
        if c == 0:
            return None
        last = ctx.workspace.rows("head_in", c, self.width, ctx.act_dtype)
        self.norm.forward(ctx, x, last, rows=ctx.logit_rows)
        logits = ctx.workspace.rows("logits", c, self.vocab, torch.float32, growable=True)
        ctx.ops.linear(last, self.weight, logits)
        if self.softcap is not None:
            ctx.ops.softcap_rows(logits, self.softcap)
        return logits
