"""Latent attention: keys and values of all heads come from one small vector per position.

A position keeps a latent ``c`` of ``rank`` numbers (the down projection of the mixer's input,
divided by its root mean square, times a weight) and ``rot_dim`` numbers of a rotated key part
that every head shares.  Head h's key is ``[W_uk[h] c | k_rot]``, its value ``W_uv[h] c``, its
query ``[q_h (dim numbers) | rotated q_h (rot_dim numbers)]``; scores are scaled dot products,
causal, with an ordinary softmax.  Queries come straight from the input (``q_rank`` None) or
through a latent of their own (down projection, root-mean-square norm, up projection).

The cache is never expanded into per-head keys: the key map is folded into the query
(``q'_h = W_uk[h]^T q_h``, one small product per head), a score is then one dot product of
``rank + rot_dim`` terms against the cached vector, attention returns the weighted sum of
latents per head, and the value map is applied to that sum.  The same arithmetic serves prompt
portions and single rows, so a position's result does not depend on how the prompt was cut.

Rotation: entries 2i and 2i + 1 of the rotated part form pair i, turned by ``pos * base ** (-2i
/ dims)``; ``rot_pairs`` pairs are turned and the rest of the part passes unchanged.  A position
encoding whose ``layout`` is "half" pairs entry i with entry i + dims / 2 instead.  A layer
may read the cache of an earlier layer instead of writing one (``shares_cache``): it then has
no down projection for keys and values.

Options: ``sink`` (a learned logit per head, tensor ``sink``, whose exponential joins the softmax's
denominator: it has no key and no value and is not scaled) and ``gate`` ("entry" or "head": the
heads' values are multiplied by the sigmoid of a projection of the mixer's input, per entry or
per head, before the output projection; :class:`OutputGate`).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import KEEP32, MATRIX, ParamSpec
from .base import Mixer, PagedLatentNeed, PagedLatentView, PositionEncoding, StepContext, register_mixer
from .gate import OutputGate


class LatentAttention(Mixer):
    graph_safe = True  # kernels only; launches depend on the step's sizes and ctx.max_keys

    NAMES = {"q": "q", "q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm",
             "k_up": "uk", "v_up": "uv", "out": "o", "sink": "sink", "gate": "g"}

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, rank: int, scale: float, eps: float,
                 position: Optional[PositionEncoding] = None, q_rank: Optional[int] = None,
                 shares_cache: bool = False, window: Optional[int] = None, names: Optional[Dict[str, str]] = None,
                 sink: bool = False, gate: Optional[str] = None, stack_inputs: bool = False):
        for what, v in (("heads", heads), ("dim", dim), ("vdim", vdim), ("rank", rank)):
            if v <= 0:
                raise ValueError(f"latent attention: {what} must be positive, got {v}")
        if rot_dim < 0 or (q_rank is not None and q_rank <= 0):
            raise ValueError("latent attention: negative rotated size or latent query size")
        self.width, self.heads, self.dim, self.rot_dim, self.vdim, self.rank = width, heads, dim, rot_dim, vdim, rank
        self.scale, self.eps = float(scale), float(eps)
        self.position, self.q_rank, self.shares_cache, self.window = position, q_rank, shares_cache, window
        self.names = dict(self.NAMES, **(names or {}))
        self.q_width = heads * (dim + rot_dim)
        self.w_q = self.w_q_down = self.q_norm = self.w_kv_down = self.kv_norm = None
        self.w_k_fold = self.w_v_up = self.w_o = None
        self.sink, self.sinks = bool(sink), None
        self.gate = OutputGate(width, heads, vdim, gate, self.names["gate"]) if gate else None
        self.half_layout = getattr(position, "layout", "pairs") == "half"
        # one product for everything that reads the mixer's input (both down projections and the gate), its rows
        # laid out [keys' and values' latent | rotated key part | queries' latent | gate]
        self.stacked = bool(stack_inputs) and q_rank is not None and not shares_cache
        self.w_in = None

    @property
    def _layout(self):
        # (only the half layout is named to the kernels, so that earlier designs' calls stay as they were)
        return {"half_layout": True} if self.half_layout else {}

    def cache_need(self):
        return PagedLatentNeed(self.rank, self.rot_dim, self.window)

    def query_tile_rows(self, ops=None):
        if ops is not None and hasattr(ops, "latent_attention_tile_heights"):
            return list(ops.latent_attention_tile_heights(self.heads, self.rank, self.rot_dim))
        return [max(1, 32 // self.heads)]

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        n = self.names
        specs = []
        if self.q_rank is None:
            specs.append(ParamSpec(f"{prefix}.{n['q']}", (self.q_width, self.width), MATRIX))
        else:
            specs += [ParamSpec(f"{prefix}.{n['q_down']}", (self.q_rank, self.width), MATRIX),
                      ParamSpec(f"{prefix}.{n['q_norm']}", (self.q_rank,), KEEP32, init="ones"),
                      ParamSpec(f"{prefix}.{n['q_up']}", (self.q_width, self.q_rank), MATRIX)]
        if not self.shares_cache:
            specs += [ParamSpec(f"{prefix}.{n['kv_down']}", (self.rank + self.rot_dim, self.width), MATRIX),
                      ParamSpec(f"{prefix}.{n['kv_norm']}", (self.rank,), KEEP32, init="ones")]
        specs += [ParamSpec(f"{prefix}.{n['k_up']}", (self.heads * self.dim, self.rank), MATRIX),
                  ParamSpec(f"{prefix}.{n['v_up']}", (self.heads * self.vdim, self.rank), MATRIX),
                  ParamSpec(f"{prefix}.{n['out']}", (self.width, self.heads * self.vdim), MATRIX)]
        if self.sink:
            specs.append(ParamSpec(f"{prefix}.{n['sink']}", (self.heads,), KEEP32))
        if self.gate is not None:
            specs += self.gate.param_specs(prefix)
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        n = self.names
        if self.q_rank is None:
            self.w_q = state[f"{prefix}.{n['q']}"]
        else:
            self.w_q_down = state[f"{prefix}.{n['q_down']}"]
            self.q_norm = state[f"{prefix}.{n['q_norm']}"]
            self.w_q = state[f"{prefix}.{n['q_up']}"]
        if not self.shares_cache:
            self.w_kv_down = state[f"{prefix}.{n['kv_down']}"]
            self.kv_norm = state[f"{prefix}.{n['kv_norm']}"]
        # the key map per head, transposed: folding it into a query is the product q_h W_uk[h]
        w_uk = state[f"{prefix}.{n['k_up']}"]
        self.w_k_fold = w_uk.reshape(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_v_up = state[f"{prefix}.{n['v_up']}"].reshape(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = state[f"{prefix}.{n['out']}"]
        if self.sink:
            self.sinks = state[f"{prefix}.{n['sink']}"]
        if self.gate is not None:
            self.gate.load_params(state, prefix)
        if self.stacked:
            parts = [self.w_kv_down, self.w_q_down] + ([self.gate.weight] if self.gate is not None else [])
            self.w_in = torch.cat(parts, 0).contiguous()
            # the separate matrices become views of the stacked one (a run that only reads a cache uses them)
            dk = self.rank + self.rot_dim
            self.w_kv_down, self.w_q_down = self.w_in[:dk], self.w_in[dk:dk + self.q_rank]
            if self.gate is not None:
                self.gate.weight = self.w_in[dk + self.q_rank:]

    def param_bytes(self) -> int:
        ts = (self.w_q, self.w_q_down, self.q_norm, self.w_kv_down, self.kv_norm, self.w_k_fold, self.w_v_up, self.w_o,
              self.sinks)
        return sum(t.numel() * t.element_size() for t in ts if t is not None) + (
            self.gate.param_bytes() if self.gate is not None else 0)

    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor, cache: PagedLatentView,
                accumulate: bool = True) -> None:
        """``accumulate`` False: the output is written to ``x`` instead of added to it."""
        ops, ws, n = ctx.ops, ctx.workspace, ctx.n
        act = ctx.act_dtype
        dk = self.rank + self.rot_dim
        tables = self.position.rotary_tables(x.device) if self.position is not None and self.rot_dim else None
        cos, sin = tables if tables is not None else (None, None)
        # queries
        gate_logits = None
        stacked = self.stacked and cache.writable
        if stacked:
            u = ws.rows("latent_in32", n, self.w_in.shape[0], torch.float32)
            ops.linear(xn, self.w_in, u)
            q_in = ws.rows("latent_q", n, self.q_rank, act)
            ops.latent_store(u, self.kv_norm, self.eps, ctx.pos, ctx.row_seq, cos, sin, cache.block_table, cache.latent,
                             self.rank, self.rot_dim, q_latent=(self.q_norm, q_in), **self._layout)
            if self.gate is not None:
                gate_logits = u[:, dk + self.q_rank:]
        elif self.q_rank is None:
            q_in = xn
        else:
            cq = ws.rows("latent_q32", n, self.q_rank, torch.float32)
            ops.linear(xn, self.w_q_down, cq)
            q_in = ws.rows("latent_q", n, self.q_rank, act)
            ops.rmsnorm(cq, self.q_norm, self.eps, q_in)
        q = ws.rows("latent_heads_q", n, self.q_width, act)
        ops.linear(q_in, self.w_q, q)
        # this layer's entry of the cache
        if cache.writable and not self.shares_cache and not stacked:
            d = ws.rows("latent_kv32", n, dk, torch.float32)
            ops.linear(xn, self.w_kv_down, d)
            ops.latent_store(d, self.kv_norm, self.eps, ctx.pos, ctx.row_seq, cos, sin, cache.block_table, cache.latent,
                             self.rank, self.rot_dim, **self._layout)
        # the key maps folded into the queries, the rotated parts beside them
        qf = ws.rows("latent_folded_q", n, self.heads * dk, act)
        ops.grouped_linear(q, self.w_k_fold, qf, n, x_group_cols=self.dim + self.rot_dim, o_group_cols=dk)
        if self.rot_dim:
            ops.rotate_heads(q, self.heads, self.dim + self.rot_dim, self.dim, self.rot_dim, qf, dk, self.rank, ctx.pos,
                             cos, sin, **self._layout)
        mixed = ws.rows("latent_mixed", n, self.heads * self.rank, act)
        ops.latent_attention(qf, cache.latent, cache.block_table, mixed, self.heads, self.rank, self.rot_dim, self.scale,
                             ctx, self.window or 0, **({"sinks": self.sinks} if self.sink else {}))
        values = ws.rows("latent_values", n, self.heads * self.vdim, act)
        ops.grouped_linear(mixed, self.w_v_up, values, n, x_group_cols=self.rank, o_group_cols=self.vdim)
        if self.gate is not None:
            self.gate.apply(ctx, xn, values, gate_logits)
        ops.linear(values, self.w_o, x, residual=x if accumulate else None)


register_mixer("latent_attention", LatentAttention)
