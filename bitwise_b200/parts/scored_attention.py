"""Grouped-query softmax attention over paged keys and values, with its steps as options.

Before the scores, each on or off by a constructor argument:

* biases of the q, k and v projections (``bias``; tensors ``<name>.b``), added in 32-bit;
* ``value_mix``: the layer's values become ``(1 - lambda) v + lambda v_first`` with ``v_first`` the values
  that the model's first such layer (``"source"``) formed for the same token and ``lambda`` the
  layer's scalar tensor (``"mix"``); the mixed values are what is cached;
* a short causal convolution over time on every channel of q, k and v, directly after the
  projection: ``y_t = sum_j w[:, j] * u_(t - taps + 1 + j)``, zeros before the sequence's start.
  The last ``taps - 1`` projected rows of a request are its state, kept in a state slot;
* a root-mean-square norm of every head of q and of k, with one weight of the head's size each
  (``qk_norm="unit"``: without weights, the head is only divided by its root mean square);
* a rotation of the first ``rot_dims`` entries of every head of q and k: entries 2i and 2i + 1
  form pair i, turned by ``pos * base ** (-2i / rot_dims)`` (tables from a ``RotaryEncoding``).

On the scores ``s = (q . k) * scale``:

* ``softcap``: ``s <- cap * tanh(s / cap)``;
* ``slopes``: ``s <- s - slope_h * (i - j)`` for query position i and key position j;
* ``distance_log``: ``s <- s - a_h * ln(1 + b_h * (i - j))`` with two learned numbers per head;
* ``window``: position i sees the keys j with ``0 <= i - j < window`` (every j <= i without), and
  with ``keep_first`` also the keys ``j < keep_first``, at their true distance;
* ``sink``: one is added to the softmax's denominator (a key of score 0 that has no value);
  ``sink="learned"``: ``exp(sink_h)`` with a learned number per head instead.

``gate`` ("entry" or "head"): the heads' outputs are multiplied by the sigmoid of a projection of the
mixer's input, per entry or per head, before the output projection (:class:`OutputGate`).

``values_are_keys``: there is no value projection and nothing but the keys is cached; the
weighted sum runs over the keys as projected.  ``shares_cache``: the layer has no key and value
tensors; it reads the pages that an earlier layer wrote (keys after convolution, norm and
rotation; values after convolution), with its own queries and its own convolution state.

Projections may run in the activation type; what follows them up to the stored key (convolution,
norm, rotation), the scores and the softmax weights are 32-bit in both precisions.  Head h reads
key/value head ``h // (heads / kv_heads)``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..weights.loader import KEEP32, MATRIX, ParamSpec
from .base import Mixer, PagedKVNeed, PagedKVView, PositionEncoding, SlotStateNeed, StepContext, register_mixer
from .gate import OutputGate


def distance_slopes(heads: int, exponent: float = 8.0) -> List[float]:
    """slope_h = 2 ** (-exponent * (h + 1) / heads) for h = 0 .. heads - 1."""
    return [2.0 ** (-exponent * (h + 1) / heads) for h in range(heads)]


class ScoredAttention(Mixer):
    graph_safe = True  # kernels only; launches depend on the step's sizes and ctx.max_keys

    NAMES = {"q": "q", "k": "k", "v": "v", "out": "o", "conv": ".conv", "norm": ".norm", "bias": ".b", "vmix": "vmix",
             "dist_a": "r1", "dist_b": "r2", "sink": "sink", "gate": "g"}

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float = 1e-6,
                 conv_taps: int = 0, qk_norm: bool = False, position: Optional[PositionEncoding] = None, rot_dims: int = 0,
                 softcap: Optional[float] = None, sink: bool = False, slopes: Optional[Sequence[float]] = None,
                 window: Optional[int] = None, values_are_keys: bool = False, shares_cache: bool = False,
                 names: Optional[Dict[str, str]] = None, bias: bool = False, distance_log: bool = False,
                 keep_first: int = 0, value_mix: Optional[str] = None, gate: Optional[str] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} key/value heads")
        if values_are_keys and vdim != dim:
            raise ValueError("values that are the keys have the keys' size")
        if slopes is not None and len(slopes) != heads:
            raise ValueError("one slope per head is needed")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"{rot_dims} turned entries do not fit a head of {dim}")
        if value_mix not in (None, "source", "mix"):
            raise ValueError(f"value_mix is None, 'source' or 'mix', not {value_mix!r}")
        if value_mix and (values_are_keys or shares_cache):
            raise ValueError("values can only be mixed where the layer forms values of its own")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.scale, self.eps = float(scale), float(eps)
        self.taps = int(conv_taps or 0)  # 0: no convolution; 1: a factor per channel and no state
        self.qk_norm, self.position, self.rot_dims = bool(qk_norm), position, rot_dims
        self.unit_norm = qk_norm == "unit"  # no weights: a head is divided by its root mean square and no more
        self.softcap, self.sink, self.window = softcap, bool(sink), window
        self.learned_sink = sink == "learned"
        self.bias, self.distance_log, self.value_mix = bool(bias), bool(distance_log), value_mix
        self.keep_first = int(keep_first or 0) if window else 0
        self.slopes_host = [float(s) for s in slopes] if slopes is not None else None
        self.values_are_keys, self.shares_cache = values_are_keys, shares_cache
        self.names = dict(self.NAMES, **(names or {}))
        self.q_cols = heads * dim
        self.k_cols = 0 if shares_cache else kv_heads * dim
        self.v_cols = 0 if shares_cache or values_are_keys else kv_heads * vdim
        self.cols = self.q_cols + self.k_cols + self.v_cols
        self.w_in = self.w_o = self.conv_w = self.conv_wt = self.q_norm = self.k_norm = self.slopes = None
        self.b_in = self.dist_a = self.dist_b = self.sinks = self.vmix = None
        self.gate = OutputGate(width, heads, vdim, gate, self.names["gate"]) if gate else None

    # -- what the cache keeps --------------------------------------------------------------
    def cache_need(self):
        return PagedKVNeed(self.kv_heads, self.dim, self.window, v_dim=0 if self.values_are_keys else self.vdim,
                           keep_first=self.keep_first)

    def state_need(self):
        """The convolution's inputs of the last ``taps - 1`` positions, for every channel it runs on."""
        if self.taps <= 1:
            return None
        return SlotStateNeed((self.taps - 1, self.cols), torch.float32)

    def query_tile_rows(self, ops=None):
        group = self.heads // self.kv_heads
        heights = list(ops.scored_attention_tile_heights(group, self.dim, self.vdim)) if ops is not None and hasattr(
            ops, "scored_attention_tile_heights") else [max(1, 32 // group)]
        if self.taps > 1:
            heights.append(SEQUENCE_TILE)
        return heights

    # -- parameters ------------------------------------------------------------------------
    def _projections(self):
        n = self.names
        out = [(n["q"], self.q_cols, self.dim, True)]
        if not self.shares_cache:
            out.append((n["k"], self.k_cols, self.dim, True))
            if not self.values_are_keys:
                out.append((n["v"], self.v_cols, self.vdim, False))
        return out  # (name, columns, head size, normed)

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        n = self.names
        specs = []
        for name, cols, size, normed in self._projections():
            specs.append(ParamSpec(f"{prefix}.{name}", (cols, self.width), MATRIX))
            if self.bias:
                specs.append(ParamSpec(f"{prefix}.{name}{n['bias']}", (cols,), KEEP32))
            if self.taps:
                specs.append(ParamSpec(f"{prefix}.{name}{n['conv']}", (cols, self.taps), KEEP32))
            if self.qk_norm and normed and not self.unit_norm:
                specs.append(ParamSpec(f"{prefix}.{name}{n['norm']}", (size,), KEEP32, init="ones"))
        if self.value_mix:  # (the first such layer has the tensor too and no use for it)
            specs.append(ParamSpec(f"{prefix}.{n['vmix']}", (), KEEP32, optional=self.value_mix == "source"))
        if self.distance_log:
            specs += [ParamSpec(f"{prefix}.{n['dist_a']}", (self.heads,), KEEP32),
                      ParamSpec(f"{prefix}.{n['dist_b']}", (self.heads,), KEEP32, init="positive")]
        if self.learned_sink:
            specs.append(ParamSpec(f"{prefix}.{n['sink']}", (self.heads,), KEEP32))
        if self.gate is not None:
            specs += self.gate.param_specs(prefix)
        specs.append(ParamSpec(f"{prefix}.{n['out']}", (self.width, self.heads * self.vdim), MATRIX))
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        n = self.names
        proj = self._projections()
        ws = [state[f"{prefix}.{name}"] for name, _, _, _ in proj]
        self.w_in = torch.cat(ws, 0).contiguous() if len(ws) > 1 else ws[0]
        if self.taps:
            self.conv_w = torch.cat([state[f"{prefix}.{name}{n['conv']}"] for name, _, _, _ in proj], 0).contiguous()
            self.conv_wt = self.conv_w.t().contiguous()  # [taps, channels]: four channels of a tap lie together
        if self.unit_norm:
            ones = torch.ones(self.dim, dtype=torch.float32, device=ws[0].device)
            self.q_norm, self.k_norm = ones, None if self.shares_cache else ones
        elif self.qk_norm:
            self.q_norm = state[f"{prefix}.{n['q']}{n['norm']}"]
            self.k_norm = None if self.shares_cache else state[f"{prefix}.{n['k']}{n['norm']}"]
        if self.gate is not None:
            # the gate reads the mixer's input like the projections: its rows ride behind theirs in one product
            self.gate.load_params(state, prefix)
            self.w_in = torch.cat([self.w_in, self.gate.weight], 0).contiguous()
            self.gate.weight = self.w_in[self.cols:]
        self.w_o = state[f"{prefix}.{n['out']}"]
        if self.bias:
            self.b_in = torch.cat([state[f"{prefix}.{name}{n['bias']}"] for name, _, _, _ in proj], 0).contiguous()
        if self.value_mix == "mix":
            self.vmix = state[f"{prefix}.{n['vmix']}"].reshape(1).contiguous()
        if self.distance_log:
            self.dist_a, self.dist_b = state[f"{prefix}.{n['dist_a']}"], state[f"{prefix}.{n['dist_b']}"]
        if self.learned_sink:
            self.sinks = state[f"{prefix}.{n['sink']}"]
        if self.slopes_host is not None:
            self.slopes = torch.tensor(self.slopes_host, dtype=torch.float32, device=self.w_o.device)

    def param_bytes(self) -> int:
        ts = (self.w_in, self.w_o, self.conv_w, None if self.unit_norm else self.q_norm,
              None if self.unit_norm else self.k_norm, self.b_in, self.vmix, self.dist_a, self.dist_b,
              self.sinks)  # (the transposed taps are a copy)
        return sum(t.numel() * t.element_size() for t in ts if t is not None)  # (the gate's rows are part of w_in)

    # -- one step --------------------------------------------------------------------------
    def forward(self, ctx: StepContext, xn: torch.Tensor, x: torch.Tensor, cache: PagedKVView,
                accumulate: bool = True) -> None:
        """``accumulate`` False: the output is written to ``x`` instead of added to it."""
        ops, ws, n = ctx.ops, ctx.workspace, ctx.n
        gate_logits = None
        if self.gate is not None:
            wide = ws.rows("scored_qkv32", n, self.cols + self.gate.cols, torch.float32)
            ops.linear(xn, self.w_in, wide)
            u, gate_logits = wide[:, :self.cols], wide[:, self.cols:]
        else:
            u = ws.rows("scored_qkv32", n, self.cols, torch.float32)
            ops.linear(xn, self.w_in, u)
        tables = self.position.rotary_tables(x.device) if self.position is not None and self.rot_dims else None
        cos, sin = tables if tables is not None else (None, None)
        q = ws.rows("scored_q", n, self.q_cols, ctx.act_dtype)
        state = cache.state if self.taps > 1 else None
        writes = cache.writable and not self.shares_cache
        extra = {}
        if self.bias:
            extra["bias"] = self.b_in
        if self.value_mix and writes:
            # the first mixing layer's values of the step's rows, in 32-bit, for the layers after it
            first = ws.rows("mixed_values_first", n, self.v_cols, torch.float32)
            if self.value_mix == "source":
                extra["v_keep"] = first
            else:
                extra["vmix_src"], extra["vmix_lambda"] = first, self.vmix
        ops.qkv_prepare(u, self.conv_w, state.state if state is not None else None, self.q_norm, self.k_norm, self.eps,
                        cos, sin, ctx, cache.block_table, cache.k, cache.v, q, self.heads,
                        self.kv_heads if writes else 0, self.dim, self.vdim, conv_wt=self.conv_wt, **extra)
        if state is not None:
            ops.conv_state_update(u, state.state, ctx, self.taps, ctx.query_tiles(SEQUENCE_TILE))
        mixed = ws.rows("scored_mixed", n, self.heads * self.vdim, ctx.act_dtype)
        ops.scored_attention(q, cache.k, cache.v, cache.block_table, mixed, self.heads, self.kv_heads, self.dim, self.vdim,
                             self.scale, self.softcap or 0.0, self.sink, self.slopes, self.window or 0, ctx,
                             dist_a=self.dist_a, dist_b=self.dist_b, sinks=self.sinks, keep_first=self.keep_first)
        if self.gate is not None:
            self.gate.apply(ctx, xn, mixed, gate_logits)
        ops.linear(mixed, self.w_o, x, residual=x if accumulate else None)


# A query-tile height larger than any step: the step's tile list of this height has one entry
# per sequence (sequence, first row, rows), which is what kernels that walk a sequence need.
SEQUENCE_TILE = 1 << 20

register_mixer("scored_attention", ScoredAttention)
