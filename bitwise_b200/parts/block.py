"""The arrangements of a layer: the pre-norm residual block, and the parallel block whose mixer
and feed-forward read the same input.

``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (src/model.cpp:281-305).  The
block owns nothing but its four parts and the sub-names under which their tensors are
found; which mixer and which feed-forward it holds is decided where the model is assembled,
layer by layer.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import KEEP32, ParamSpec
from .base import FeedForward, Mixer, Norm, Part, SlotStateNeed, StepContext


class PreNormBlock(Part):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, width: int, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm,
                 names: Dict[str, str]):
        self.width = width
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.names = names  # keys: mixer_norm, mixer, ffn_norm, feed_forward

    def _children(self, prefix: str):
        return [(self.mixer_norm, f"{prefix}.{self.names['mixer_norm']}"),
                (self.mixer, f"{prefix}.{self.names['mixer']}"),
                (self.ffn_norm, f"{prefix}.{self.names['ffn_norm']}"),
                (self.feed_forward, f"{prefix}.{self.names['feed_forward']}")]

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [s for part, p in self._children(prefix) for s in part.param_specs(p)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        for part, p in self._children(prefix):
            part.load_params(state, p)

    def param_bytes(self) -> int:
        return sum(part.param_bytes() for part, _ in self._children(""))

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def prepare(self, ops) -> None:
        for part, _ in self._children(""):
            part.prepare(ops)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        """Run the block on the float32 stream ``x`` in place."""
        xn = ctx.workspace.rows("normed", ctx.n, self.width, ctx.act_dtype)
        self.mixer_norm.forward(ctx, x, xn)
        self.mixer.forward(ctx, xn, x, cache)
        self.ffn_norm.forward(ctx, x, xn)
        self.feed_forward.forward(ctx, xn, x)


class ParallelBlock(PreNormBlock):
    """``x += mixer(norm1(x)) + feed_forward(norm2(x))``: both parts see the same x, their
    outputs are added to each other first and to the stream last.  The mixer writes into a
    float32 buffer, the feed-forward adds to it, and the sum goes into the stream; a feed-forward
    that has ``forward_sum`` does the last two in its own last kernel.  ``feed_forward`` None: the
    layer is its mixer alone."""

    def _children(self, prefix: str):
        kids = super()._children(prefix)
        return [(p, n) for p, n in kids if p is not None]

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        xn = ctx.workspace.rows("normed", ctx.n, self.width, ctx.act_dtype)
        if self.feed_forward is None:
            self.mixer_norm.forward(ctx, x, xn)
            self.mixer.forward(ctx, xn, x, cache)
            return
        xn2 = ctx.workspace.rows("normed_b", ctx.n, self.width, ctx.act_dtype)
        pair = getattr(self.mixer_norm, "forward_pair", None)
        if pair is not None and type(self.ffn_norm) is type(self.mixer_norm):
            pair(ctx, x, xn, self.ffn_norm, xn2)
        else:
            self.mixer_norm.forward(ctx, x, xn)
            self.ffn_norm.forward(ctx, x, xn2)
        delta = ctx.workspace.rows("block_sum", ctx.n, self.width, torch.float32)
        self.mixer.forward(ctx, xn, delta, cache, accumulate=False)
        fused = getattr(self.feed_forward, "forward_sum", None)
        if fused is not None:
            fused(ctx, xn2, delta, x)
        else:
            self.feed_forward.forward(ctx, xn2, delta)
            ctx.ops.add_rows(x, delta)


class SandwichBlock(PreNormBlock):
    """A norm before and after each sublayer: ``x += norm1b(mixer(norm1(x)))``, then ``x +=
    norm2b(feed_forward(norm2(x)))``.  A sublayer writes its output into a float32 buffer; the
    norm after it reads that buffer and adds the normed rows to the stream in one kernel
    (``Norm.forward_residual``).  ``feed_forward`` None: the layer is its mixer alone, with the
    two norms around it.  ``names`` has the keys of :class:`PreNormBlock` plus ``mixer_post`` and
    ``ffn_post``."""

    def __init__(self, width: int, mixer: Mixer, feed_forward, mixer_norm: Norm, mixer_post: Norm, ffn_norm,
                 ffn_post, names: Dict[str, str]):
        super().__init__(width, mixer, feed_forward, mixer_norm, ffn_norm, names)
        self.mixer_post, self.ffn_post = mixer_post, ffn_post

    def _children(self, prefix: str):
        kids = super()._children(prefix) + [(self.mixer_post, f"{prefix}.{self.names['mixer_post']}"),
                                            (self.ffn_post, f"{prefix}.{self.names['ffn_post']}")]
        return [(p, n) for p, n in kids if p is not None]

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        xn = ctx.workspace.rows("normed", ctx.n, self.width, ctx.act_dtype)
        out = ctx.workspace.rows("sublayer_out", ctx.n, self.width, torch.float32)
        self.mixer_norm.forward(ctx, x, xn)
        self.mixer.forward(ctx, xn, out, cache, accumulate=False)
        if self.feed_forward is None:
            self.mixer_post.forward_residual(ctx, out, x)
            return
        fused = getattr(self.mixer_post, "forward_residual_then", None)
        if fused is not None:  # the norm after the mixer and the one before the feed-forward in one kernel
            fused(ctx, out, x, self.ffn_norm, xn)
        else:
            self.mixer_post.forward_residual(ctx, out, x)
            self.ffn_norm.forward(ctx, x, xn)
        self.feed_forward.forward(ctx, xn, out, accumulate=False)
        self.ffn_post.forward_residual(ctx, out, x)


class DepthMix:
    """What a block hands on is a weighted sum of the embedding's output and of every block's result so
    far: with X_0 the embedding's output and X_(j+1) the result of block j, block i hands on ``sum_j a[j]
    X_j`` for j = 0 .. i + 1, ``a`` its tensor of i + 2 numbers.  The results of a step's rows are kept in
    the step's workspace, ``layers + 1`` entries per row."""

    def __init__(self, index: int, layers: int, name: str = "dwa"):
        if not (0 <= index < layers):
            raise ValueError(f"block {index} of {layers}")
        self.index, self.layers, self.name = index, layers, name
        self.weights: Optional[torch.Tensor] = None


class ScaledResidualBlock(PreNormBlock):
    """A pre-norm block whose sublayers' outputs are scaled on their way into the stream, with three
    optional additions, each switched by a constructor argument:

    * ``x += mult * scale_1 * mixer(read_1(x))``, then ``x += mult * scale_2 * feed_forward(read_2(x))``:
      ``scale_k`` a stored vector per sublayer (``layer_scale`` False: ones), ``mult`` a constant;
    * ``taps`` > 0: a sublayer reads ``h + conv(h)`` instead of ``h = norm(x)``, with ``conv(h)_t = sum_j
      c[:, j] h_(t - taps + 1 + j)`` over time on every channel (zeros before the sequence's start).  The
      last ``taps - 1`` normed rows of a request, for both sublayers, are its state (a state slot);
    * ``side``: a :class:`TokenSide`, added after the feed-forward as ``x += mult * norm(side(x))``;
    * ``depth``: a :class:`DepthMix`, applied last.

    ``feed_forward`` None: the layer is its mixer alone.  ``names`` has the keys of
    :class:`PreNormBlock` plus ``scale_1``, ``scale_2``, ``conv_1``, ``conv_2``, ``side``."""
    graph_safe = True  # kernels only; the launches depend on the step's sizes alone

    def __init__(self, width: int, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Norm,
                 ffn_norm: Optional[Norm], names: Dict[str, str], mult: float = 1.0, layer_scale: bool = True,
                 taps: int = 0, side=None, depth: Optional[DepthMix] = None):
        super().__init__(width, mixer, feed_forward, mixer_norm, ffn_norm, names)
        self.mult, self.layer_scale, self.taps = float(mult), bool(layer_scale), int(taps or 0)
        self.side, self.depth = side, depth
        self.sublayers = 2 if feed_forward is not None else 1
        if self.taps > 1 and mixer.state_need() is not None:
            raise NotImplementedError("a block with a convolution's state around a mixer that keeps state of its own")
        self.scale = [None, None]     # mult * scale_k, float32 [width]
        self.conv_t = [None, None]    # the taps of each sublayer's convolution, transposed: [taps, width]

    def _children(self, prefix: str):
        kids = super()._children(prefix)
        if self.side is not None:
            kids.append((self.side, f"{prefix}.{self.names['side']}"))
        return [(p, n) for p, n in kids if p is not None]

    def state_need(self):
        if self.taps > 1:
            return SlotStateNeed((self.taps - 1, self.sublayers * self.width), torch.float32)
        return self.mixer.state_need()

    def query_tile_rows(self, ops=None):
        from .scored_attention import SEQUENCE_TILE
        return [SEQUENCE_TILE] if self.taps > 1 else []

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        specs = super().param_specs(prefix)
        for k in range(self.sublayers):
            if self.layer_scale:
                specs.append(ParamSpec(f"{prefix}.{self.names[f'scale_{k + 1}']}", (self.width,), KEEP32, init="ones"))
            if self.taps:
                specs.append(ParamSpec(f"{prefix}.{self.names[f'conv_{k + 1}']}", (self.width, self.taps), KEEP32))
        if self.depth is not None:
            specs.append(ParamSpec(f"{prefix}.{self.depth.name}", (self.depth.index + 2,), KEEP32))
        return specs

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        super().load_params(state, prefix)
        for k in range(self.sublayers):
            if self.layer_scale:
                self.scale[k] = (state[f"{prefix}.{self.names[f'scale_{k + 1}']}"] * self.mult).contiguous()
            else:
                like = self.mixer_norm.weight
                self.scale[k] = torch.full((self.width,), self.mult, dtype=torch.float32, device=like.device)
            if self.taps:
                self.conv_t[k] = state[f"{prefix}.{self.names[f'conv_{k + 1}']}"].t().contiguous()
        if self.depth is not None:
            self.depth.weights = state[f"{prefix}.{self.depth.name}"]

    def param_bytes(self) -> int:
        own = [t for t in self.scale + self.conv_t + [self.depth.weights if self.depth is not None else None] if t is not None]
        return super().param_bytes() + sum(t.numel() * t.element_size() for t in own)

    def _read(self, ctx: StepContext, x, norm: Norm, k: int, xn, normed, state) -> None:
        """What sublayer k reads: the normed rows, with the convolution over time where the block has one."""
        if not self.taps:
            norm.forward(ctx, x, xn)
            return
        ctx.ops.norm_conv(x, norm.weight, norm.eps, self.conv_t[k], state.state if state is not None else None,
                          k * self.width, ctx, xn, normed, k * self.width)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        from .scored_attention import SEQUENCE_TILE
        ops, ws, n, width = ctx.ops, ctx.workspace, ctx.n, self.width
        state = getattr(cache, "state", None) if self.taps > 1 else None
        history = None
        if self.depth is not None:
            history = ws.rows("depth_history", n, (self.depth.layers + 1) * width, torch.float32)
            if self.depth.index == 0:
                ops.copy_history(x, history)
        xn = ws.rows("normed", n, width, ctx.act_dtype)
        normed = ws.rows("conv_normed", n, self.sublayers * width, torch.float32) if self.taps else None
        out = ws.rows("sublayer_out", n, width, torch.float32)
        # the stream in the activation type, for the token input's first product
        rounded = ws.rows("stream_rounded", n, width, ctx.act_dtype) if self.side is not None and ctx.act_dtype != torch.float32 else None
        self._read(ctx, x, self.mixer_norm, 0, xn, normed, state)
        self.mixer.forward(ctx, xn, out, cache, accumulate=False)
        ops.scaled_add(x, self.scale[0], out, rounded if self.feed_forward is None else None)
        if self.feed_forward is not None:
            self._read(ctx, x, self.ffn_norm, 1, xn, normed, state)
            scaled = getattr(self.feed_forward, "forward_scaled", None)
            if scaled is not None:
                scaled(ctx, xn, x, self.scale[1])
                if rounded is not None:
                    ops.scaled_add(x, None, None, rounded)
            else:
                self.feed_forward.forward(ctx, xn, out, accumulate=False)
                ops.scaled_add(x, self.scale[1], out, rounded)
        if state is not None:
            ops.conv_state_update(normed, state.state, ctx, self.taps, ctx.query_tiles(SEQUENCE_TILE))
        if self.side is None and self.depth is None:
            return
        y = self.side.forward(ctx, rounded if rounded is not None else x) if self.side is not None else None
        ops.normed_add_mix(x, y, self.side.norm_weight if self.side is not None else None,
                           self.side.eps if self.side is not None else 0.0, self.mult, history,
                           self.depth.index + 1 if self.depth is not None else 0,
                           self.depth.weights if self.depth is not None else None)
