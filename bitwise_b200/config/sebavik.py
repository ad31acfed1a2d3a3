"""Typed configuration of the Sebavik design, read from config.json.

Keys: ``architecture`` ("Sebavik"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (the factor
on everything a layer adds to the stream), ``embedding.scale``, optionally ``embedding.bigram``
(``buckets``, ``mul_prev``, ``mul_cur``: a second table indexed by a hash of the previous and the
current token), optionally ``canon.taps`` (a causal convolution over time on what every sublayer
reads), optionally ``token_side.dim`` (a gated per-layer token input), and ``layers``, a list with one
entry per layer: ``type`` ("attention"), ``mixer`` and ``mlp``.

* mixer: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, optionally ``softcap``, ``mask.size``
  (window) with ``mask.keep_first`` (first positions that stay visible), ``v_mix`` (the layer's values
  are mixed with those of the first such layer);
* mlp: null, ``{"kind": "dense", "ff", "limit"}`` or ``{"kind": "moe", "expert": {"ff"}, "router":
  {"experts", "top"}}``.

Every size and constant of a model comes from here or from a tensor's shape.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError

MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense", "moe")


def _get(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def _count(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v < 0:
        raise ConfigError(f"config.json: {what} must be a non-negative integer, got {v!r}")
    return v


@dataclass(frozen=True)
class SebavikMixerConfig:
    heads: int
    kv_heads: int
    dim: int                        # query/key size per head
    vdim: int                       # value size per head
    scale: float
    softcap: Optional[float] = None
    window: Optional[int] = None    # keys a position sees inside its window, itself included
    keep_first: int = 0             # first positions that stay visible beyond the window
    v_mix: bool = False

    @staticmethod
    def from_json(d: dict, where: str) -> "SebavikMixerConfig":
        heads = _positive_int(_get(d, "heads", where), where + ".heads")
        kv_heads = _positive_int(_get(d, "kv_heads", where), where + ".kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}: {heads} heads are no multiple of {kv_heads} key/value heads")
        mask = d.get("mask") or {}
        window = _positive_int(mask["size"], where + ".mask.size") if mask.get("size") is not None else None
        keep = _count(mask.get("keep_first", 0) or 0, where + ".mask.keep_first")
        cap = d.get("softcap")
        if cap is not None:
            cap = float(cap)
            if not cap > 0:
                raise ConfigError(f"config.json: {where}.softcap must be positive, got {cap!r}")
        return SebavikMixerConfig(heads=heads, kv_heads=kv_heads, dim=_positive_int(_get(d, "dim", where), where + ".dim"),
                                  vdim=_positive_int(_get(d, "vdim", where), where + ".vdim"),
                                  scale=float(_get(d, "scale", where)), softcap=cap, window=window,
                                  keep_first=keep if window is not None else 0, v_mix=bool(d.get("v_mix", False)))

    def to_json(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "v_mix": self.v_mix,
             "vdim": self.vdim}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.window is not None:
            d["mask"] = {"keep_first": self.keep_first, "size": self.window}
        return d


@dataclass(frozen=True)
class SebavikMlpConfig:
    kind: str                  # one of MLP_KINDS
    ff: int                    # inner size (of every expert for "moe")
    limit: Optional[float] = None   # dense: the clamp
    experts: int = 0
    top: int = 0

    @staticmethod
    def from_json(d: dict, where: str) -> "SebavikMlpConfig":
        kind = _get(d, "kind", where)
        if kind == "dense":
            limit = float(_get(d, "limit", where))
            if not limit > 0:
                raise ConfigError(f"config.json: {where}.limit must be positive, got {limit!r}")
            return SebavikMlpConfig("dense", _positive_int(_get(d, "ff", where), where + ".ff"), limit)
        if kind == "moe":
            router = _get(d, "router", where)
            experts = _positive_int(_get(router, "experts", where + ".router"), where + ".router.experts")
            top = _positive_int(_get(router, "top", where + ".router"), where + ".router.top")
            if top > experts:
                raise ConfigError(f"config.json: {where}: {top} choices among {experts} experts")
            ff = _positive_int(_get(_get(d, "expert", where), "ff", where + ".expert"), where + ".expert.ff")
            return SebavikMlpConfig("moe", ff, None, experts, top)
        raise ConfigError(f"config.json: {where}.kind = {kind!r} is not supported (supported: {', '.join(MLP_KINDS)})")

    def to_json(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense", "limit": self.limit}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class SebavikLayerConfig:
    mixer: SebavikMixerConfig
    mlp: Optional[SebavikMlpConfig] = None


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class SebavikConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    embedding_scale: float
    layers: Tuple[SebavikLayerConfig, ...]
    bigram: Optional[BigramConfig] = None
    canon_taps: int = 0          # 0: sublayers read their normed input as it is
    side_dim: int = 0            # 0: no per-layer token input
    architectures: tuple = ("Sebavik",)
    eos_token_id: int = -1

    architecture_name = "Sebavik"

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if not self.eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.eps!r}")
        if not self.layers:
            raise ConfigError("config.json: no layers")
        mixing = [l.mixer for l in self.layers if l.mixer.v_mix]
        for m in mixing[1:]:
            if (m.kv_heads, m.vdim) != (mixing[0].kv_heads, mixing[0].vdim):
                raise ConfigError("config.json: layers that mix their values with the first such layer's must have "
                                  "its key/value heads and value size")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_json(d: dict) -> "SebavikConfig":
        layers = []
        for i, entry in enumerate(_get(d, "layers", "the model")):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where} has the unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            mixer = SebavikMixerConfig.from_json(_get(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            layers.append(SebavikLayerConfig(mixer, SebavikMlpConfig.from_json(mlp, where + ".mlp") if mlp else None))
        emb = d.get("embedding") or {}
        bigram = None
        if emb.get("bigram"):
            b = emb["bigram"]
            bigram = BigramConfig(_positive_int(_get(b, "buckets", "embedding.bigram"), "embedding.bigram.buckets"),
                                  _count(_get(b, "mul_prev", "embedding.bigram"), "embedding.bigram.mul_prev"),
                                  _count(_get(b, "mul_cur", "embedding.bigram"), "embedding.bigram.mul_cur"))
        canon = d.get("canon") or {}
        side = d.get("token_side") or {}
        eos = d.get("eos_token_id", -1)
        return SebavikConfig(vocab=_get(d, "vocab", "the model"), width=_get(d, "width", "the model"),
                             eps=float(_get(_get(d, "norm", "the model"), "eps", "norm")),
                             residual_mult=float(d.get("residual_mult", 1.0)), embedding_scale=float(emb.get("scale", 1.0)),
                             layers=tuple(layers), bigram=bigram,
                             canon_taps=_count(canon.get("taps", 0) or 0, "canon.taps"),
                             side_dim=_count(side.get("dim", 0) or 0, "token_side.dim"),
                             eos_token_id=-1 if eos is None else int(eos))

    def to_json(self) -> dict:
        emb = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram.buckets, "mul_cur": self.bigram.mul_cur, "mul_prev": self.bigram.mul_prev}
        d = {"architecture": "Sebavik", "embedding": emb,
             "layers": [{"mixer": l.mixer.to_json(), "mlp": l.mlp.to_json() if l.mlp else None, "type": "attention"}
                        for l in self.layers],
             "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d
