"""Typed configuration of the Kezuvik design, read from config.json.

Keys: ``architecture`` ("Kezuvik"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (the factor on
what a sublayer adds to the stream), ``logit_softcap`` and ``layers``, a list with one entry per layer:
``type``, ``mixer`` and ``mlp`` (null for none, else ``kind`` "dense" with ``ff``).  A mixer's keys by type:

* ``latent_attention`` and ``latent_attention_2``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``,
  ``q_rank``, ``scale``, ``rot.base``, ``rot.dims`` and optionally ``rot.scaling`` (``factor``, ``original``,
  ``fast``, ``slow``).  The second kind has a sink per head in its softmax and one gate number per head;
  the first an ordinary softmax and one gate number per entry of the heads' outputs;
* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, and optionally ``conv`` (taps of
  the short convolution on q, k and v) and ``mask.size`` (the window).

Every size and constant of a model comes from here or from a tensor's shape.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError

MIXER_TYPES = ("latent_attention", "latent_attention_2", "attention")


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def _positive(v, what: str) -> float:
    try:
        f = float(v)
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: {what} must be a number, got {v!r}") from None
    if not f > 0:
        raise ConfigError(f"config.json: {what} must be positive, got {v!r}")
    return f


@dataclass(frozen=True)
class RotScalingConfig:
    factor: float
    original: float
    fast: float
    slow: float

    @staticmethod
    def from_json(d: dict, where: str) -> "RotScalingConfig":
        return RotScalingConfig(*(_positive(_get(d, k, where), f"{where}.{k}") for k in ("factor", "original", "fast", "slow")))

    def to_json(self) -> dict:
        return {"factor": self.factor, "fast": self.fast, "original": self.original, "slow": self.slow}


@dataclass(frozen=True)
class KezuvikMixerConfig:
    kind: str                          # one of MIXER_TYPES
    heads: int
    dim: int                           # query/key size per head (the latent kinds: the part that is not rotated)
    vdim: int
    scale: float
    # the latent kinds
    rot_dim: Optional[int] = None      # rotated query/key size per head (the key part is shared by the heads)
    kv_rank: Optional[int] = None
    q_rank: Optional[int] = None
    rot_base: Optional[float] = None
    rot_dims: Optional[int] = None     # how many of the rot_dim entries turn
    rot_scaling: Optional[RotScalingConfig] = None
    # attention
    kv_heads: Optional[int] = None
    conv: Optional[int] = None         # taps of the short convolution on q, k and v
    window: Optional[int] = None

    @property
    def latent(self) -> bool:
        return self.kind != "attention"

    @staticmethod
    def from_json(kind: str, d: dict, where: str) -> "KezuvikMixerConfig":
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where} has the unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
        common = dict(kind=kind, heads=_positive_int(_get(d, "heads", where), where + ".heads"),
                      dim=_positive_int(_get(d, "dim", where), where + ".dim"),
                      vdim=_positive_int(_get(d, "vdim", where), where + ".vdim"),
                      scale=float(_get(d, "scale", where)))
        if kind == "attention":
            mask = d.get("mask")
            c = KezuvikMixerConfig(
                **common, kv_heads=_positive_int(d.get("kv_heads", common["heads"]), where + ".kv_heads"),
                conv=_positive_int(d["conv"], where + ".conv") if d.get("conv") is not None else None,
                window=_positive_int(_get(mask, "size", where + ".mask"), where + ".mask.size") if mask else None)
            if c.heads % c.kv_heads:
                raise ConfigError(f"config.json: {where}: {c.heads} heads are not a multiple of {c.kv_heads} key/value heads")
            return c
        rot = _get(d, "rot", where)
        rot_dim = _positive_int(_get(d, "rot_dim", where), where + ".rot_dim")
        scaling = rot.get("scaling")
        c = KezuvikMixerConfig(
            **common, rot_dim=rot_dim, kv_rank=_positive_int(_get(d, "kv_rank", where), where + ".kv_rank"),
            q_rank=_positive_int(_get(d, "q_rank", where), where + ".q_rank"),
            rot_base=_positive(_get(rot, "base", where + ".rot"), where + ".rot.base"),
            rot_dims=_positive_int(rot.get("dims", rot_dim), where + ".rot.dims"),
            rot_scaling=RotScalingConfig.from_json(scaling, where + ".rot.scaling") if scaling else None)
        if c.rot_dims > c.rot_dim or c.rot_dims % 2:
            raise ConfigError(f"config.json: {where}.rot.dims = {c.rot_dims} must be even and at most rot_dim = {c.rot_dim}")
        return c

    def to_json(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "scale": self.scale, "vdim": self.vdim}
        if self.kind == "attention":
            d["kv_heads"] = self.kv_heads
            if self.conv is not None:
                d["conv"] = self.conv
            if self.window is not None:
                d["mask"] = {"size": self.window}
            return d
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = self.rot_scaling.to_json()
        d.update({"kv_rank": self.kv_rank, "q_rank": self.q_rank, "rot": rot, "rot_dim": self.rot_dim})
        return d


@dataclass(frozen=True)
class KezuvikLayerConfig:
    mixer: KezuvikMixerConfig
    ff: Optional[int]  # inner size of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class KezuvikConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[KezuvikLayerConfig, ...]
    residual_mult: float = 1.0
    logit_softcap: Optional[float] = None
    architectures: tuple = ("Kezuvik",)
    eos_token_id: int = -1

    architecture_name = "Kezuvik"

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if not self.eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.eps!r}")
        if not self.layers:
            raise ConfigError("config.json: no layers")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError(f"config.json: logit_softcap must be positive, got {self.logit_softcap!r}")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_json(d: dict) -> "KezuvikConfig":
        layers = []
        for i, entry in enumerate(_get(d, "layers", "the model")):
            where = f"layers[{i}]"
            mixer = KezuvikMixerConfig.from_json(_get(entry, "type", where), _get(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            ff = None
            if mlp:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind = {mlp.get('kind')!r} is not supported (supported: 'dense')")
                ff = _positive_int(_get(mlp, "ff", where + ".mlp"), where + ".mlp.ff")
            layers.append(KezuvikLayerConfig(mixer, ff))
        eos = d.get("eos_token_id", -1)
        cap = d.get("logit_softcap")
        return KezuvikConfig(vocab=_get(d, "vocab", "the model"), width=_get(d, "width", "the model"),
                             eps=float(_get(_get(d, "norm", "the model"), "eps", "norm")), layers=tuple(layers),
                             residual_mult=float(d.get("residual_mult", 1.0)),
                             logit_softcap=float(cap) if cap is not None else None,
                             eos_token_id=-1 if eos is None else int(eos))

    def to_json(self) -> dict:
        d = {"architecture": "Kezuvik",
             "layers": [{"mixer": l.mixer.to_json(), "mlp": {"ff": l.ff, "kind": "dense"} if l.ff else None,
                         "type": l.mixer.kind} for l in self.layers],
             "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d
